// Tensor-core (tcgen05 / TMEM / TMA) family for the selected-block branch.
//
// The computation is organised KV-block-stationary.  An integer pre-pass turns
// the per-query selection (idx, mask) into, for every (batch, KV head, KV
// block j), the list of queries that attend block j -- the selected slots and,
// for the own block, its 64 queries.  A list is cut into chunks of 128/G
// queries; with the G query heads of the group that makes a dense 128-row
// tile.  A persistent CTA takes an item (one list, up to kChunksPerItem
// chunks), brings the K and V tiles of block j into shared memory once with
// TMA, and for every chunk gathers the 128 query rows and runs dense tcgen05
// MMAs against the resident tiles:
//
//   forward : S = Q K^T -> per-row softmax of that block -> O_part = P V.
//             Every (row, slot) writes its partial output (sum of p v, bf16)
//             and its (max, sum); a second kernel merges the partials of a row
//             into the output and the log-sum-exp.
//   backward: S = Q K^T and dP = dO V^T -> P = exp(S - lse), dS = P (dP - delta)
//             -> dV += P^T dO and dK += dS^T Q stay in tensor memory across the
//             chunks of the item (flushed once with fp32 reductions), and
//             dQ_chunk = dS K goes out as a bf16 partial per (row, slot) that a
//             last kernel sums into dq.
//
// All operand tiles are [rows x 64 columns] bf16 with 128-byte rows and the
// 128-byte swizzle, which serves both as a K-major and as an MN-major operand.
// Every wait on an mbarrier is bounded; a wait that runs out raises a status
// word in the work buffer instead of hanging, and the CTA still frees its
// tensor memory.

#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nsa_common.cuh"
#include "nsa_kernels.h"
#include "nsa_sm100_ptx.cuh"

namespace nsa {

using namespace ptx;

constexpr int kBlock = 64;           // keys per selection block served by this family
constexpr int kRows = 128;           // rows of a chunk tile (queries x heads of the group)
constexpr int kChunksPerItem = 16;   // chunks a CTA processes per resident K/V tile
constexpr uint32_t kInvalidEntry = 0xffffffffu;

// Which keys a query attends.  The three NSA branches differ only in this rule; everything after the index pre-pass
// (lists of (query, slot) per key block, dense 128-row chunks) is shared.
//   kModeSel : the blocks named by idx/mask plus the own block as `diag` says         (slot = position in idx; own = nsel)
//   kModeSwa : causal window, keys i-window..i                                         (slot = own block - key block)
//   kModeCmp : compressed keys, rows 0 .. num_mem + i/stride - 1 of a [num_mem + ncb]-row key tensor (slot = key block)
enum { kModeSel = 0, kModeSwa = 1, kModeCmp = 2 };

struct BlockRule {
  const int64_t* idx;
  const uint8_t* mask;
  int N;        // queries
  int nkb;      // key blocks of 64 rows
  int nsel;     // slots in idx (kModeSel)
  int ns;       // slots a query can have: the partial results of a query are indexed 0..ns-1
  int diag, mode, window, stride, num_mem;
};

// Slot s of query i (selection head bh): does it exist, and which key block is it?
template <int MODE>
__device__ __forceinline__ bool slot_block(const BlockRule& R, int bh, int i, int s, int* blk) {
  if (MODE == kModeSel) {
    if (s == R.nsel) {
      *blk = i / 64;
      return R.diag != NSA_DIAG_NONE;
    }
    const int64_t at = ((int64_t)bh * R.N + i) * R.nsel + s;
    const int64_t b = R.idx[at];
    *blk = (int)b;
    return R.mask[at] != 0 && b >= 0 && b < R.nkb;
  }
  if (MODE == kModeSwa) {
    *blk = i / 64 - s;
    return *blk >= 0 && *blk * 64 + 63 >= i - R.window;
  }
  *blk = s;
  return s * 64 < R.num_mem + i / R.stride;
}

struct SelPlan {
  int nqb, nkb, ns, G, QT, nlists;
  int64_t entries_cap, items_cap;
  // byte offsets into the work buffer
  int64_t off_status, off_num_items, off_counts, off_totals, off_list_base, off_items, off_entries;
  int64_t off_partial, off_stats, off_delta;
  int64_t index_bytes;   // the leading part that holds the index (what the backward can take from the forward)
  int64_t total_bytes;
};

struct SelParams {
  const __nv_bfloat16 *q, *dout;
  __nv_bfloat16* out;
  int64_t q_sb, q_sh, q_sn, do_sb, do_sh, do_sn, o_sb, o_sh, o_sn;
  const int64_t* idx;
  const uint8_t* mask;
  const uint32_t* entries;
  const int4* items;
  const int* num_items;    // [0] items, [1] the tag the item kernel left
  __nv_bfloat16* dq_lp;    // optional bf16 dq with its own batch / head / row strides (dq merge)
  int64_t dq_sb, dq_sh, dq_sn;
  uint32_t index_tag;
  __nv_bfloat16* partial;
  float2* stats;
  float* lse;
  const float* delta;
  float *dq, *dk, *dv, *slot_grads;
  int* status;
  int B, Hq, Hkv, N, Nk, G, nsel, nfb, diag;   // nfb = key blocks (lists per head); N queries, Nk key rows
  int ns;                                       // slots per query in the partial buffers
  float scale, scale_log2;
  BlockRule rule;
  // compressed branch only: the head-averaged logits of every compressed block column, [B, Hkv, N, ncb] fp32
  float* importance;
  int ncb, round_bf16;
  // or, instead of it, those logits averaged over runs of `cpf` columns (one value per selection block of
  // pool_block = cpf * stride queries) and rounded to bf16: [B, Hkv, N, pool_cols], written for the blocks that lie
  // wholly before the query's own block
  __nv_bfloat16* pooled;
  int cpf, pool_cols, pool_block;
};

// Number of items of the index, or 0 (and status 2) when the index was not built for these sizes: a caller-kept
// index that belongs to another problem, or a buffer nobody filled, must not steer any address.
__device__ __forceinline__ int item_count(const SelParams& P) {
  if ((uint32_t)P.num_items[1] != P.index_tag) {
    if (threadIdx.x == 0) atomicExch(P.status, 2);
    return 0;
  }
  return P.num_items[0];
}

// ---- index pre-pass --------------------------------------------------------------

// counts[(bh*nqb + qb)*nkb + j] = entries that the queries of block qb contribute to list (bh, j)
template <int MODE>
__global__ void __launch_bounds__(kBlock) sel_hist_kernel(const BlockRule R, int* counts) {
  extern __shared__ int hist[];
  const int qb = blockIdx.x, nqb = gridDim.x, bh = blockIdx.y * gridDim.z + blockIdx.z;  // bh = b*Hkv + h
  for (int j = threadIdx.x; j < R.nkb; j += kBlock) hist[j] = 0;
  __syncthreads();
  const int i = qb * kBlock + threadIdx.x;
  if (i < R.N) {
    for (int s = 0; s < R.ns; ++s) {
      int blk;
      if (slot_block<MODE>(R, bh, i, s, &blk)) atomicAdd(&hist[blk], 1);
    }
  }
  __syncthreads();
  int* row = counts + ((int64_t)bh * nqb + qb) * R.nkb;
  for (int j = threadIdx.x; j < R.nkb; j += kBlock) row[j] = hist[j];
}

// per list: exclusive prefix over the contributing query blocks, and the list total.  A block handles 32
// neighbouring lists (threadIdx.x, so that loads stay coalesced) with kScanSeg threads each (threadIdx.y): every
// thread sums its segment of query blocks, the segments' sums are prefixed through shared memory, and a second pass
// over the segment writes the prefixes.
constexpr int kScanSeg = 8;
__global__ void __launch_bounds__(32 * kScanSeg) sel_scan_kernel(int* counts, int* totals, int nlists, int nqb, int nkb) {
  __shared__ int seg_sum[kScanSeg][32];
  const int l = blockIdx.x * 32 + threadIdx.x, seg = threadIdx.y;
  const bool live = l < nlists;
  const int bh = live ? l / nkb : 0, j = live ? l - bh * nkb : 0;
  const int per = (nqb + kScanSeg - 1) / kScanSeg;
  const int q0 = min(nqb, seg * per), q1 = min(nqb, q0 + per);
  int* base = counts + (int64_t)bh * nqb * nkb + j;
  int sum = 0;
  if (live)
    for (int qb = q0; qb < q1; ++qb) sum += base[(int64_t)qb * nkb];
  seg_sum[seg][threadIdx.x] = sum;
  __syncthreads();
  int running = 0;
  for (int k = 0; k < seg; ++k) running += seg_sum[k][threadIdx.x];
  if (live) {
    for (int qb = q0; qb < q1; ++qb) {
      int* c = base + (int64_t)qb * nkb;
      const int v = *c;
      *c = running;
      running += v;
    }
    if (seg == kScanSeg - 1) totals[l] = running;
  }
}

// list bases (padded to whole chunks) and the item table; one CTA of 1024 threads
__global__ void __launch_bounds__(1024) sel_items_kernel(const int* totals, int* list_base, int4* items, int* num_items,
                                                         int nlists, int QT, uint32_t tag) {
  __shared__ int s_pad[1024], s_it[1024];
  __shared__ int carry_pad, carry_it;
  if (threadIdx.x == 0) carry_pad = carry_it = 0;
  __syncthreads();
  for (int t0 = 0; t0 < nlists; t0 += 1024) {
    const int l = t0 + threadIdx.x;
    const int cnt = l < nlists ? totals[l] : 0;
    const int nch = (cnt + QT - 1) / QT;
    const int nit = (nch + kChunksPerItem - 1) / kChunksPerItem;
    s_pad[threadIdx.x] = nch * QT;
    s_it[threadIdx.x] = nit;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      int a = 0, b = 0;
      if ((int)threadIdx.x >= o) { a = s_pad[threadIdx.x - o]; b = s_it[threadIdx.x - o]; }
      __syncthreads();
      s_pad[threadIdx.x] += a;
      s_it[threadIdx.x] += b;
      __syncthreads();
    }
    const int base = carry_pad + s_pad[threadIdx.x] - nch * QT;  // exclusive
    const int ibase = carry_it + s_it[threadIdx.x] - nit;
    if (l < nlists) {
      list_base[l] = base;
      for (int k = 0; k < nit; ++k) {
        const int c0 = k * kChunksPerItem;
        items[ibase + k] = make_int4(l, c0, min(kChunksPerItem, nch - c0), base + c0 * QT);
      }
    }
    __syncthreads();
    if (threadIdx.x == 1023) { carry_pad += s_pad[1023]; carry_it += s_it[1023]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    num_items[0] = carry_it;
    num_items[1] = (int)tag;   // marks the index as built, and for which sizes
  }
}

// writes the entries (query | slot << 24) in a fixed order: by query block, then slot, then query
template <int MODE>
__global__ void __launch_bounds__(kBlock) sel_fill_kernel(const BlockRule R, const int* counts, const int* list_base,
                                                          uint32_t* entries) {
  extern __shared__ int cursor[];
  const int qb = blockIdx.x, nqb = gridDim.x, bh = blockIdx.y * gridDim.z + blockIdx.z;
  const int* row = counts + ((int64_t)bh * nqb + qb) * R.nkb;
  for (int j = threadIdx.x; j < R.nkb; j += kBlock) cursor[j] = list_base[bh * R.nkb + j] + row[j];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = qb * kBlock + threadIdx.x;
  for (int s = 0; s < R.ns; ++s) {
    int blk = 0;
    const bool valid = i < R.N && slot_block<MODE>(R, bh, i, s, &blk);
    for (int w = 0; w < 2; ++w) {
      if (warp == w) {
        const unsigned vm = __ballot_sync(kFullMask, valid);
        if (valid) {
          const unsigned peers = __match_any_sync(vm, blk);
          const int rank = __popc(peers & ((1u << lane) - 1u));
          const int leader = __ffs(peers) - 1;
          int pos = 0;
          if (lane == leader) {
            pos = cursor[blk];
            cursor[blk] = pos + __popc(peers);
          }
          pos = __shfl_sync(peers, pos, leader);
          entries[pos + rank] = (uint32_t)i | ((uint32_t)s << 24);
        }
      }
      __syncthreads();
    }
  }
}

// ---- shared pieces of the two main kernels -----------------------------------------

struct RowInfo {
  int i, slot;
  int lo, lim;   // first and last visible key column of the block (lim = -1: the row is padding)
  bool valid;
};

__device__ __forceinline__ RowInfo decode_row(uint32_t e, int j, const BlockRule& R) {
  RowInfo r;
  r.valid = e != kInvalidEntry;
  r.i = (int)(e & 0xffffffu);
  r.slot = (int)(e >> 24);
  r.lo = 0;
  r.lim = kBlock - 1;
  if (R.mode == kModeSel) {
    if (r.slot == R.nsel && R.diag == NSA_DIAG_CAUSAL) r.lim = r.i - j * kBlock;
  } else if (R.mode == kModeSwa) {
    r.lim = min(kBlock - 1, r.i - j * kBlock);
    r.lo = max(0, r.i - R.window - j * kBlock);
  } else {
    r.lim = min(kBlock - 1, R.num_mem + r.i / R.stride - 1 - j * kBlock);
  }
  if (!r.valid) r.lim = -1;
  return r;
}

// All 128 threads copy the 128 rows of a chunk (D bf16 each) from global memory into swizzled [128 x 128 B]
// tiles, one tile per 64 columns.  D/8 neighbouring threads share a row, so a warp reads whole 128-byte lines.
// `base` points at batch element b; row r of the tile is query entries[r / G], head h*G + r % G.
template <int D>
__device__ __forceinline__ void gather_tile(uint32_t tile, const __nv_bfloat16* base, int64_t stride_h, int64_t stride_n,
                                            const uint32_t* entries, int g_shift, int h, int tid) {
  constexpr int CH = D / 8;         // 16-byte pieces per row
  constexpr int RPP = kRows / CH;   // rows covered by one pass of the 128 threads
  const int sub = tid % CH, r0 = tid / CH;
  uint4 v[CH];
#pragma unroll
  for (int it = 0; it < CH; ++it) {
    const int row = r0 + it * RPP;
    const int ql = row >> g_shift, g = row - (ql << g_shift);
    const uint32_t e = __ldg(entries + ql);
    v[it] = make_uint4(0u, 0u, 0u, 0u);
    if (e != kInvalidEntry)
      v[it] = ldg_nc_v4(base + (int64_t)((h << g_shift) + g) * stride_h + (int64_t)(e & 0xffffffu) * stride_n + sub * 8);
  }
#pragma unroll
  for (int it = 0; it < CH; ++it) {
    const int row = r0 + it * RPP;
    sts_v4(tile + (sub / 8) * (kRows * 128) + sw128_offset(row, sub % 8), v[it]);
  }
}

// The same gather with 16-byte cp.async: returns at once, the rows land later (cp_async_wait).  Padding rows are
// zero-filled.
template <int D>
__device__ __forceinline__ void gather_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride_h,
                                                  int64_t stride_n, const uint32_t* entries, int g_shift, int h,
                                                  int tid) {
  constexpr int CH = D / 8;
  constexpr int RPP = kRows / CH;
  const int sub = tid % CH, r0 = tid / CH;
  uint32_t ev[CH];
#pragma unroll
  for (int it = 0; it < CH; ++it) ev[it] = __ldg(entries + ((r0 + it * RPP) >> g_shift));
#pragma unroll
  for (int it = 0; it < CH; ++it) {
    const int row = r0 + it * RPP;
    const int g = row & ((1 << g_shift) - 1);
    const bool valid = ev[it] != kInvalidEntry;
    const int64_t i = valid ? (int64_t)(ev[it] & 0xffffffu) : 0;
    cp_async16(tile + (sub / 8) * (kRows * 128) + sw128_offset(row, sub % 8),
               base + (int64_t)((h << g_shift) + g) * stride_h + i * stride_n + sub * 8, valid ? 16u : 0u);
  }
}

__device__ __forceinline__ void store_row_bf16(uint32_t tile, int row, const float (&x)[64]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v;
    v.x = pack_bf16(x[c * 8 + 0], x[c * 8 + 1]);
    v.y = pack_bf16(x[c * 8 + 2], x[c * 8 + 3]);
    v.z = pack_bf16(x[c * 8 + 4], x[c * 8 + 5]);
    v.w = pack_bf16(x[c * 8 + 6], x[c * 8 + 7]);
    sts_v4(tile + sw128_offset(row, c), v);
  }
}


// Ships the 128 rows of a staging area (ROW_BYTES each, padded to `stride`) to scattered global rows.  Row r goes to
// gbase + dst[r] * ROW_BYTES (skipped when dst[r] < 0); ROW_BYTES/16 neighbouring threads share a row, so every
// store instruction writes whole 128-byte lines.  `t` is the thread's index among the 128 callers, which must have
// synchronised after filling the staging area and dst[].  (One bulk copy per row would be simpler, but an SM issues
// only about one bulk copy per 20 cycles, which made that the slowest step of a chunk.)
template <int ROW_BYTES>
__device__ __forceinline__ void store_rows_coalesced(uint32_t stage, uint32_t stride, const int* dst,
                                                     uint8_t* gbase, int t) {
  constexpr int TPR = ROW_BYTES / 16;
  constexpr int RPP = kRows / TPR;
  const int sub = t % TPR, r0 = t / TPR;
  uint4 v[TPR];
  int d[TPR];
#pragma unroll
  for (int k = 0; k < TPR; ++k) {
    const int row = r0 + k * RPP;
    d[k] = dst[row];
    v[k] = lds_v4(stage + row * stride + sub * 16);
  }
#pragma unroll
  for (int k = 0; k < TPR; ++k)
    if (d[k] >= 0) *reinterpret_cast<uint4*>(gbase + (int64_t)d[k] * ROW_BYTES + sub * 16) = v[k];
}

// ---- forward -------------------------------------------------------------------------

// Forward of the selected-block branch.  A CTA of 256 threads walks gather -> S -> softmax -> P V -> store chunk by
// chunk; several CTAs share an SM (4 at dim_head 64) and fill each other's waits.  Two threads share a row (32 of the
// block's 64 columns each; they exchange maximum and sum through shared memory), which halves the serial work per
// thread and, above all, doubles the number of warps that issue the gather: a warp gets only about 1.3 bytes per
// clock of scattered 128-byte rows out of the L2 however many copies it has in flight (measured: 5.5 B/clk per SM
// with 4 warps copying, 17 with 16, 26 with 32), and the gather of the Q rows is what bounds this kernel.
template <int D>
__device__ __forceinline__ void gather_tile_async2(uint32_t tile, const __nv_bfloat16* base, int64_t stride_h,
                                                   int64_t stride_n, const uint32_t* entries, int g_shift, int h,
                                                   int tid) {
  constexpr int CH = D / 8;               // 16-byte pieces per row
  constexpr int RPP = 2 * kRows / CH;     // rows covered by one pass of the 256 threads
  const int sub = tid % CH, r0 = tid / CH;
  uint32_t ev[kRows / RPP];
#pragma unroll
  for (int it = 0; it < kRows / RPP; ++it) ev[it] = __ldg(entries + ((r0 + it * RPP) >> g_shift));
#pragma unroll
  for (int it = 0; it < kRows / RPP; ++it) {
    const int row = r0 + it * RPP;
    const int g = row & ((1 << g_shift) - 1);
    const bool valid = ev[it] != kInvalidEntry;
    const int64_t i = valid ? (int64_t)(ev[it] & 0xffffffu) : 0;
    cp_async16(tile + (sub / 8) * (kRows * 128) + sw128_offset(row, sub % 8),
               base + (int64_t)((h << g_shift) + g) * stride_h + i * stride_n + sub * 8, valid ? 16u : 0u);
  }
}

template <int D>
__global__ void __launch_bounds__(2 * kRows, D == 64 ? 4 : 2)
sel_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelParams P) {
  constexpr int NC = D / 64;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ int row_dst[kRows];
  __shared__ float xmax[2][kRows], xsum[2][kRows];
  const int nitems = item_count(P);
  if ((int)blockIdx.x >= nitems) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = sQ + NC * 16384, sV = sK + NC * 8192, sStage = sV + NC * 8192;
  constexpr uint32_t kStageStride = D * 2 + 16;   // one padded partial-output row per row of the chunk
  const uint32_t bar_kv = smem_u32(&bars[0]), bar_s = smem_u32(&bars[1]), bar_o = smem_u32(&bars[2]);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int half = tid >> 7, row = tid & (kRows - 1);   // this thread: columns 32*half .. 32*half+31 of row `row`
  constexpr uint32_t kCols = D == 64 ? 128 : 256;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_slot;
  const uint32_t tm_lane = tm + ((uint32_t)((warp & 3) * 32) << 16);   // warps w and w + 4 share a lane quarter
  const uint32_t tS = 0, tO = 64;

  const int G = P.G, QT = kRows / G, g_shift = 31 - __clz(G);
  const int q_local = row >> g_shift, g = row - (q_local << g_shift);
  uint32_t ph_kv = 0, ph_s = 0, ph_o = 0;
  constexpr uint32_t idS = instr_desc_bf16(128, 64, false, false);
  constexpr uint32_t idO = instr_desc_bf16(128, D, false, true);

  for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
    const int4 item = P.items[it];
    const int list = item.x, j = list % P.nfb, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * NC * 8192);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        tma_load_4d(sK + c * 8192, &tmK, bar_kv, c * 64, j * kBlock, h, b);
        tma_load_4d(sV + c * 8192, &tmV, bar_kv, c * 64, j * kBlock, h, b);
      }
    }
    bool prefetched = false;
    for (int c = 0; c < item.z; ++c) {
      const uint32_t* chunk_entries = P.entries + item.w + c * QT;
      const uint32_t e = chunk_entries[q_local];
      if (!prefetched) gather_tile_async2<D>(sQ, P.q + b * P.q_sb, P.q_sh, P.q_sn, chunk_entries, g_shift, h, tid);
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncthreads();
      if (warp == 0) {   // the whole warp runs the issue code, one elected lane issues
        if (c == 0) {
          mbar_wait_bounded(bar_kv, ph_kv, &abort_flag);
          __syncwarp();
        }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ch = k / 4, in = (k % 4) * 32;
          mma_bf16_elect(tm + tS, smem_desc_sw128(sQ + ch * 16384 + in, 16), smem_desc_sw128(sK + ch * 8192 + in, 16),
                         idS, k > 0);
        }
        mma_commit_elect(bar_s);
      }
      __syncwarp();
      mbar_wait_warp(bar_s, ph_s, &abort_flag);
      ph_s ^= 1;
      tc_fence_after_sync();
      // S is complete, so the Q tile is free: request the next chunk's rows now; they travel while this chunk's
      // softmax, second MMA and output run
      prefetched = c + 1 < item.z;
      if (prefetched)
        gather_tile_async2<D>(sQ, P.q + b * P.q_sb, P.q_sh, P.q_sn, chunk_entries + QT, g_shift, h, tid);
      __syncwarp();
      const RowInfo r = decode_row(e, j, P.rule);
      const int lim = r.lim - half * 32;   // last visible column of this thread's half (negative: none)
      float s[32];
      tmem_ld32(tm_lane + tS + half * 32, s);
      tmem_ld_wait();
      const bool all_full = __all_sync(kFullMask, lim >= 31);
      float mm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (all_full) {
#pragma unroll
        for (int x = 0; x < 32; ++x) mm[x & 3] = fmaxf(mm[x & 3], s[x]);
      } else {
#pragma unroll
        for (int x = 0; x < 32; ++x) mm[x & 3] = x <= lim ? fmaxf(mm[x & 3], s[x]) : mm[x & 3];
      }
      float m = fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3]));
      xmax[half][row] = m;
      __syncthreads();
      m = fmaxf(m, xmax[half ^ 1][row]);
      const float m2 = r.valid ? m * P.scale_log2 : 0.f;
      float ll[4] = {0.f, 0.f, 0.f, 0.f};
      if (all_full) {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          s[x] = ex2(fmaf(s[x], P.scale_log2, -m2));
          ll[x & 3] += s[x];   // the fp32 sum: the log-sum-exp stays exact although P is rounded to bf16 for the MMA
        }
      } else {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          s[x] = x <= lim ? ex2(fmaf(s[x], P.scale_log2, -m2)) : 0.f;
          ll[x & 3] += s[x];
        }
      }
      xsum[half][row] = (ll[0] + ll[1]) + (ll[2] + ll[3]);
      // P goes to the tensor cores through tensor memory, over the first half of this row's S columns (both threads
      // of the row have read their S columns: the exchange of the maxima lies in between)
      tmem_st_bf16_row32(tm_lane + tS + half * 16, s);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncthreads();
      if (warp == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_bf16_tmem_a_elect(tm + tO, tm + tS + k * 8, smem_desc_sw128(sV + k * 2048, 8192), idO, k > 0);
        mma_commit_elect(bar_o);
      }
      const float l = xsum[0][row] + xsum[1][row];
      const int64_t hq = (int64_t)h * G + g;
      const int64_t row_global = ((int64_t)b * P.Hq + hq) * P.N + r.i;
      const int64_t pslot = r.valid ? row_global * P.ns + r.slot : 0;
      __syncwarp();
      mbar_wait_warp(bar_o, ph_o, &abort_flag);
      ph_o ^= 1;
      tc_fence_after_sync();
      __syncwarp();
      // the partial row stays unnormalised (sum of p * v, at most 64 max|v|): the merge divides once per row
#pragma unroll
      for (int c2 = 0; c2 < D / 64; ++c2) {
        float t[32];
        tmem_ld32(tm_lane + tO + half * (D / 2) + c2 * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          uint4 v;
          v.x = pack_bf16(t[x * 8 + 0], t[x * 8 + 1]);
          v.y = pack_bf16(t[x * 8 + 2], t[x * 8 + 3]);
          v.z = pack_bf16(t[x * 8 + 4], t[x * 8 + 5]);
          v.w = pack_bf16(t[x * 8 + 6], t[x * 8 + 7]);
          sts_v4(sStage + row * kStageStride + half * D + c2 * 64 + x * 16, v);
        }
      }
      if (half == 0) row_dst[row] = r.valid ? (int)pslot : -1;
      tc_fence_before_sync();
      __syncthreads();
      {   // whole 128-byte lines per store instruction: D/8 neighbouring threads share a row
        constexpr int TPR = D / 8, RPP = 2 * kRows / TPR;
        const int sub = tid % TPR, r0 = tid / TPR;
        uint8_t* const pbase = reinterpret_cast<uint8_t*>(P.partial);
#pragma unroll
        for (int k = 0; k < kRows / RPP; ++k) {
          const int rr = r0 + k * RPP;
          const int dst = row_dst[rr];
          const uint4 v = lds_v4(sStage + rr * kStageStride + sub * 16);
          if (dst >= 0) *reinterpret_cast<uint4*>(pbase + (int64_t)dst * (D * 2) + sub * 16) = v;
        }
      }
      if (half == 0 && r.valid) P.stats[pslot] = make_float2(m2, l);
    }
    ph_kv ^= 1;
    __syncthreads();   // every thread is done with this item's tiles before the next TMA overwrites them
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kCols);
  if (tid == 0 && abort_flag) atomicExch(P.status, 1);
}

// merges the partial results of every (batch, query head, query): one group of D/8 threads per row.
// The statistics were cleared before the forward kernel ran, so a slot the query does not have reads (0, 0) and needs
// no look-up in the index; its partial row was never written and is not read.  Loads are issued eight slots at a time
// with nothing depending on them in between: the kernel is a stream over the partial buffer.
template <int D>
__global__ void __launch_bounds__(256) sel_merge_kernel(const SelParams P) {
  constexpr int TPR = D / 8;
  const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const int64_t nrows = (int64_t)P.B * P.Hq * P.N;
  if (row >= nrows) return;
  const int i = (int)(row % P.N);
  const int hq = (int)((row / P.N) % P.Hq);
  const int b = (int)(row / ((int64_t)P.N * P.Hq));
  const int ns = P.ns;
  const float2* st = P.stats + row * ns;
  const __nv_bfloat16* prow = P.partial + row * ns * D + part * 8;
  float M = -INFINITY;
#pragma unroll 4
  for (int s = 0; s < ns; ++s) {
    const float2 ml = st[s];
    if (ml.y > 0.f) M = fmaxf(M, ml.x);
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float L = 0.f;
  for (int s0 = 0; s0 < ns; s0 += 8) {
    float w[8];
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool in = s0 + u < ns;
      const float2 ml = in ? st[s0 + u] : make_float2(0.f, 0.f);
      const bool ok = ml.y > 0.f;
      w[u] = ok ? ex2(ml.x - M) : 0.f;
      L = fmaf(w[u], ml.y, L);
      v[u] = ok ? *reinterpret_cast<const uint4*>(prow + (int64_t)(s0 + u) * D) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        acc[2 * x] = fmaf(w[u], __uint_as_float(q[x] << 16), acc[2 * x]);
        acc[2 * x + 1] = fmaf(w[u], __uint_as_float(q[x] & 0xffff0000u), acc[2 * x + 1]);
      }
    }
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  uint4 o;
  o.x = pack_bf16(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  o.z = pack_bf16(acc[4] * inv, acc[5] * inv);
  o.w = pack_bf16(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(P.out + b * P.o_sb + (int64_t)hq * P.o_sh + (int64_t)i * P.o_sn + part * 8) = o;
  if (part == 0) P.lse[row] = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
}

// The merge of the selected branch that also does the gated combine and the head merge (and, with several
// destinations, the all-gather of the head-sharded layout): the merged selected row is rounded to bf16 as the tensor
// between the two kernels would be, combined with the compressed and the sliding row exactly as combine_gather_kernel
// does (the same three fused multiply-adds in the same order), and stored into every destination.  The selected
// branch's own output tensor is not written.  Thread groups walk the rows position-major (b, i, head), so that the
// heads of one position land next to each other in the destinations' [B, N, features] rows.
template <int D, bool MC>
__global__ void __launch_bounds__(256) sel_merge_combine_kernel(const SelParams P, const CombineParams Cp, const GatherTargets Gt) {
  constexpr int TPR = D / 8;
  const int64_t t = ((int64_t)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const int64_t nrows = (int64_t)P.B * P.Hq * P.N;
  if (t < nrows) {
    const int hq = (int)(t % P.Hq);
    const int i = (int)((t / P.Hq) % P.N);
    const int b = (int)(t / ((int64_t)P.N * P.Hq));
    const int64_t row = ((int64_t)b * P.Hq + hq) * P.N + i;
    const int ns = P.ns;
    const float2* st = P.stats + row * ns;
    const __nv_bfloat16* prow = P.partial + row * ns * D + part * 8;
    float M = -INFINITY;
#pragma unroll 4
    for (int s = 0; s < ns; ++s) {
      const float2 ml = st[s];
      if (ml.y > 0.f) M = fmaxf(M, ml.x);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float Lsum = 0.f;
    for (int s0 = 0; s0 < ns; s0 += 8) {
      float w[8];
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = s0 + u < ns;
        const float2 ml = in ? st[s0 + u] : make_float2(0.f, 0.f);
        const bool ok = ml.y > 0.f;
        w[u] = ok ? ex2(ml.x - M) : 0.f;
        Lsum = fmaf(w[u], ml.y, Lsum);
        v[u] = ok ? *reinterpret_cast<const uint4*>(prow + (int64_t)(s0 + u) * D) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          acc[2 * x] = fmaf(w[u], __uint_as_float(q[x] << 16), acc[2 * x]);
          acc[2 * x + 1] = fmaf(w[u], __uint_as_float(q[x] & 0xffff0000u), acc[2 * x + 1]);
        }
      }
    }
    const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
    if (part == 0 && P.lse != nullptr) P.lse[row] = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
    // combine: gates in the order compressed, selected, sliding
    const __nv_bfloat16* g = (const __nv_bfloat16*)Cp.gates + b * Cp.g_sb + hq * Cp.g_sh + (int64_t)i * Cp.g_sn;
    const float g0 = __bfloat162float(g[0]), g1 = __bfloat162float(g[1]), g2 = __bfloat162float(g[2]);
    const uint4 rc = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)Cp.o[0] + b * Cp.o_sb[0] + hq * Cp.o_sh[0] +
                                                     (int64_t)i * Cp.o_sn[0] + part * 8);
    const uint4 rw = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)Cp.o[2] + b * Cp.o_sb[2] + hq * Cp.o_sh[2] +
                                                     (int64_t)i * Cp.o_sn[2] + part * 8);
    const uint32_t qc[4] = {rc.x, rc.y, rc.z, rc.w}, qw[4] = {rw.x, rw.y, rw.z, rw.w};
    uint32_t packed[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      // the selected row as its bf16 tensor would hold it
      const uint32_t os = pack_bf16(acc[2 * x] * inv, acc[2 * x + 1] * inv);
      float lo = fmaf(g0, __uint_as_float(qc[x] << 16), 0.f);
      float hi = fmaf(g0, __uint_as_float(qc[x] & 0xffff0000u), 0.f);
      lo = fmaf(g1, __uint_as_float(os << 16), lo);
      hi = fmaf(g1, __uint_as_float(os & 0xffff0000u), hi);
      lo = fmaf(g2, __uint_as_float(qw[x] << 16), lo);
      hi = fmaf(g2, __uint_as_float(qw[x] & 0xffff0000u), hi);
      packed[x] = pack_bf16(lo, hi);
    }
    const int64_t at = ((int64_t)b * P.N + i) * Gt.total_features + Gt.feature_offset + (int64_t)hq * D + part * 8;
    if (MC) {
      asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"((__nv_bfloat16*)Gt.outs[0] + at),
                   "f"(__uint_as_float(packed[0])), "f"(__uint_as_float(packed[1])), "f"(__uint_as_float(packed[2])),
                   "f"(__uint_as_float(packed[3]))
                   : "memory");
    } else {
      const int rot = (int)(blockIdx.x % (unsigned)Gt.num_outs);
      for (int r = 0; r < Gt.num_outs; ++r) {
        int k = r + rot;
        if (k >= Gt.num_outs) k -= Gt.num_outs;
        *reinterpret_cast<uint4*>((__nv_bfloat16*)Gt.outs[k] + at) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
  }
  if (MC) __threadfence_system();
}

// ---- forward of the dense causal branches, query-tile stationary ---------------------------------------------
//
// The compressed and the sliding-window branch attend a contiguous range of key blocks per query, the same range for
// neighbouring queries.  For them the key-block-stationary form above pays for partial results it does not need: one
// CTA here owns a tile of 128/G consecutive queries (128 rows with the G heads of the group), walks the key blocks
// the tile can see and keeps the running maximum and sum of every row in registers and the output accumulator in
// tensor memory, as a flash-attention forward does.  No index, no partial results, no merge.
//   * Two threads share a row (32 of a block's 64 columns each; they exchange their maxima through shared memory),
//     so a CTA has eight warps to hide latencies with.
//   * S of block t+2 is issued as soon as P of block t has been handed to the PV MMA, so the tensor cores work on
//     PV(t) and S(t+2) while the threads do the softmax of block t+1 (two S buffers in tensor memory, two K and two V
//     buffers in shared memory, filled by TMA).
//   * The accumulator is rescaled lazily: a row keeps its reference maximum until a block exceeds it by more than 2^8;
//     only then is the O row read from tensor memory, scaled and written back (P stays below 2^8, exact in bf16's
//     range, and the sum is fp32).
//   * MODE compressed with IMP also writes the head-averaged logits of the visible columns (the importance), or with
//     POOL their per-selection-block means: the head means of the last 128 compressed columns of every query wait in
//     a ring in shared memory, and after every key block the threads average the selection blocks it completed.
template <int D, int MODE, int GI, bool POOL = false>   // GI: 0 = no importance output, else the heads per KV head
__global__ void __launch_bounds__(2 * kRows, 2)
dense_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelParams P) {
  constexpr int NC = D / 64;
  constexpr uint32_t kTileQ = NC * 16384, kTileKV = NC * 8192;
  constexpr uint32_t kStageStride = D * 2 + 16;
  constexpr uint32_t kCols = 256;
  constexpr int kThreads = 2 * kRows;   // two threads per row: each owns 32 of the 64 columns of a key block
  // The dynamic segment is declared 1024-byte aligned (the swizzled tiles need it) and holds exactly the tiles: with
  // dim_head 128 two CTAs then fill an SM's shared memory to the byte.
  extern __shared__ __align__(1024) uint8_t dense_smem[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bars[8];

  const uint32_t base = smem_u32(dense_smem);
  const uint32_t sQ = base, sX = sQ + kTileQ, sK0 = sX + 16384, sV0 = sK0 + 2 * kTileKV;
  // sX (16 KB): the two threads of a row exchange their partial maxima (and, at the end, sums) through it.  The Q tile
  // and sX become the staging area of the output rows at the end, followed by the rows' destinations.
  const uint32_t sStage = sQ;
  int* const row_dst = reinterpret_cast<int*>(dense_smem + kRows * kStageStride);
  float* const xchg = reinterpret_cast<float*>(dense_smem + kTileQ);   // [2 halves][kRows]
  // POOL: the head means of the last 128 logit columns of every query of the tile, [QT][kRing] bf16 (rows padded so
  // that neighbouring queries fall on different banks)
  constexpr int kRing = 128 + 32;
  __nv_bfloat16* const ring = reinterpret_cast<__nv_bfloat16*>(dense_smem + kTileQ + 1024);
  // barriers: K buffers full (2), V buffers full (2), S buffers complete (2), PV complete, drain
  const uint32_t bar0 = smem_u32(&bars[0]), bar_pv = bar0 + 48;
  auto bar_k = [&](int t) { return bar0 + (uint32_t)(t & 1) * 8; };
  auto bar_v = [&](int t) { return bar0 + 16 + (uint32_t)(t & 1) * 8; };
  auto bar_s = [&](int t) { return bar0 + 32 + (uint32_t)(t & 1) * 8; };
  const int tid = threadIdx.x, warp = tid >> 5;
  const int half = tid >> 7, row = tid & (kRows - 1);

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars[i]), 1);
    if (base & 1023u) abort_flag = 1;   // the tiles would be mis-swizzled: report instead of computing
    fence_mbar_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_slot;
  const uint32_t tm_lane = tm + ((uint32_t)((warp & 3) * 32) << 16);   // warps w and w + 4 share a lane quarter
  const uint32_t tO = 128;
  constexpr uint32_t idS = instr_desc_bf16(128, 64, false, false);
  constexpr uint32_t idO = instr_desc_bf16(128, D, false, true);

  // the tile: heavy tiles (late queries) are launched first
  constexpr bool IMP = GI > 0;
  const int G = IMP ? GI : P.G, QT = kRows / G, g_shift = 31 - __clz(G);
  const int tiles_per_head = (P.N + QT - 1) / QT;
  const int64_t tile = (int64_t)gridDim.x - 1 - blockIdx.x;
  const int qt = (int)(tile % tiles_per_head), bh = (int)(tile / tiles_per_head), h = bh % P.Hkv, b = bh / P.Hkv;
  const int i0 = qt * QT, i_last = min(i0 + QT - 1, P.N - 1);
  const int q_local = row >> g_shift, g = row - (q_local << g_shift);
  const int i = i0 + q_local;
  const bool valid = i < P.N;
  const int64_t hq = (int64_t)h * G + g;
  int jb, je;
  if (MODE == kModeCmp) {
    jb = 0;
    je = min(P.nfb, (P.rule.num_mem + i_last / P.rule.stride + kBlock - 1) / kBlock);
  } else {
    jb = max(0, i0 - P.rule.window) / kBlock;
    je = i_last / kBlock + 1;
  }
  const int nb = je - jb;

  // Q rows of the tile (zero rows past the end of the sequence) and the first K/V blocks
  {
    constexpr int CH = D / 8, RPP = kThreads / CH;
    const int sub = tid % CH, r0 = tid / CH;
    const __nv_bfloat16* qb = P.q + b * P.q_sb;
#pragma unroll
    for (int it = 0; it < kRows / RPP; ++it) {
      const int rr = r0 + it * RPP;
      const int qi = i0 + (rr >> g_shift), gg = rr & ((1 << g_shift) - 1);
      const bool ok = qi < P.N;
      cp_async16(sQ + (sub / 8) * (kRows * 128) + sw128_offset(rr, sub % 8),
                 qb + (int64_t)((h << g_shift) + gg) * P.q_sh + (int64_t)(ok ? qi : 0) * P.q_sn + sub * 8, ok ? 16u : 0u);
    }
    cp_async_commit();
  }
  auto load_k = [&](int t) {   // thread 0: key block jb + t into K buffer t & 1
    mbar_arrive_expect_tx(bar_k(t), kTileKV);
#pragma unroll
    for (int c = 0; c < NC; ++c) tma_load_4d(sK0 + (t & 1) * kTileKV + c * 8192, &tmK, bar_k(t), c * 64, (jb + t) * kBlock, h, b);
  };
  auto load_v = [&](int t) {
    mbar_arrive_expect_tx(bar_v(t), kTileKV);
#pragma unroll
    for (int c = 0; c < NC; ++c) tma_load_4d(sV0 + (t & 1) * kTileKV + c * 8192, &tmV, bar_v(t), c * 64, (jb + t) * kBlock, h, b);
  };
  auto issue_s = [&](int t) {   // warp 0, converged: S(t) = Q K(t)^T into S buffer t & 1
    mbar_wait_bounded(bar_k(t), (uint32_t)(t >> 1) & 1, &abort_flag);
    __syncwarp();
    tc_fence_after_sync();
    const uint32_t sK = sK0 + (t & 1) * kTileKV;
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
      const uint32_t ch = k / 4, in = (k % 4) * 32;
      mma_bf16_elect(tm + (t & 1) * 64, smem_desc_sw128(sQ + ch * 16384 + in, 16), smem_desc_sw128(sK + ch * 8192 + in, 16),
                     idS, k > 0);
    }
    mma_commit_elect(bar_s(t));
  };
  if (tid == 0) {
    load_k(0);
    load_v(0);
    if (nb > 1) load_k(1);
  }
  cp_async_wait<0>();
  fence_proxy_async_smem();
  __syncthreads();
  if (warp == 0) {
    issue_s(0);
    if (nb > 1) issue_s(1);
  }

  // POOL: selection blocks per key block, and the (batch, head) slice of the pooled output
  const int cpf_shift = POOL ? 31 - __clz(P.cpf) : 0, kb_shift = 6 - cpf_shift;
  const float inv_cpf = POOL ? 1.f / (float)P.cpf : 1.f;
  __nv_bfloat16* const pooled_head = POOL ? P.pooled + ((int64_t)b * P.Hkv + h) * P.N * P.pool_cols : nullptr;

  float m_ref = -INFINITY, l = 0.f;   // l: this thread's half of the row sum
  for (int t = 0; t < nb; ++t) {
    const int j = jb + t, sb = t & 1;
    __syncwarp();
    mbar_wait_warp(bar_s(t), (uint32_t)(t >> 1) & 1, &abort_flag);
    tc_fence_after_sync();
    if (tid == 0 && t + 2 < nb) load_k(t + 2);   // S(t) is complete: its K buffer is free
    __syncwarp();
    float s[32];
    tmem_ld32(tm_lane + sb * 64 + half * 32, s);
    tmem_ld_wait();
    // visible columns of this block for this row, relative to this thread's half
    int lo = 0, lim;
    if (MODE == kModeCmp) {
      lim = min(kBlock - 1, P.rule.num_mem + i / P.rule.stride - 1 - j * kBlock);
    } else {
      lim = min(kBlock - 1, i - j * kBlock);
      lo = max(0, i - P.rule.window - j * kBlock);
    }
    if (!valid) lim = -1;
    lim -= half * 32;
    lo -= half * 32;
    if constexpr (IMP) {
      // the scaled logit of every visible block column, averaged over the G heads of the query (G neighbouring
      // lanes), as the tensor of that dtype would hold it upstream: product, scaled logit and mean each rounded to
      // bf16.  The G lanes reduce-scatter: every step a lane hands half of its columns to its partner and keeps the
      // other half, so that it ends with 32/G fully summed columns, which it stores.
      float v[32];
#pragma unroll
      for (int x = 0; x < 32; ++x) v[x] = round_bf16(round_bf16(s[x]) * P.scale);
      int first = 0;
#pragma unroll
      for (int step = 0; step < 4; ++step) {
        constexpr int kG = IMP ? GI : 1;
        const int width = 16 >> step;
        if ((1 << step) < kG) {
          const bool upper = (g >> step) & 1;
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            if (x < width) {
              const float give = upper ? v[x] : v[x + width];
              const float keep = upper ? v[x + width] : v[x];
              v[x] = keep + __shfl_xor_sync(kFullMask, give, 1 << step);
            }
          }
          first += upper ? width : 0;
        }
      }
      constexpr int owned = 32 / (IMP ? (GI > 16 ? 16 : GI) : 1);
      float* imp_row = P.importance + (((int64_t)b * P.Hkv + h) * P.N + (valid ? i : 0)) * P.ncb;
      constexpr float inv_g = 1.f / (float)(IMP ? GI : 1);
      const int col0 = j * kBlock + half * 32 + first - P.rule.num_mem;
      if constexpr (POOL) {
        // this lane's `owned` neighbouring columns in one store (indexed by logit column, memory slots included)
        uint32_t w[owned / 2];
#pragma unroll
        for (int x = 0; x < owned / 2; ++x) w[x] = pack_bf16(v[2 * x] * inv_g, v[2 * x + 1] * inv_g);
        __nv_bfloat16* dst = ring + q_local * kRing + ((j & 1) * kBlock + half * 32 + first);
        if constexpr (owned == 2) *reinterpret_cast<uint32_t*>(dst) = w[0];
        else if constexpr (owned == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
#pragma unroll
        for (int x = 0; x < owned; ++x) {
          const int col = col0 + x;
          if (valid && first + x <= lim && col >= 0 && col < P.ncb) imp_row[col] = round_bf16(v[x] * inv_g);
        }
      }
    }
    // most blocks are fully visible to every row of the warp: they take the loops without per-column tests
    const bool all_full = __all_sync(kFullMask, lim >= 31 && lo <= 0);
    float m = -INFINITY;
    if (all_full) {
#pragma unroll
      for (int x = 0; x < 32; ++x) m = fmaxf(m, s[x]);
    } else {
#pragma unroll
      for (int x = 0; x < 32; ++x) m = ((MODE == kModeCmp || x >= lo) && x <= lim) ? fmaxf(m, s[x]) : m;
    }
    // the row maximum over both halves
    xchg[half * kRows + row] = m;
    __syncthreads();
    m = fmaxf(m, xchg[(half ^ 1) * kRows + row]);
    if constexpr (POOL) {
      // the selection blocks whose last column this key block brought: mean of their cpf columns in the order and
      // with the roundings of the selection kernel's own averaging; only blocks wholly before the query's own block
      // are stored (all others have probability 0 in the selection, whatever their logits)
      const int nm = P.rule.num_mem;
      const int b_lo = t == 0 ? 0 : (j * kBlock - nm) >> cpf_shift;
      const int b_hi = min(P.pool_cols, (j * kBlock + kBlock - nm) >> cpf_shift);
      for (int e = tid; e < (QT << kb_shift); e += kThreads) {
        const int pq = e >> kb_shift, bb = b_lo + (e & ((1 << kb_shift) - 1));
        const int qi = i0 + pq;
        if (bb < b_hi && qi < P.N && (bb + 1) * P.pool_block <= qi) {
          const __nv_bfloat16* src = ring + pq * kRing;
          const int c0 = (bb << cpf_shift) + nm;
          float sum = 0.f;
          for (int c = 0; c < (1 << cpf_shift); ++c) sum += __bfloat162float(src[(c0 + c) & 127]);
          pooled_head[(int64_t)qi * P.pool_cols + bb] = __float2bfloat16_rn(sum * inv_cpf);   // cpf is a power of two
        }
      }
    }
    const float m_blk2 = m * P.scale_log2;   // -inf when the row sees nothing of this block
    bool need = false;
    float alpha = 1.f;
    if (m_ref == -INFINITY) {
      m_ref = m_blk2;
    } else if (m_blk2 > m_ref + 8.f) {
      alpha = ex2(m_ref - m_blk2);
      m_ref = m_blk2;
      l *= alpha;
      need = true;
    }
    if (t > 0 && __any_sync(kFullMask, need)) {
      // some row of this warp outgrew its reference maximum: scale the accumulator rows (PV(t-1) must be complete);
      // each half scales its half of the output columns
      mbar_wait_warp(bar_pv, (uint32_t)(t - 1) & 1, &abort_flag);
      tc_fence_after_sync();
#pragma unroll 1
      for (int c2 = 0; c2 < D / 32; ++c2) {
        float o[16];
        tmem_ld16(tm_lane + tO + half * (D / 2) + c2 * 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 16; ++x) o[x] *= alpha;
        tmem_st16(tm_lane + tO + half * (D / 2) + c2 * 16, o);
      }
      tmem_st_wait();
    }
    if (all_full) {
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const float p = ex2(s[x] * P.scale_log2 - m_ref);
        s[x] = p;
        l += p;
      }
    } else {
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const float p = ((MODE == kModeCmp || x >= lo) && x <= lim) ? ex2(s[x] * P.scale_log2 - m_ref) : 0.f;
        s[x] = p;
        l += p;
      }
    }
    if (t > 0) {   // PV(t-1) is complete: V buffer (t-1) & 1 is free
      mbar_wait_warp(bar_pv, (uint32_t)(t - 1) & 1, &abort_flag);
      tc_fence_after_sync();
    }
    if (tid == 0 && t + 1 < nb) load_v(t + 1);
    // P through tensor memory, over the first 32 columns of S buffer sb (both threads of the row have read their S
    // columns: the exchange of the maxima lies in between); S(t+2), which is issued after PV(t) by the same lane,
    // overwrites them only after PV(t) has read them
    tmem_st_bf16_row32(tm_lane + sb * 64 + half * 16, s);
    tmem_st_wait();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
      mbar_wait_bounded(bar_v(t), (uint32_t)(t >> 1) & 1, &abort_flag);
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t sV = sV0 + sb * kTileKV;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_bf16_tmem_a_elect(tm + tO, tm + sb * 64 + k * 8, smem_desc_sw128(sV + k * 2048, 8192), idO, t > 0 || k > 0);
      mma_commit_elect(bar_pv);
      if (t + 2 < nb) issue_s(t + 2);
    }
  }

  // output rows: O / l through the staging area, whole 128-byte lines per store instruction
  __syncwarp();
  if (nb > 0) {
    mbar_wait_warp(bar_pv, (uint32_t)(nb - 1) & 1, &abort_flag);
    tc_fence_after_sync();
  }
  __syncthreads();                       // nobody reads the maxima any more: the exchange area takes the sums
  xchg[half * kRows + row] = l;
  __syncthreads();
  l += xchg[(half ^ 1) * kRows + row];
  __syncthreads();                       // the sums are read: the staging area (which covers them) may be written
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int64_t row_global = ((int64_t)b * P.Hq + hq) * P.N + (valid ? i : 0);
#pragma unroll
  for (int c2 = 0; c2 < D / 64; ++c2) {
    float tt[32];
    tmem_ld32(tm_lane + tO + half * (D / 2) + c2 * 32, tt);
    tmem_ld_wait();
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      uint4 v;
      v.x = pack_bf16(tt[x * 8 + 0] * inv, tt[x * 8 + 1] * inv);
      v.y = pack_bf16(tt[x * 8 + 2] * inv, tt[x * 8 + 3] * inv);
      v.z = pack_bf16(tt[x * 8 + 4] * inv, tt[x * 8 + 5] * inv);
      v.w = pack_bf16(tt[x * 8 + 6] * inv, tt[x * 8 + 7] * inv);
      sts_v4(sStage + row * kStageStride + half * D + c2 * 64 + x * 16, v);
    }
  }
  if (half == 0) row_dst[row] = valid && nb > 0 ? (int)row_global : -1;
  __syncthreads();
  if (half == 0) {
    store_rows_coalesced<D * 2>(sStage, kStageStride, row_dst, reinterpret_cast<uint8_t*>(P.out), row);
    if (valid) P.lse[row_global] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
  }

  // nothing of this CTA may still be running on the tensor cores when tensor memory is freed
  if (warp == 0) {
    mma_commit_elect(smem_u32(&bars[7]));
    mbar_wait_drain(smem_u32(&bars[7]), 0);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kCols);
  if (tid == 0 && abort_flag) atomicExch(P.status, 1);
}

// ---- backward --------------------------------------------------------------------------

// delta[row] = sum_c out[row][c] * dout[row][c]; D/8 threads per row
template <int D>
__global__ void __launch_bounds__(256) sel_delta_kernel(const SelParams P, float* delta) {
  constexpr int TPR = D / 8;
  const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const int64_t nrows = (int64_t)P.B * P.Hq * P.N;
  float acc = 0.f;
  if (row < nrows) {
    const int i = (int)(row % P.N);
    const int hq = (int)((row / P.N) % P.Hq);
    const int b = (int)(row / ((int64_t)P.N * P.Hq));
    const uint4 o = *reinterpret_cast<const uint4*>(P.out + b * P.o_sb + (int64_t)hq * P.o_sh + (int64_t)i * P.o_sn + part * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(P.dout + b * P.do_sb + (int64_t)hq * P.do_sh + (int64_t)i * P.do_sn + part * 8);
    const uint32_t ou[4] = {o.x, o.y, o.z, o.w}, gu[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      acc = fmaf(__uint_as_float(ou[x] << 16), __uint_as_float(gu[x] << 16), acc);
      acc = fmaf(__uint_as_float(ou[x] & 0xffff0000u), __uint_as_float(gu[x] & 0xffff0000u), acc);
    }
  }
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(kFullMask, acc, o);
  if (row < nrows && part == 0) delta[row] = acc;
}


template <int D>
__global__ void __launch_bounds__(kRows, D == 64 ? 2 : 1)
sel_bwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelParams P) {
  constexpr int NC = D / 64;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bars[3];
  const int nitems = item_count(P);
  if ((int)blockIdx.x >= nitems) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sDO = sQ + NC * 16384, sK = sDO + NC * 16384, sV = sK + NC * 8192;
  const uint32_t sP = sV + NC * 8192, sDS = sP + 16384;
  // the P and dS tiles (plus a tail) double as the staging area of the dQ rows (one padded fp32 row per thread)
  constexpr uint32_t kStageStride = D * 4 + 16;
  const uint32_t sStage = sP;
  const uint32_t bar_kv = smem_u32(&bars[0]), bar_1 = smem_u32(&bars[1]), bar_2 = smem_u32(&bars[2]);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t kCols = D == 64 ? 256 : 512;
  // tensor-memory columns: S and dP first; dQ overwrites them once they have been read
  constexpr uint32_t tS = 0, tDP = 64, tDQ = 0, tDK = 128, tDV = 128 + D;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_1, 1);
    mbar_init(bar_2, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_slot;
  const uint32_t tm_lane = tm + ((uint32_t)(warp * 32) << 16);

  const int G = P.G, QT = kRows / G, g_shift = 31 - __clz(G);
  const int q_local = tid / G, g = tid - q_local * G;
  uint32_t ph_kv = 0, ph_1 = 0, ph_2 = 0;
  constexpr uint32_t idS = instr_desc_bf16(128, 64, false, false);    // S, dP : K-major A and B
  constexpr uint32_t idDQ = instr_desc_bf16(128, D, false, true);     // dQ = dS K    : B MN-major
  constexpr uint32_t idKV = instr_desc_bf16(64, D, true, true);       // dK, dV       : A and B MN-major

  for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
    const int4 item = P.items[it];
    const int list = item.x, j = list % P.nfb, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * NC * 8192);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        tma_load_4d(sK + c * 8192, &tmK, bar_kv, c * 64, j * kBlock, h, b);
        tma_load_4d(sV + c * 8192, &tmV, bar_kv, c * 64, j * kBlock, h, b);
      }
    }
    for (int c = 0; c < item.z; ++c) {
      const uint32_t* chunk_entries = P.entries + item.w + c * QT;
      const uint32_t e = chunk_entries[q_local];
      const RowInfo r = decode_row(e, j, P.rule);
      const int64_t hq = (int64_t)h * G + g;
      const int64_t row_global = ((int64_t)b * P.Hq + hq) * P.N + r.i;
      gather_tile<D>(sQ, P.q + b * P.q_sb, P.q_sh, P.q_sn, chunk_entries, g_shift, h, tid);
      gather_tile<D>(sDO, P.dout + b * P.do_sb, P.do_sh, P.do_sn, chunk_entries, g_shift, h, tid);
      const float lse2 = r.valid ? P.lse[row_global] * kLog2e : 0.f;
      const float delta = r.valid ? P.delta[row_global] : 0.f;
      fence_proxy_async_smem();
      bulk_wait_read();   // the previous chunk's dQ rows have left the staging area (= the P and dS tiles)
      __syncthreads();
      if (tid == 0) {
        if (c == 0) mbar_wait_bounded(bar_kv, ph_kv, &abort_flag);
        tc_fence_after_sync();
        // (an MMA that accumulates into the previous one's tile waits for it, so independent chains are interleaved)
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ch = k / 4, in = (k % 4) * 32;
          mma_bf16(tm + tS, smem_desc_sw128(sQ + ch * 16384 + in, 16), smem_desc_sw128(sK + ch * 8192 + in, 16), idS,
                   k > 0);
          mma_bf16(tm + tDP, smem_desc_sw128(sDO + ch * 16384 + in, 16), smem_desc_sw128(sV + ch * 8192 + in, 16), idS,
                   k > 0);
        }
        mma_commit(bar_1);
      }
      __syncwarp();
      mbar_wait_bounded(bar_1, ph_1, &abort_flag);
      ph_1 ^= 1;
      tc_fence_after_sync();
      __syncwarp();
      float p[64], ds[64];
      {
        float t[32];
        tmem_ld32(tm_lane + tS, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 32; ++x) p[x] = t[x];
        tmem_ld32(tm_lane + tS + 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 32; ++x) p[32 + x] = t[x];
        tmem_ld32(tm_lane + tDP, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 32; ++x) ds[x] = t[x];
        tmem_ld32(tm_lane + tDP + 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 32; ++x) ds[32 + x] = t[x];
      }
      float slot_part = 0.f;
#pragma unroll
      for (int x = 0; x < 64; ++x) {
        const float sx = p[x];
        const float px = (x >= r.lo && x <= r.lim) ? ex2(sx * P.scale_log2 - lse2) : 0.f;
        const float dsx = px * (ds[x] - delta);
        slot_part = fmaf(dsx, sx * P.scale, slot_part);
        p[x] = px;
        ds[x] = dsx * P.scale;
      }
      store_row_bf16(sP, tid, p);
      store_row_bf16(sDS, tid, ds);
      if (P.slot_grads != nullptr) {
        for (int o = G / 2; o > 0; o >>= 1) slot_part += __shfl_xor_sync(kFullMask, slot_part, o);
        if (r.valid && g == 0 && r.slot < P.nsel)
          P.slot_grads[(((int64_t)b * P.Hkv + h) * P.N + r.i) * P.nsel + r.slot] = slot_part;
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after_sync();
        // dV += P^T dO, dK += dS^T Q over the 128 rows of the chunk (8 steps of 16 rows) and dQ_chunk = dS K over
        // the 64 keys (4 steps of 16 keys), the three chains interleaved
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          mma_bf16(tm + tDV, smem_desc_sw128(sP + k * 2048, 16384), smem_desc_sw128(sDO + k * 2048, 16384), idKV,
                   c > 0 || k > 0);
          mma_bf16(tm + tDK, smem_desc_sw128(sDS + k * 2048, 16384), smem_desc_sw128(sQ + k * 2048, 16384), idKV,
                   c > 0 || k > 0);
          if (k < 4)
            mma_bf16(tm + tDQ, smem_desc_sw128(sDS + k * 32, 16), smem_desc_sw128(sK + k * 2048, 8192), idDQ, k > 0);
        }
        mma_commit(bar_2);
      }
      __syncwarp();
      mbar_wait_bounded(bar_2, ph_2, &abort_flag);
      ph_2 ^= 1;
      tc_fence_after_sync();
      __syncwarp();
#pragma unroll
      for (int c2 = 0; c2 < D / 32; ++c2) {
        float t[32];
        tmem_ld32(tm_lane + tDQ + c2 * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 8; ++x)
          sts_v4f(sStage + tid * kStageStride + c2 * 128 + x * 16, t[x * 4], t[x * 4 + 1], t[x * 4 + 2], t[x * 4 + 3]);
      }
      // each thread adds its own dQ row into global memory with one bulk reduction
      fence_proxy_async_smem();
      if (r.valid) bulk_reduce_add_f32(P.dq + row_global * D, sStage + tid * kStageStride, D * 4);
      bulk_commit();
      tc_fence_before_sync();
    }
    // flush dK, dV of this item: accumulator rows 16w..16w+15 live in lanes 0..15 of warp w
    {
      const int key = j * kBlock + warp * 16 + lane;
      const bool ok = lane < 16 && key < P.Nk;
      float* dkp = P.dk + (((int64_t)b * P.Hkv + h) * P.Nk + key) * D;
      float* dvp = P.dv + (((int64_t)b * P.Hkv + h) * P.Nk + key) * D;
#pragma unroll
      for (int c2 = 0; c2 < D / 32; ++c2) {
        float t[32];
        tmem_ld32(tm_lane + tDK + c2 * 32, t);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
          for (int x = 0; x < 8; ++x) red_add_v4(dkp + c2 * 32 + x * 4, t[x * 4], t[x * 4 + 1], t[x * 4 + 2], t[x * 4 + 3]);
        }
        tmem_ld32(tm_lane + tDV + c2 * 32, t);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
          for (int x = 0; x < 8; ++x) red_add_v4(dvp + c2 * 32 + x * 4, t[x * 4], t[x * 4 + 1], t[x * 4 + 2], t[x * 4 + 3]);
        }
      }
      tc_fence_before_sync();
    }
    ph_kv ^= 1;
    __syncthreads();
  }

  bulk_wait_read();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kCols);
  if (tid == 0 && abort_flag) atomicExch(P.status, 1);
}


// ---- backward, warp-specialised ---------------------------------------------------------------
//
// One CTA per SM, 13 warps with fixed roles, so that the gathers, the tensor-core work and the per-row
// arithmetic of different chunks overlap instead of taking turns:
//   warps 0-3, 4-7  two softmax groups; chunk n (counted per CTA) belongs to group n % 2.  A thread owns one row:
//                   it reads S and dP from tensor memory, writes P and dS (bf16) for the second set of MMAs and
//                   later stores its dQ row as a bf16 partial result (summed by sel_dq_merge_kernel).  Group t % 2
//                   also flushes dK/dV of item t with fp32 reductions.
//   warp 8          one thread issues every tcgen05.mma: S/dP of chunk n+1 before dQ/dV/dK of chunk n.
//   warps 9-12      gather the Q and dO rows with 16-byte cp.async into a ring of kStages stages; a stage announces
//                   itself (cp.async.mbarrier.arrive) when the copies have landed, the threads never wait for data.
//   warp 13         one thread requests the K/V tiles of each item by TMA (double buffered).  It is a role of its
//                   own because it waits for the consumer: a gathering thread that did so would hold back the
//                   announcements the consumer is waiting for.
// Tensor memory (512 columns): per softmax group S, dP and dQ (64 columns each), then dK and dV (64 each).  dQ has
// columns of its own so that a group can go on to the S/dP of its next chunk and read dQ of the previous one out
// afterwards, while the tensor cores are busy with the other group's chunk.
// Every hand-over is an mbarrier; every wait is bounded.
namespace ws {
constexpr int kStages = 3;
constexpr uint32_t kMetaBytes = 3 * kRows * 4;   // per stage: entry, lse, delta of every row of the chunk
constexpr uint32_t kPBytes = 32768;   // P and dS tiles
constexpr uint32_t kDqRow = 64;       // staged half dQ row; its 16-byte pieces are swizzled with the row pair's index
constexpr uint32_t kDqStage = 32 * kDqRow;   // per softmax warp
constexpr int kThreads = 14 * 32;
constexpr int kLoaderThreads = 128;

struct Bars {
  uint64_t q_full[kStages], q_free[kStages];
  uint64_t s_full[2], p_full[2], mma2_done[2], dq_free[2];
  uint64_t kv_full[2], kv_free[2], acc_full[2], acc_free;
  uint64_t drain;
};
}  // namespace ws

__global__ void __launch_bounds__(ws::kThreads, 1)
sel_bwd_ws_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelParams P) {
  using namespace ws;
  constexpr int D = 64;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) Bars bars;
  const int nitems = item_count(P);
  if ((int)blockIdx.x >= nitems) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // stage s: Q tile then dO tile (16 KB each); buffer b: P tile then dS tile; KV buffer: K tile then V tile (8 KB each)
  const uint32_t sQ0 = base, sP0 = sQ0 + kStages * 32768, sKV0 = sP0 + 2 * kPBytes, sMeta0 = sKV0 + 2 * 16384,
                 sDq0 = sMeta0 + kStages * kMetaBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), kLoaderThreads);
      mbar_init(smem_u32(&bars.q_free[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.p_full[i]), kRows);
      mbar_init(smem_u32(&bars.mma2_done[i]), 1);
      mbar_init(smem_u32(&bars.dq_free[i]), kRows);
      mbar_init(smem_u32(&bars.kv_full[i]), 1);
      mbar_init(smem_u32(&bars.kv_free[i]), 1);
    }
    mbar_init(smem_u32(&bars.acc_full[0]), 1);
    mbar_init(smem_u32(&bars.acc_full[1]), 1);
    mbar_init(smem_u32(&bars.acc_free), kRows);
    mbar_init(smem_u32(&bars.drain), 1);
    fence_mbar_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_slot;
  const int G = P.G, QT = kRows / G, g_shift = 31 - __clz(G);

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax groups
    const int wg = warp >> 2, r_tid = tid & 127;
    const uint32_t tm_lane = tm + ((uint32_t)((warp & 3) * 32) << 16);
    const int q_local = r_tid >> g_shift, g = r_tid - (q_local << g_shift);
    const uint32_t tS = wg * 192, tDP = tS + 64, tDQ = tS + 128;
    const uint32_t sP = sP0 + wg * kPBytes, sDS = sP + 16384;
    // dQ row of the group's previous chunk, still to be read out of tensor memory: index of its (row, slot) partial
    int prev_dst = -1;
    bool have_prev = false;
    uint32_t prev_use = 0;
    const uint32_t sDq = sDq0 + warp * kDqStage;
    // The dQ rows go out as the bf16 partial results of their (row, slot); sel_dq_merge_kernel sums them (plain stores
    // run at memory speed, fp32 reductions into dq are limited by the L2 atomic units).  A thread that stored its own
    // 128-byte row would make every store instruction touch 32 lines; the warp stages half rows in shared memory
    // instead and stores them eight rows per instruction.
    auto dq_out = [&]() {
      mbar_wait_warp(smem_u32(&bars.mma2_done[wg]), prev_use & 1, &abort_flag);
      tc_fence_after_sync();
      __syncwarp();
      uint8_t* const pbase = reinterpret_cast<uint8_t*>(P.partial);
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        float tq[32];
        tmem_ld32(tm_lane + tDQ + half * 32, tq);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          uint4 v;
          v.x = pack_bf16(tq[x * 8 + 0], tq[x * 8 + 1]); v.y = pack_bf16(tq[x * 8 + 2], tq[x * 8 + 3]);
          v.z = pack_bf16(tq[x * 8 + 4], tq[x * 8 + 5]); v.w = pack_bf16(tq[x * 8 + 6], tq[x * 8 + 7]);
          sts_v4(sDq + lane * kDqRow + ((x ^ ((lane >> 1) & 3)) << 4), v);   // conflict-free to write and to read
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int rr = k * 8 + (lane >> 2);
          const int dst = __shfl_sync(kFullMask, prev_dst, rr);
          const uint4 v = lds_v4(sDq + rr * kDqRow + (((lane & 3) ^ ((rr >> 1) & 3)) << 4));
          if (dst >= 0)
            *reinterpret_cast<uint4*>(pbase + (int64_t)dst * (D * 2) + half * 64 + (lane & 3) * 16) = v;
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars.dq_free[wg]));   // the dQ columns of this group may be overwritten
      have_prev = false;
    };
    // one chunk of this group; the thread's entry and its row's statistics come from the stage's metadata, which
    // the loaders fetched together with the rows
    auto process_chunk = [&](const int4 item, const int n) {
      {
        const int list = item.x, j = list % P.nfb, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
        const uint32_t use = (uint32_t)(n >> 1);   // how many chunks this group has had before
        const uint32_t sMeta = sMeta0 + (n % kStages) * kMetaBytes + r_tid * 4;
        mbar_wait_warp(smem_u32(&bars.s_full[wg]), use & 1, &abort_flag);
        tc_fence_after_sync();
        const uint32_t e = lds_u32(sMeta);
        const float lse2 = __uint_as_float(lds_u32(sMeta + kRows * 4)) * kLog2e;
        const float delta = __uint_as_float(lds_u32(sMeta + 2 * kRows * 4));
        const RowInfo r = decode_row(e, j, P.rule);
        const int64_t hq = (int64_t)h * G + g;
        const int64_t row_global = ((int64_t)b * P.Hq + hq) * P.N + r.i;
        float slot_part = 0.f;
        const bool want_slot = P.slot_grads != nullptr;
        // rows that see the whole block need no per-column test; only own-block (causal) and padding rows do
        const bool all_full = __all_sync(kFullMask, r.lim == kBlock - 1 && r.lo == 0);
        // 16 columns at a time in a rolled loop: the body stays small enough for the instruction cache, which four
        // roles share
        auto math16 = [&](float (&sv)[16], float (&dv)[16], const int q4) {
          const int rem = r.lim - q4 * 16, rlo = r.lo - q4 * 16;   // columns rlo..rem of this group are visible
          if (all_full) {
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              const float sx = sv[x];
              const float px = ex2(sx * P.scale_log2 - lse2);
              const float dsx = px * (dv[x] - delta);
              if (want_slot) slot_part = fmaf(dsx, sx, slot_part);
              sv[x] = px;
              dv[x] = dsx;
            }
          } else {
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              const float sx = sv[x];
              const float px = (x >= rlo && x <= rem) ? ex2(sx * P.scale_log2 - lse2) : 0.f;
              const float dsx = px * (dv[x] - delta);
              if (want_slot) slot_part = fmaf(dsx, sx, slot_part);
              sv[x] = px;
              dv[x] = dsx;
            }
          }
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            uint4 pv, dsv;
            pv.x = pack_bf16(sv[x * 8 + 0], sv[x * 8 + 1]); pv.y = pack_bf16(sv[x * 8 + 2], sv[x * 8 + 3]);
            pv.z = pack_bf16(sv[x * 8 + 4], sv[x * 8 + 5]); pv.w = pack_bf16(sv[x * 8 + 6], sv[x * 8 + 7]);
            dsv.x = pack_bf16(dv[x * 8 + 0], dv[x * 8 + 1]); dsv.y = pack_bf16(dv[x * 8 + 2], dv[x * 8 + 3]);
            dsv.z = pack_bf16(dv[x * 8 + 4], dv[x * 8 + 5]); dsv.w = pack_bf16(dv[x * 8 + 6], dv[x * 8 + 7]);
            sts_v4(sP + sw128_offset(r_tid, q4 * 2 + x), pv);
            sts_v4(sDS + sw128_offset(r_tid, q4 * 2 + x), dsv);
          }
        };
        {
          float sa[16], da[16], sb[16], db[16];
          tmem_ld16(tm_lane + tS, sa);
          tmem_ld16(tm_lane + tDP, da);
          tmem_ld_wait();
#pragma unroll 1
          for (int q2 = 0; q2 < 2; ++q2) {
            tmem_ld16(tm_lane + tS + q2 * 32 + 16, sb);
            tmem_ld16(tm_lane + tDP + q2 * 32 + 16, db);
            math16(sa, da, q2 * 2);
            tmem_ld_wait();
            if (q2 == 0) {
              tmem_ld16(tm_lane + tS + 32, sa);
              tmem_ld16(tm_lane + tDP + 32, da);
            }
            math16(sb, db, q2 * 2 + 1);
            tmem_ld_wait();
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bars.p_full[wg]));
        if (P.slot_grads != nullptr) {
          for (int o = G / 2; o > 0; o >>= 1) slot_part += __shfl_xor_sync(kFullMask, slot_part, o);
          if (r.valid && g == 0 && r.slot < P.nsel)
            P.slot_grads[(((int64_t)b * P.Hkv + h) * P.N + r.i) * P.nsel + r.slot] = slot_part * P.scale;
        }
        // while the tensor cores work on this chunk's P and dS, read out dQ of the previous chunk of the group
        if (have_prev) dq_out();
        prev_dst = r.valid ? (int)(row_global * P.ns + r.slot) : -1;
        prev_use = use;
        have_prev = true;
      }
    };
    uint32_t flushes = 0;   // items this group has flushed
    auto flush_item = [&](const int4 item, const int t) {
      const int list = item.x, j = list % P.nfb, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
      {
        // flush dK/dV of this item: accumulator rows 16w..16w+15 live in lanes 0..15 of warp w of the group.
        // "Accumulator complete" has one barrier per flushing group, counted by that group: with one barrier for both,
        // a group that reached its wait before the other group's item was complete saw the phase before that one
        // (same parity) as its own and flushed early.
        mbar_wait_warp(smem_u32(&bars.acc_full[wg]), flushes & 1, &abort_flag);
        ++flushes;
        tc_fence_after_sync();
        __syncwarp();
        const int key = j * kBlock + (warp & 3) * 16 + lane;
        const bool ok = lane < 16 && key < P.Nk;
        float* dkp = P.dk + (((int64_t)b * P.Hkv + h) * P.Nk + key) * D;
        float* dvp = P.dv + (((int64_t)b * P.Hkv + h) * P.Nk + key) * D;
        const uint32_t tDK = 384, tDV = 448;
#pragma unroll
        for (int c2 = 0; c2 < D / 32; ++c2) {
          float tk[32];
          tmem_ld32(tm_lane + tDK + c2 * 32, tk);
          tmem_ld_wait();
          if (ok) {
#pragma unroll
            for (int x = 0; x < 8; ++x)
              red_add_v4(dkp + c2 * 32 + x * 4, tk[x * 4] * P.scale, tk[x * 4 + 1] * P.scale, tk[x * 4 + 2] * P.scale, tk[x * 4 + 3] * P.scale);
          }
          tmem_ld32(tm_lane + tDV + c2 * 32, tk);
          tmem_ld_wait();
          if (ok) {
#pragma unroll
            for (int x = 0; x < 8; ++x) red_add_v4(dvp + c2 * 32 + x * 4, tk[x * 4], tk[x * 4 + 1], tk[x * 4 + 2], tk[x * 4 + 3]);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bars.acc_free));
      }
    };
    // dK/dV of an item are flushed by the group that had the item's last chunk, as soon as the tensor cores are done
    // with it: the next item's dV/dK MMAs wait for the accumulator
    int n = 0, t = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++t) {
      const int4 item = P.items[it];
      for (int c = 0; c < item.z; ++c, ++n) {
        if ((n & 1) != wg) continue;
        process_chunk(item, n);
        if (c == item.z - 1) flush_item(item, t);
      }
    }
    if (have_prev) dq_out();
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer: the whole warp runs the loop
    // (so that its state lives in uniform registers), one elected lane issues
    {
    constexpr uint32_t idS = instr_desc_bf16(128, 64, false, false);
    constexpr uint32_t idDQ = instr_desc_bf16(128, D, false, true);
    constexpr uint32_t idKV = instr_desc_bf16(64, D, true, true);
    int n = 0, t = 0;
    // state of the chunk whose second set of MMAs is still to be issued
    bool pending = false;
    int p_n = 0, p_t = 0, p_c = 0;
    bool p_last = false;
    auto issue_mma2 = [&](int pn, int pt, int pc, bool last) {
      const int grp = pn & 1, stage = pn % kStages, kb = pt & 1;
      const uint32_t sQ = sQ0 + stage * 32768, sDO = sQ + 16384;
      const uint32_t sP = sP0 + grp * kPBytes, sDS = sP + 16384;
      const uint32_t sK = sKV0 + kb * 16384;
      mbar_wait_bounded(smem_u32(&bars.p_full[grp]), (uint32_t)(pn >> 1) & 1, &abort_flag);
      // the accumulators are single: the first chunk of an item waits until the previous item has been flushed
      if (pc == 0 && pt >= 1) mbar_wait_bounded(smem_u32(&bars.acc_free), (uint32_t)(pt - 1) & 1, &abort_flag);
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t tDK = 384, tDV = 448, tDQ = grp * 192 + 128;
      // One descriptor per tile (the leading-offset field is unused for 64-wide tiles, so the same descriptor
      // serves the K-major and the MN-major reading of a tile); every MMA then costs one 64-bit add to issue.
      const uint64_t dQt = smem_desc_sw128(sQ, 16), dDOt = smem_desc_sw128(sDO, 16), dPt = smem_desc_sw128(sP, 16),
                     dDSt = smem_desc_sw128(sDS, 16), dKt = smem_desc_sw128(sK, 16);
      // dV and dK first: the group reads dQ of its previous chunk out right after it has handed P and dS over, and
      // is done with it by the time these sixteen MMAs have been issued.
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_bf16_elect(tm + tDV, desc_advance(dPt, k * 2048), desc_advance(dDOt, k * 2048), idKV, pc > 0 || k > 0);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_bf16_elect(tm + tDK, desc_advance(dDSt, k * 2048), desc_advance(dQt, k * 2048), idKV, pc > 0 || k > 0);
      if (pn >= 2) {
        mbar_wait_bounded(smem_u32(&bars.dq_free[grp]), (uint32_t)((pn >> 1) - 1) & 1, &abort_flag);
        __syncwarp();
        tc_fence_after_sync();
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_bf16_elect(tm + tDQ, desc_advance(dDSt, k * 32), desc_advance(dKt, k * 2048), idDQ, k > 0);
      mma_commit_elect(smem_u32(&bars.mma2_done[grp]));
      mma_commit_elect(smem_u32(&bars.q_free[stage]));
      if (last) {
        mma_commit_elect(smem_u32(&bars.kv_free[kb]));
        mma_commit_elect(smem_u32(&bars.acc_full[grp]));   // the group of the item's last chunk flushes
      }
    };
    for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++t) {
      const int4 item = P.items[it];
      const int kb = t & 1;
      for (int c = 0; c < item.z; ++c, ++n) {
        const int grp = n & 1, stage = n % kStages;
        const uint32_t sQ = sQ0 + stage * 32768, sDO = sQ + 16384;
        const uint32_t sK = sKV0 + kb * 16384, sV = sK + 8192;
        mbar_wait_bounded(smem_u32(&bars.q_full[stage]), (uint32_t)(n / kStages) & 1, &abort_flag);
        if (c == 0) mbar_wait_bounded(smem_u32(&bars.kv_full[kb]), (uint32_t)(t >> 1) & 1, &abort_flag);
        __syncwarp();
        tc_fence_after_sync();
        {
          // S and dP of the group are free: the group handed P and dS of its previous chunk over (waited for in
          // issue_mma2 of that chunk, which ran before this point) only after reading them
          const uint32_t tS = grp * 192, tDP = tS + 64;
          const uint64_t dQt = smem_desc_sw128(sQ, 16), dDOt = smem_desc_sw128(sDO, 16), dKt = smem_desc_sw128(sK, 16),
                         dVt = smem_desc_sw128(sV, 16);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_bf16_elect(tm + tS, desc_advance(dQt, k * 32), desc_advance(dKt, k * 32), idS, k > 0);
            mma_bf16_elect(tm + tDP, desc_advance(dDOt, k * 32), desc_advance(dVt, k * 32), idS, k > 0);
          }
          mma_commit_elect(smem_u32(&bars.s_full[grp]));
        }
        if (pending) issue_mma2(p_n, p_t, p_c, p_last);
        pending = true;
        p_n = n; p_t = t; p_c = c; p_last = (c == item.z - 1);
      }
    }
    if (pending) issue_mma2(p_n, p_t, p_c, p_last);
    // nothing of this block may still be running on the tensor cores when tensor memory is freed
    mma_commit_elect(smem_u32(&bars.drain));
    mbar_wait_drain(smem_u32(&bars.drain), 0);
    }
  } else if (warp == 13) {
    // ------------------------------------------------------------------ K/V tiles
    if (lane == 0) {
      int t = 0;
      for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++t) {
        const int4 item = P.items[it];
        const int list = item.x, j = list % P.nfb, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
        const int kb = t & 1;
        if (t >= 2) mbar_wait_bounded(smem_u32(&bars.kv_free[kb]), (uint32_t)((t >> 1) - 1) & 1, &abort_flag);
        const uint32_t sK = sKV0 + kb * 16384, sV = sK + 8192;
        const uint32_t bar = smem_u32(&bars.kv_full[kb]);
        mbar_arrive_expect_tx(bar, 2 * 8192);
        tma_load_4d(sK, &tmK, bar, 0, j * kBlock, h, b);
        tma_load_4d(sV, &tmV, bar, 0, j * kBlock, h, b);
      }
      // the last two requests must have landed before the block may exit
      for (int back = 1; back <= 2 && t - back >= 0; ++back) {
        const int tt = t - back;
        mbar_wait_drain(smem_u32(&bars.kv_full[tt & 1]), (uint32_t)(tt >> 1) & 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ loaders
    const int lt = tid - 9 * 32;           // 0..127
    const int sub = lt & 7, r0 = lt >> 3;  // 16-byte piece of a row, first row (rows r0 + 16*k)
    int n = 0, t = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++t) {
      const int4 item = P.items[it];
      const int list = item.x, bh = list / P.nfb, h = bh % P.Hkv, b = bh / P.Hkv;
      const __nv_bfloat16* qb = P.q + b * P.q_sb;
      const __nv_bfloat16* dob = P.dout + b * P.do_sb;
      for (int c = 0; c < item.z; ++c, ++n) {
        const int stage = n % kStages;
        if (n >= kStages) mbar_wait_warp(smem_u32(&bars.q_free[stage]), (uint32_t)(n / kStages - 1) & 1, &abort_flag);
        const uint32_t sQ = sQ0 + stage * 32768, sDO = sQ + 16384;
        const uint32_t* chunk_entries = P.entries + item.w + c * QT;
        // read the entries first: the copies below are compiler barriers, a load placed between them would be
        // waited for eight times per chunk
        uint32_t ev[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) ev[k] = __ldg(chunk_entries + ((r0 + k * 16) >> g_shift));
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int row = r0 + k * 16;
          const int g = row & ((1 << g_shift) - 1);
          const uint32_t e = ev[k];
          const bool valid = e != kInvalidEntry;
          const int64_t i = valid ? (int64_t)(e & 0xffffffu) : 0;
          const int64_t hq = (int64_t)((h << g_shift) + g);
          const uint32_t off = sw128_offset(row, sub);
          cp_async16(sQ + off, qb + hq * P.q_sh + i * P.q_sn + sub * 8, valid ? 16u : 0u);
          cp_async16(sDO + off, dob + hq * P.do_sh + i * P.do_sn + sub * 8, valid ? 16u : 0u);
        }
        {
          // metadata of row lt: its entry and the statistics of its (query, head)
          const uint32_t e = __ldg(chunk_entries + (lt >> g_shift));
          const bool valid = e != kInvalidEntry;
          const int64_t row = ((int64_t)b * P.Hq + (int64_t)((h << g_shift) + (lt & ((1 << g_shift) - 1)))) * P.N +
                              (valid ? (int64_t)(e & 0xffffffu) : 0);
          const uint32_t sMeta = sMeta0 + stage * kMetaBytes + lt * 4;
          cp_async4(sMeta, chunk_entries + (lt >> g_shift), 4u);
          cp_async4(sMeta + kRows * 4, P.lse + row, valid ? 4u : 0u);
          cp_async4(sMeta + 2 * kRows * 4, P.delta + row, valid ? 4u : 0u);
        }
        // the stage announces itself when this thread's copies have landed; the thread moves on at once
        cp_async_arrive_noinc(smem_u32(&bars.q_full[stage]));
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && abort_flag) atomicExch(P.status, 1);
}


// sums the bf16 dQ partials of every (batch, query head, query) into the fp32 dq row: D/8 threads per row
template <int D, int MODE>
__global__ void __launch_bounds__(256) sel_dq_merge_kernel(const SelParams P) {
  constexpr int TPR = D / 8;
  const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const int64_t nrows = (int64_t)P.B * P.Hq * P.N;
  if (row >= nrows) return;
  const int i = (int)(row % P.N);
  const int hq = (int)((row / P.N) % P.Hq);
  const int b = (int)(row / ((int64_t)P.N * P.Hq));
  const int h = hq / P.G;
  const int ns = P.ns;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const __nv_bfloat16* prow = P.partial + row * ns * D + part * 8;
  // eight slots at a time: first which of them the query has, then their loads together, then the sums
  for (int s0 = 0; s0 < ns; s0 += 8) {
    bool ok[8];
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      int blk_;
      ok[u] = s0 + u < ns && slot_block<MODE>(P.rule, b * P.Hkv + h, i, s0 + u, &blk_);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      v[u] = ok[u] ? *reinterpret_cast<const uint4*>(prow + (int64_t)(s0 + u) * D) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        acc[2 * x] += __uint_as_float(q[x] << 16);
        acc[2 * x + 1] += __uint_as_float(q[x] & 0xffff0000u);
      }
    }
  }
  // the partials hold dS K without the logit scale
  if (P.dq_lp != nullptr) {   // the caller asked for dq in the dtype and row layout of q
    uint4 o;
    o.x = pack_bf16(acc[0] * P.scale, acc[1] * P.scale); o.y = pack_bf16(acc[2] * P.scale, acc[3] * P.scale);
    o.z = pack_bf16(acc[4] * P.scale, acc[5] * P.scale); o.w = pack_bf16(acc[6] * P.scale, acc[7] * P.scale);
    *reinterpret_cast<uint4*>(P.dq_lp + b * P.dq_sb + hq * P.dq_sh + i * P.dq_sn + part * 8) = o;
    return;
  }
  float4* dst = reinterpret_cast<float4*>(P.dq + row * D + part * 8);
  dst[0] = make_float4(acc[0] * P.scale, acc[1] * P.scale, acc[2] * P.scale, acc[3] * P.scale);
  dst[1] = make_float4(acc[4] * P.scale, acc[5] * P.scale, acc[6] * P.scale, acc[7] * P.scale);
}

__global__ void fill_kernel(float* dst, float value, int64_t count) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) dst[i] = value;
}

// Importance columns a causal query cannot see (column c of row i is visible iff c < i / stride): `value` from the
// first invisible column on; the attention kernel writes the visible ones.  A warp takes query i and query N-1-i of
// a (batch, head) together, so that every warp writes about one row's worth.
__device__ __forceinline__ void fill_row_from(float* r, int first, int ncb, float value, int lane) {
  const int head = min(ncb, (first + 3) & ~3);          // scalar stores up to the next 16-byte boundary
  if (first + lane < head) r[first + lane] = value;
  const float4 v4 = make_float4(value, value, value, value);
  for (int c = head + 4 * lane; c < ncb; c += 128) *reinterpret_cast<float4*>(r + c) = v4;
}

__global__ void __launch_bounds__(256) fill_invisible_kernel(float* dst, float value, int64_t slices, int N, int ncb, int stride) {
  const int lane = threadIdx.x & 31;
  const int half = (N + 1) / 2;
  const int64_t warps = (int64_t)gridDim.x * 8, pairs = slices * half;
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < pairs; p += warps) {
    const int64_t slice = p / half;
    const int i = (int)(p % half), i2 = N - 1 - i;
    fill_row_from(dst + (slice * N + i) * ncb, min(ncb, i / stride), ncb, value, lane);
    if (i2 != i) fill_row_from(dst + (slice * N + i2) * ncb, min(ncb, i2 / stride), ncb, value, lane);
  }
}

// ---- host ----------------------------------------------------------------------------------

static int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// One problem of any of the three branches, as the host code sees it.
struct SelProblem {
  nsa_tensor q, k, v, out, dout;
  const int64_t* idx;
  const uint8_t* mask;
  float* lse;
  float *dq, *dk, *dv, *slot_grads;
  nsa_tensor dq_out;       // backward, optional: dq in the dtype and strides the caller chose
  float* importance;
  __nv_bfloat16* pooled;   // compressed forward, instead of importance: per-selection-block means, see SelParams
  int cpf;
  void* workspace;
  int64_t workspace_bytes;
  const CombineParams* fuse_combine;   // selected forward, optional: the merge also combines and stores (see
  const GatherTargets* fuse_targets;   // sel_merge_combine_kernel); `out` is then not written
  const void* index;       // backward: the index part of the forward's work buffer, or NULL to rebuild it
  int64_t index_bytes;
  const float* delta;      // backward, optional: sum_d out * dout per row from the caller
  int B, Hq, Hkv, N, Nk, D;
  int nsel, diag, mode, window, stride, num_mem, ncb, round_bf16;
  float scale;
};

static int slots_per_query(const SelProblem& a) {
  if (a.mode == kModeSel) return a.nsel + 1;
  if (a.mode == kModeSwa) return a.window / kBlock + 2;   // own block + every older block the window can touch
  return (a.Nk + kBlock - 1) / kBlock;
}

// Shapes served by this family; everything else goes to the generic kernels.
static bool supported(const SelProblem& a) {
  if (a.D != 64 && a.D != 128) return false;
  const int G = a.Hq / a.Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return false;
  if (a.N < 1 || a.N >= (1 << 24) || a.Nk < 1 || a.B < 1) return false;
  if (a.mode == kModeSel && a.diag == NSA_DIAG_NONE) return false;   // a query must see at least one key
  const int64_t ns = slots_per_query(a);
  if (ns > 255) return false;
  const int64_t nqb = (a.N + kBlock - 1) / kBlock, nkb = (a.Nk + kBlock - 1) / kBlock;
  if (nkb > 8192) return false;
  const int64_t lists = (int64_t)a.B * a.Hkv * nkb;
  if (lists * nqb > (1ll << 31) - 1) return false;
  if ((int64_t)a.B * a.Hkv * ((int64_t)a.N * ns + nkb * kRows) > (1ll << 31) - 1) return false;
  if ((int64_t)a.B * a.Hq * (int64_t)a.N * ns > (1ll << 31) - 1) return false;   // (row, slot) ids are 32-bit
  if (a.k.stride_n < a.D || a.v.stride_n < a.D) return false;
  return true;
}

// The forward of the compressed and the sliding-window branch runs query-tile stationary (dense_fwd_kernel).  It
// stores whole rows of a plain contiguous output; other layouts of `out` (and a compressed branch without a memory
// slot, where a query may see no key) are left to the generic kernels.
static bool dense_forward(const SelProblem& a) { return a.mode != kModeSel; }
static bool dense_forward_serves(const SelProblem& a) {
  if (a.mode == kModeCmp && a.num_mem < 1) return false;
  return a.out.stride_n == a.D && a.out.stride_h == (int64_t)a.N * a.D && a.out.stride_b == (int64_t)a.Hq * a.N * a.D;
}

static SelPlan make_plan(const SelProblem& a, bool backward) {
  SelPlan p;
  p.nqb = (a.N + kBlock - 1) / kBlock;
  p.nkb = (a.Nk + kBlock - 1) / kBlock;
  p.ns = slots_per_query(a);
  p.G = a.Hq / a.Hkv;
  p.QT = kRows / p.G;
  p.nlists = a.B * a.Hkv * p.nkb;
  p.entries_cap = (int64_t)a.B * a.Hkv * (int64_t)a.N * p.ns + (int64_t)p.nlists * p.QT;
  p.items_cap = p.entries_cap / p.QT / kChunksPerItem + p.nlists + 1;
  int64_t off = 0;
  p.off_status = off; off += 256;
  p.off_num_items = p.off_status + 128;
  if (!backward && dense_forward(a)) {   // only the status word is needed
    p.off_counts = p.off_totals = p.off_list_base = p.off_items = p.off_entries = off;
    p.off_partial = p.off_stats = p.off_delta = off;
    p.index_bytes = 0;
    p.total_bytes = off;
    return p;
  }
  p.off_counts = off; off = align_up(off + (int64_t)a.B * a.Hkv * p.nqb * p.nkb * 4, 256);
  p.off_totals = off; off = align_up(off + (int64_t)p.nlists * 4, 256);
  p.off_list_base = off; off = align_up(off + (int64_t)p.nlists * 4, 256);
  p.off_items = off; off = align_up(off + p.items_cap * 16, 256);
  p.off_entries = off; off = align_up(off + p.entries_cap * 4, 256);
  p.index_bytes = off;   // status word, counts, list bases, items, entries: the same layout forward and backward
  const int64_t rows = (int64_t)a.B * a.Hq * a.N;
  p.off_partial = p.off_stats = p.off_delta = off;
  if (!backward) {
    p.off_partial = off; off = align_up(off + rows * p.ns * a.D * 2, 256);
    p.off_stats = off; off = align_up(off + rows * p.ns * 8, 256);
  } else {
    p.off_delta = off; off = align_up(off + rows * 4, 256);
    if (a.D == 64) { p.off_partial = off; off = align_up(off + rows * p.ns * a.D * 2, 256); }
  }
  p.total_bytes = off;
  return p;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over a [B, H, N, d] bf16 view; one box is a [64 rows x 64 columns] tile of one head.
static int make_kv_map(CUtensorMap* map, const nsa_tensor& t, int B, int H, int N, int d) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return fail(NSA_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)t.stride_n * 2, (cuuint64_t)(H > 1 ? t.stride_h : t.stride_n * N) * 2,
                           (cuuint64_t)(B > 1 ? t.stride_b : (H > 1 ? t.stride_h * H : t.stride_n * N)) * 2};
  cuuint32_t box[4] = {64, 64, 1, 1}, es[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return NSA_ERR_UNSUPPORTED;   // strides the tiled format cannot express
  return NSA_OK;
}

#define CUDA_TRY(expr)                                                        \
  do {                                                                        \
    const cudaError_t e_ = (expr);                                            \
    if (e_ != cudaSuccess) return fail((int)e_, cudaGetErrorString(e_));     \
  } while (0)

static BlockRule make_rule(const SelProblem& a, const SelPlan& p) {
  BlockRule R;
  R.idx = a.idx; R.mask = a.mask;
  R.N = a.N; R.nkb = p.nkb; R.nsel = a.nsel; R.ns = p.ns;
  R.diag = a.diag; R.mode = a.mode; R.window = a.window; R.stride = a.stride > 0 ? a.stride : 1; R.num_mem = a.num_mem;
  return R;
}

// A hash of everything the index depends on besides idx/mask themselves: sizes, head grouping, branch and its rule.
static uint32_t index_tag(const SelProblem& a, const SelPlan& p) {
  const uint32_t f[] = {(uint32_t)a.B, (uint32_t)a.Hkv, (uint32_t)p.G, (uint32_t)a.N, (uint32_t)a.Nk, (uint32_t)p.ns,
                        (uint32_t)a.mode, (uint32_t)a.diag, (uint32_t)a.window, (uint32_t)a.stride, (uint32_t)a.num_mem,
                        (uint32_t)a.nsel, (uint32_t)p.QT, (uint32_t)p.entries_cap};
  uint32_t h = 0x4e534149u;
  for (uint32_t v : f) h = (h ^ v) * 0x01000193u + 0x9E3779B1u;
  return h == 0 ? 1u : h;   // 0 is what a cleared buffer holds
}

static int build_index(const SelProblem& a, const SelPlan& p, uint8_t* ws, cudaStream_t st) {
  int* counts = reinterpret_cast<int*>(ws + p.off_counts);
  int* totals = reinterpret_cast<int*>(ws + p.off_totals);
  int* list_base = reinterpret_cast<int*>(ws + p.off_list_base);
  int4* items = reinterpret_cast<int4*>(ws + p.off_items);
  int* num_items = reinterpret_cast<int*>(ws + p.off_num_items);
  uint32_t* entries = reinterpret_cast<uint32_t*>(ws + p.off_entries);
  CUDA_TRY(cudaMemsetAsync(ws + p.off_status, 0, 256, st));
  CUDA_TRY(cudaMemsetAsync(entries, 0xff, (size_t)p.entries_cap * 4, st));
  const BlockRule R = make_rule(a, p);
  const dim3 grid(p.nqb, a.B, a.Hkv);
  const size_t hist_smem = (size_t)p.nkb * sizeof(int);
  if (a.mode == kModeSel) sel_hist_kernel<kModeSel><<<grid, kBlock, hist_smem, st>>>(R, counts);
  else if (a.mode == kModeSwa) sel_hist_kernel<kModeSwa><<<grid, kBlock, hist_smem, st>>>(R, counts);
  else sel_hist_kernel<kModeCmp><<<grid, kBlock, hist_smem, st>>>(R, counts);
  sel_scan_kernel<<<(p.nlists + 31) / 32, dim3(32, kScanSeg), 0, st>>>(counts, totals, p.nlists, p.nqb, p.nkb);
  sel_items_kernel<<<1, 1024, 0, st>>>(totals, list_base, items, num_items, p.nlists, p.QT, index_tag(a, p));
  if (a.mode == kModeSel) sel_fill_kernel<kModeSel><<<grid, kBlock, hist_smem, st>>>(R, counts, list_base, entries);
  else if (a.mode == kModeSwa) sel_fill_kernel<kModeSwa><<<grid, kBlock, hist_smem, st>>>(R, counts, list_base, entries);
  else sel_fill_kernel<kModeCmp><<<grid, kBlock, hist_smem, st>>>(R, counts, list_base, entries);
  CUDA_TRY(cudaGetLastError());
  count_launches(4);   // histogram, scan, items, fill
  return NSA_OK;
}

static void fill_params(SelParams& P, const SelProblem& a, const SelPlan& p, uint8_t* ws, const uint8_t* ix = nullptr) {
  if (ix == nullptr) ix = ws;   // the index lives in the work buffer unless the caller kept the forward's
  memset(&P, 0, sizeof(P));
  P.q = (const __nv_bfloat16*)a.q.ptr; P.q_sb = a.q.stride_b; P.q_sh = a.q.stride_h; P.q_sn = a.q.stride_n;
  P.out = (__nv_bfloat16*)a.out.ptr; P.o_sb = a.out.stride_b; P.o_sh = a.out.stride_h; P.o_sn = a.out.stride_n;
  P.idx = a.idx; P.mask = a.mask;
  P.entries = reinterpret_cast<const uint32_t*>(ix + p.off_entries);
  P.items = reinterpret_cast<const int4*>(ix + p.off_items);
  P.num_items = reinterpret_cast<const int*>(ix + p.off_num_items);
  P.index_tag = index_tag(a, p);
  P.status = reinterpret_cast<int*>(ws + p.off_status);
  P.lse = a.lse;
  P.B = a.B; P.Hq = a.Hq; P.Hkv = a.Hkv; P.N = a.N; P.Nk = a.Nk; P.G = p.G; P.nsel = a.nsel; P.nfb = p.nkb;
  P.ns = p.ns;
  P.diag = a.diag; P.scale = a.scale; P.scale_log2 = a.scale * kLog2e;
  P.rule = make_rule(a, p);
  P.importance = a.importance; P.ncb = a.ncb; P.round_bf16 = a.round_bf16;
  P.pooled = a.pooled; P.cpf = a.cpf > 0 ? a.cpf : 1; P.pool_cols = a.ncb / P.cpf; P.pool_block = P.cpf * a.stride;
}

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int D>
static int run_fwd(const SelProblem& a, const SelPlan& p, uint8_t* ws, cudaStream_t st) {
  CUtensorMap tmK, tmV;
  int rc = make_kv_map(&tmK, a.k, a.B, a.Hkv, a.Nk, D);
  if (rc != NSA_OK) return rc;
  rc = make_kv_map(&tmV, a.v, a.B, a.Hkv, a.Nk, D);
  if (rc != NSA_OK) return rc;
  if (dense_forward(a)) {
    CUDA_TRY(cudaMemsetAsync(ws + p.off_status, 0, 256, st));
    SelParams P;
    fill_params(P, a, p, ws);
    const int QT = kRows / p.G;
    const int64_t tiles = (int64_t)a.B * a.Hkv * ((a.N + QT - 1) / QT);
    if (tiles > 0x7fffffffLL) return NSA_ERR_UNSUPPORTED;
    const int smem = (D / 64) * 16384 + 16384 + 4 * (D / 64) * 8192;
#define NSA_DENSE_LAUNCH(MODE, GI)                                                                                   \
    do {                                                                                                              \
      CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<D, MODE, GI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
      CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<D, MODE, GI>, cudaFuncAttributePreferredSharedMemoryCarveout,    \
                                    cudaSharedmemCarveoutMaxShared));                                                 \
      dense_fwd_kernel<D, MODE, GI><<<(unsigned)tiles, 2 * kRows, smem, st>>>(tmK, tmV, P);                               \
    } while (0)
#define NSA_DENSE_LAUNCH_POOL(GI)                                                                                     \
    do {                                                                                                              \
      CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<D, kModeCmp, GI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
      CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<D, kModeCmp, GI, true>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                                    cudaSharedmemCarveoutMaxShared));                                                 \
      dense_fwd_kernel<D, kModeCmp, GI, true><<<(unsigned)tiles, 2 * kRows, smem, st>>>(tmK, tmV, P);                   \
    } while (0)
    if (a.mode == kModeSwa) NSA_DENSE_LAUNCH(kModeSwa, 0);
    else if (P.pooled != nullptr && p.G == 4) NSA_DENSE_LAUNCH_POOL(4);
    else if (P.pooled != nullptr && p.G == 8) NSA_DENSE_LAUNCH_POOL(8);
    else if (P.pooled != nullptr && p.G == 16) NSA_DENSE_LAUNCH_POOL(16);
    else if (P.pooled != nullptr) return NSA_ERR_UNSUPPORTED;
    else if (P.importance == nullptr) NSA_DENSE_LAUNCH(kModeCmp, 0);
    else if (p.G == 1) NSA_DENSE_LAUNCH(kModeCmp, 1);
    else if (p.G == 2) NSA_DENSE_LAUNCH(kModeCmp, 2);
    else if (p.G == 4) NSA_DENSE_LAUNCH(kModeCmp, 4);
    else if (p.G == 8) NSA_DENSE_LAUNCH(kModeCmp, 8);
    else NSA_DENSE_LAUNCH(kModeCmp, 16);
#undef NSA_DENSE_LAUNCH
#undef NSA_DENSE_LAUNCH_POOL
    CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return NSA_OK;
  }
  const uint8_t* ix = nullptr;
  if (a.index != nullptr) {   // the caller kept the index of an earlier forward over the same selection
    if (a.index_bytes != p.index_bytes) return fail(NSA_ERR_WORKSPACE, "index: not the size nsa_sel_index_bytes reports");
    ix = static_cast<const uint8_t*>(a.index);
    CUDA_TRY(cudaMemsetAsync(ws + p.off_status, 0, 256, st));
  } else {
    rc = build_index(a, p, ws, st);
    if (rc != NSA_OK) return rc;
  }
  SelParams P;
  fill_params(P, a, p, ws, ix);
  P.partial = reinterpret_cast<__nv_bfloat16*>(ws + p.off_partial);
  P.stats = reinterpret_cast<float2*>(ws + p.off_stats);
  // a slot that no list holds keeps (0, 0): the merge reads the statistics of every slot and skips those
  CUDA_TRY(cudaMemsetAsync(P.stats, 0, (size_t)a.B * a.Hq * a.N * p.ns * sizeof(float2), st));
  constexpr int NC = D / 64;
  const int smem = 1024 + NC * (16384 + 8192 + 8192) + kRows * (D * 2 + 16);
  const int per_sm = D == 64 ? 4 : 2;
  CUDA_TRY(cudaFuncSetAttribute(sel_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  sel_fwd_kernel<D><<<num_sms() * per_sm, 2 * kRows, smem, st>>>(tmK, tmV, P);
  const int64_t threads = (int64_t)a.B * a.Hq * a.N * (D / 8);
  const unsigned mblocks = (unsigned)((threads + 255) / 256);
  if (a.fuse_combine != nullptr) {
    if (a.fuse_targets->multicast) sel_merge_combine_kernel<D, true><<<mblocks, 256, 0, st>>>(P, *a.fuse_combine, *a.fuse_targets);
    else sel_merge_combine_kernel<D, false><<<mblocks, 256, 0, st>>>(P, *a.fuse_combine, *a.fuse_targets);
  } else {
    sel_merge_kernel<D><<<mblocks, 256, 0, st>>>(P);
  }
  CUDA_TRY(cudaGetLastError());
  count_launches(2);   // forward kernel, merge
  return NSA_OK;
}

template <int D>
static int run_bwd(const SelProblem& a, const SelPlan& p, uint8_t* ws, cudaStream_t st) {
  CUtensorMap tmK, tmV;
  int rc = make_kv_map(&tmK, a.k, a.B, a.Hkv, a.Nk, D);
  if (rc != NSA_OK) return rc;
  rc = make_kv_map(&tmV, a.v, a.B, a.Hkv, a.Nk, D);
  if (rc != NSA_OK) return rc;
  const uint8_t* ix = nullptr;
  if (a.index != nullptr) {
    if (a.index_bytes != p.index_bytes) return fail(NSA_ERR_WORKSPACE, "index: not the size nsa_sel_index_bytes reports");
    ix = static_cast<const uint8_t*>(a.index);
    CUDA_TRY(cudaMemsetAsync(ws + p.off_status, 0, 256, st));
  } else {
    rc = build_index(a, p, ws, st);
    if (rc != NSA_OK) return rc;
  }
  SelParams P;
  fill_params(P, a, p, ws, ix);
  P.dout = (const __nv_bfloat16*)a.dout.ptr; P.do_sb = a.dout.stride_b; P.do_sh = a.dout.stride_h; P.do_sn = a.dout.stride_n;
  float* delta = reinterpret_cast<float*>(ws + p.off_delta);
  P.delta = a.delta != nullptr ? a.delta : delta;
  P.dq = a.dq; P.dk = a.dk; P.dv = a.dv; P.slot_grads = a.slot_grads;
  if (a.dq_out.ptr != nullptr) {
    P.dq_lp = (__nv_bfloat16*)a.dq_out.ptr; P.dq_sb = a.dq_out.stride_b; P.dq_sh = a.dq_out.stride_h; P.dq_sn = a.dq_out.stride_n;
  }
  const int64_t threads = (int64_t)a.B * a.Hq * a.N * (D / 8);
  const int own_delta = a.delta == nullptr ? 1 : 0;   // the caller may hand the row sums over
  if (own_delta) sel_delta_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(P, delta);
  if (D == 64) {
    const int smem = 1024 + ws::kStages * 32768 + 2 * ws::kPBytes + 2 * 16384 + ws::kStages * ws::kMetaBytes +
                     8 * ws::kDqStage;
    CUDA_TRY(cudaFuncSetAttribute(sel_bwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    P.partial = reinterpret_cast<__nv_bfloat16*>(ws + p.off_partial);
    sel_bwd_ws_kernel<<<num_sms(), ws::kThreads, smem, st>>>(tmK, tmV, P);
    const unsigned mblocks = (unsigned)((threads + 255) / 256);
    if (a.mode == kModeSel) sel_dq_merge_kernel<64, kModeSel><<<mblocks, 256, 0, st>>>(P);
    else if (a.mode == kModeSwa) sel_dq_merge_kernel<64, kModeSwa><<<mblocks, 256, 0, st>>>(P);
    else sel_dq_merge_kernel<64, kModeCmp><<<mblocks, 256, 0, st>>>(P);
    CUDA_TRY(cudaGetLastError());
    count_launches(2 + own_delta);   // (delta,) backward kernel, dQ merge
    return NSA_OK;
  }
  constexpr int NC = D / 64;
  const int smem = 1024 + NC * (2 * 16384 + 2 * 8192) + kRows * (D * 4 + 16);
  const int per_sm = D == 64 ? 2 : 1;
  CUDA_TRY(cudaFuncSetAttribute(sel_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  sel_bwd_kernel<D><<<num_sms() * per_sm, kRows, smem, st>>>(tmK, tmV, P);
  CUDA_TRY(cudaGetLastError());
  count_launches(1 + own_delta);   // (delta,) backward kernel
  return NSA_OK;
}

// ---- the three branches as problems ------------------------------------------------------------

static void problem_base(SelProblem& x) { memset(&x, 0, sizeof(x)); x.stride = 1; }

static bool sel_problem(SelProblem& x, const nsa_sel_fwd_args& a) {
  problem_base(x);
  if (a.dtype != NSA_BF16 || a.block != kBlock || a.sel_heads != a.kv_heads || a.nsel > 254) return false;
  x.q = a.q; x.k = a.k; x.v = a.v; x.out = a.out; x.idx = a.idx; x.mask = a.mask; x.lse = a.lse;
  x.workspace = a.workspace; x.workspace_bytes = a.workspace_bytes;
  x.B = a.batch; x.Hq = a.q_heads; x.Hkv = a.kv_heads; x.N = a.seq; x.Nk = a.seq; x.D = a.dim_head;
  x.nsel = a.nsel; x.diag = a.diag; x.mode = kModeSel; x.scale = a.scale;
  return supported(x);
}

static bool swa_problem(SelProblem& x, const nsa_swa_fwd_args& a) {
  problem_base(x);
  if (a.dtype != NSA_BF16 || !a.causal) return false;
  x.q = a.q; x.k = a.k; x.v = a.v; x.out = a.out; x.lse = a.lse;
  x.workspace = a.workspace; x.workspace_bytes = a.workspace_bytes;
  x.B = a.batch; x.Hq = a.q_heads; x.Hkv = a.kv_heads; x.N = a.seq; x.Nk = a.seq; x.D = a.dim_head;
  x.mode = kModeSwa; x.window = a.window; x.scale = a.scale;
  return supported(x);
}

static bool cmp_problem(SelProblem& x, const nsa_cmp_fwd_args& a) {
  problem_base(x);
  if (a.dtype != NSA_BF16 || !a.causal || a.sel_heads != a.kv_heads) return false;
  x.q = a.q; x.k = a.ck; x.v = a.cv; x.out = a.out; x.lse = a.lse;
  x.workspace = a.workspace; x.workspace_bytes = a.workspace_bytes;
  x.B = a.batch; x.Hq = a.q_heads; x.Hkv = a.kv_heads; x.N = a.seq; x.Nk = a.num_mem + a.ncb; x.D = a.dim_head;
  x.mode = kModeCmp; x.stride = a.stride; x.num_mem = a.num_mem; x.ncb = a.ncb; x.round_bf16 = 1;
  x.importance = a.importance; x.scale = a.scale;
  x.pooled = static_cast<__nv_bfloat16*>(a.pooled); x.cpf = a.pool;
  return supported(x);
}

// The forward can average the importance over the selection blocks itself (`pooled`) when the ring of head means fits
// beside the row maxima in shared memory (128 / G queries x 128 columns of bf16: G >= 4) and every key block of 64
// columns completes a whole number of selection blocks' worth of columns (cpf a power of two).
bool sm100_cmp_fwd_pools(const nsa_cmp_fwd_args& a) {
  SelProblem x;
  if (a.impl == NSA_IMPL_SIMT || !cmp_problem(x, a) || !dense_forward_serves(x)) return false;
  const int G = x.Hq / x.Hkv;
  if (G != 4 && G != 8 && G != 16) return false;
  if (a.pool != 1 && a.pool != 2 && a.pool != 4 && a.pool != 8 && a.pool != 16) return false;
  return a.num_mem <= kBlock && a.ncb / a.pool >= 1;
}

static int check_ws(const SelProblem& x, const SelPlan& p, uint8_t** ws) {
  if (x.workspace == nullptr || x.workspace_bytes < p.total_bytes)
    return fail(NSA_ERR_WORKSPACE, "work buffer missing or smaller than the matching *_workspace_bytes says");
  *ws = static_cast<uint8_t*>(x.workspace);
  if (reinterpret_cast<uintptr_t>(*ws) & 255) return fail(NSA_ERR_ALIGN, "work buffer must be 256-byte aligned");
  return NSA_OK;
}

static int problem_fwd(const SelProblem& x, cudaStream_t st) {
  const SelPlan p = make_plan(x, false);
  uint8_t* ws = nullptr;
  const int rc = check_ws(x, p, &ws);
  if (rc != NSA_OK) return rc;
  return x.D == 64 ? run_fwd<64>(x, p, ws, st) : run_fwd<128>(x, p, ws, st);
}

static int problem_bwd(const SelProblem& x, cudaStream_t st) {
  // dq in the caller's dtype and strides: only the merge of the partials writes whole rows of dq
  if (x.dq_out.ptr != nullptr && !(x.D == 64)) return NSA_ERR_UNSUPPORTED;
  const SelPlan p = make_plan(x, true);
  uint8_t* ws = nullptr;
  const int rc = check_ws(x, p, &ws);
  if (rc != NSA_OK) return rc;
  return x.D == 64 ? run_bwd<64>(x, p, ws, st) : run_bwd<128>(x, p, ws, st);
}

int64_t sm100_sel_workspace_bytes(const nsa_sel_fwd_args& a, bool backward) {
  SelProblem x;
  if (!sel_problem(x, a)) return NSA_ERR_UNSUPPORTED;
  return make_plan(x, backward).total_bytes;
}
int64_t sm100_sel_index_bytes(const nsa_sel_fwd_args& a) {
  SelProblem x;
  if (!sel_problem(x, a)) return 0;
  return make_plan(x, false).index_bytes;
}
int sm100_sel_fwd(const nsa_sel_fwd_args& a, cudaStream_t st) {
  SelProblem x;
  if (!sel_problem(x, a)) return NSA_ERR_UNSUPPORTED;
  x.index = a.index; x.index_bytes = a.index_bytes;
  return problem_fwd(x, st);
}
int sm100_sel_fwd_combine(const nsa_sel_fwd_args& a, const CombineParams& c, const GatherTargets& t, cudaStream_t st) {
  SelProblem x;
  if (!sel_problem(x, a)) return NSA_ERR_UNSUPPORTED;
  if (c.batch != x.B || c.q_heads != x.Hq || c.seq != x.N || c.d != x.D) return NSA_ERR_UNSUPPORTED;
  x.index = a.index; x.index_bytes = a.index_bytes;
  x.fuse_combine = &c; x.fuse_targets = &t;
  return problem_fwd(x, st);
}
int sm100_sel_bwd(const nsa_sel_bwd_args& b, cudaStream_t st) {
  SelProblem x;
  if (!sel_problem(x, b.fwd)) return NSA_ERR_UNSUPPORTED;
  x.dout = b.dout; x.dq = b.dq; x.dk = b.dk; x.dv = b.dv; x.slot_grads = b.slot_grads;
  x.index = b.index; x.index_bytes = b.index_bytes; x.dq_out = b.dq_out; x.delta = b.delta;
  return problem_bwd(x, st);
}

// True when the backward of this problem stores every row of dq (partials + ordered merge) instead of adding into it.
bool sm100_sel_bwd_overwrites_dq(const nsa_sel_fwd_args& a) {
  SelProblem x;
  return sel_problem(x, a) && x.D == 64;
}
bool sm100_swa_bwd_overwrites_dq(const nsa_swa_fwd_args& a) {
  SelProblem x;
  return swa_problem(x, a) && x.D == 64;
}
bool sm100_cmp_bwd_overwrites_dq(const nsa_cmp_fwd_args& a) {
  SelProblem x;
  return cmp_problem(x, a) && x.D == 64;
}

// The index of the sliding and the compressed backward depends on the sizes only: a caller may keep it across calls.
int64_t sm100_swa_index_bytes(const nsa_swa_fwd_args& a) {
  SelProblem x;
  if (!swa_problem(x, a)) return 0;
  return make_plan(x, true).index_bytes;
}
int64_t sm100_cmp_index_bytes(const nsa_cmp_fwd_args& a) {
  SelProblem x;
  if (!cmp_problem(x, a)) return 0;
  x.importance = nullptr;
  return make_plan(x, true).index_bytes;
}

int64_t sm100_swa_workspace_bytes(const nsa_swa_fwd_args& a, bool backward) {
  SelProblem x;
  if (!swa_problem(x, a)) return NSA_ERR_UNSUPPORTED;
  return make_plan(x, backward).total_bytes;
}
int sm100_swa_fwd(const nsa_swa_fwd_args& a, cudaStream_t st) {
  SelProblem x;
  if (!swa_problem(x, a) || !dense_forward_serves(x)) return NSA_ERR_UNSUPPORTED;
  return problem_fwd(x, st);
}
int sm100_swa_bwd(const nsa_swa_bwd_args& b, cudaStream_t st) {
  SelProblem x;
  if (!swa_problem(x, b.fwd)) return NSA_ERR_UNSUPPORTED;
  x.dout = b.dout; x.dq = b.dq; x.dk = b.dk; x.dv = b.dv; x.dq_out = b.dq_out;
  x.index = b.index; x.index_bytes = b.index_bytes; x.delta = b.delta;
  return problem_bwd(x, st);
}

int64_t sm100_cmp_workspace_bytes(const nsa_cmp_fwd_args& a, bool backward) {
  SelProblem x;
  if (!cmp_problem(x, a)) return NSA_ERR_UNSUPPORTED;
  return make_plan(x, backward).total_bytes;
}
int sm100_cmp_fwd(const nsa_cmp_fwd_args& a, cudaStream_t st) {
  SelProblem x;
  if (!cmp_problem(x, a) || !dense_forward_serves(x)) return NSA_ERR_UNSUPPORTED;
  if (x.pooled != nullptr) {
    if (!sm100_cmp_fwd_pools(a)) return NSA_ERR_UNSUPPORTED;
    x.importance = nullptr;
  }
  if (x.importance != nullptr) {
    // columns a query cannot see carry the head mean of the sentinel; the kernel overwrites the visible ones
    float fill = 0.f;
    const int G = x.Hq / x.Hkv;
    for (int g = 0; g < G; ++g) fill += a.sentinel;
    fill = __bfloat162float(__float2bfloat16_rn(fill / (float)G));
    const int64_t count = (int64_t)x.B * x.Hkv * x.N * x.ncb;
    const int64_t rows = (int64_t)x.B * x.Hkv * x.N;
    if (x.ncb % 4 == 0 && (reinterpret_cast<uintptr_t>(x.importance) & 15u) == 0 && rows > 0) {
      const int64_t slices = (int64_t)x.B * x.Hkv;
      const int64_t blocks = (slices * ((x.N + 1) / 2) + 7) / 8;
      fill_invisible_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(x.importance, fill, slices, x.N,
                                                                                              x.ncb, x.stride);
    } else {
      fill_kernel<<<(unsigned)((count + 1023) / 1024 < 148 * 16 ? (count + 1023) / 1024 : 148 * 16), 256, 0, st>>>(x.importance, fill, count);
    }
    count_launches(1);
  }
  return problem_fwd(x, st);
}
int sm100_cmp_bwd(const nsa_cmp_bwd_args& b, cudaStream_t st) {
  SelProblem x;
  if (!cmp_problem(x, b.fwd)) return NSA_ERR_UNSUPPORTED;
  x.importance = nullptr;
  x.pooled = nullptr;
  x.dout = b.dout; x.dq = b.dq; x.dk = b.dck; x.dv = b.dcv; x.dq_out = b.dq_out;
  x.index = b.index; x.index_bytes = b.index_bytes; x.delta = b.delta;
  return problem_bwd(x, st);
}

// ---- forward without a caller-provided work buffer ---------------------------------------------
//
// Some callers cannot hand over device memory for the work buffer: code that runs where the CUDA
// allocator must not be entered (a serving loop holding an allocator lock, a plug-in host whose
// memory pool is closed to extensions, an embedder that forbids cudaMalloc after start-up).  For
// them the forward pass can run on a fixed scratch area that is part of the library image.  Every
// device that loads the library reserves kStaticScratchBytes for it until the process ends.
constexpr int64_t kStaticScratchBytes = 32ll << 20;
static __device__ __align__(256) unsigned char g_sel_scratch[kStaticScratchBytes];

// Filled on first use per device without a lock: every thread that races here stores the same address.
constexpr int kMaxDevices = 64;
static unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

// The device address of the scratch array for the current device.  In host code the array's name
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
static int static_scratch(unsigned char** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(NSA_ERR_UNSUPPORTED, "device ordinal beyond the scratch table");
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_sel_scratch));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return NSA_OK;
}

int sm100_sel_fwd_static(const nsa_sel_fwd_args& a, cudaStream_t st) {
  SelProblem x;
  if (!sel_problem(x, a)) return fail(NSA_ERR_UNSUPPORTED, "nsa_sel_fwd_static: shape outside the tensor-core family (bf16, block 64, dim_head 64/128, shared selection, own block included)");
  const SelPlan p = make_plan(x, false);
  if (p.total_bytes > kStaticScratchBytes) {
    static thread_local char msg[160];
    snprintf(msg, sizeof(msg), "nsa_sel_fwd_static: this problem needs %lld bytes of scratch, the built-in area holds %lld",
             (long long)p.total_bytes, (long long)kStaticScratchBytes);
    return fail(NSA_ERR_WORKSPACE, msg);
  }
  unsigned char* ws = nullptr;
  const int rc = static_scratch(&ws);
  if (rc != NSA_OK) return rc;
  return x.D == 64 ? run_fwd<64>(x, p, ws, st) : run_fwd<128>(x, p, ws, st);
}

int64_t sm100_static_scratch_bytes() { return kStaticScratchBytes; }

// The status word the kernels of the last nsa_sel_fwd_static call on this device left in the built-in area (its
// first four bytes): copied to `out`, host or device memory, in stream order.  Nothing is allocated.
int sm100_sel_static_status(int* out, cudaStream_t st) {
  if (out == nullptr) return fail(NSA_ERR_NULL, "nsa_sel_static_status: NULL output pointer");
  unsigned char* ws = nullptr;
  const int rc = static_scratch(&ws);
  if (rc != NSA_OK) return rc;
  CUDA_TRY(cudaMemcpyAsync(out, ws, sizeof(int), cudaMemcpyDefault, st));
  return NSA_OK;
}

// ---- self-test of the bounded waits ----------------------------------------------------------------
//
// One block that does what every tensor-core kernel here does around a wait -- allocates tensor memory, waits on an
// mbarrier with a limit, and on giving up raises its abort flag, frees the tensor memory and reports status 1 -- except
// that nobody ever arrives on its barrier and the limit is `limit_cycles` (about a millisecond in the test) instead of
// a second.  It returns by itself; nothing traps, faults or spins without a bound.
__global__ void __launch_bounds__(128) wait_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_slot;
  mbar_wait_warp(smem_u32(&bar), 0, &abort_flag, limit_cycles);   // nobody arrives: every warp runs into the limit
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 32);
  if (tid == 0 && abort_flag) atomicExch(status, 1);
}

int sm100_wait_selftest(int* status_device, int64_t limit_cycles, cudaStream_t st) {
  if (status_device == nullptr) return fail(NSA_ERR_NULL, "nsa_selftest_bounded_wait: NULL status pointer");
  if (limit_cycles < 1 || limit_cycles > kWaitLimitCycles) return fail(NSA_ERR_SHAPE, "nsa_selftest_bounded_wait: limit out of range");
  CUDA_TRY(cudaMemsetAsync(status_device, 0, sizeof(int), st));
  wait_selftest_kernel<<<1, 128, 0, st>>>(status_device, (long long)limit_cycles);
  CUDA_TRY(cudaGetLastError());
  count_launches(1);
  return NSA_OK;
}

}  // namespace nsa
