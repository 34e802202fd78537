// One decoding step of the NSA hot path in a single launch: for the newest token, compressed attention over the
// blocks compressed so far (with its per-block logits), block selection, attention over the selected blocks plus the
// part of the own block that exists, sliding window, and the gated combine into the merged row.
//
// One CTA of eight warps serves one (batch element, KV head) and the G query heads of that head together, so every
// key / value row is fetched once for the group.  All arithmetic is fp32.  Inside a branch the warps take tiles of 32
// consecutive keys in turn (lanes map to keys for the dot products and to feature pairs for the accumulation, as in
// the generic attention kernels), keep an online softmax each, and fold their results through shared memory.

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

constexpr int kDecodeWarps = 8;

template <typename T, int GT>
struct WarpSoftmax {
  float m[GT], l[GT], acc[GT][2][2];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
      acc[g][0][0] = acc[g][0][1] = acc[g][1][0] = acc[g][1][1] = 0.f;
    }
  }

  // Up to 32 consecutive key rows: rows t0 .. t0+cnt-1 of kb / vb.  `rows` holds the G query rows as fp32.  On return
  // logit[g] is this lane's scaled logit (lane < cnt).
  __device__ __forceinline__ void tile(const float* rows, const T* kb, int64_t k_sn, const T* vb, int64_t v_sn, int t0,
                                       int cnt, int d, float scale, int lane, float (&logit)[GT]) {
    constexpr int V = Elem<T>::kVec;
    const bool present = lane < cnt;
#pragma unroll
    for (int g = 0; g < GT; ++g) logit[g] = 0.f;
    if (present) {
      const T* key = kb + (int64_t)(t0 + lane) * k_sn;
      for (int c = 0; c < d; c += V) {
        float kv[V];
        Elem<T>::load_vec(key + c, kv);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
#pragma unroll
          for (int e = 0; e < V; ++e) logit[g] = fmaf(rows[g * d + c + e], kv[e], logit[g]);
        }
      }
    }
    float p[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      logit[g] *= scale;
      const float tile_max = warp_max(present ? logit[g] : -INFINITY);
      const float m_new = fmaxf(m[g], tile_max);
      const float alpha = exp2f((m[g] - m_new) * kLog2e);
      p[g] = present ? exp2f((logit[g] - m_new) * kLog2e) : 0.f;
      l[g] = l[g] * alpha + warp_sum(p[g]);
      m[g] = m_new;
      acc[g][0][0] *= alpha; acc[g][0][1] *= alpha;
      acc[g][1][0] *= alpha; acc[g][1][1] *= alpha;
    }
    for (int kk = 0; kk < cnt; ++kk) {
      const T* vrow = vb + (int64_t)(t0 + kk) * v_sn;
      float2 vv[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int dim = 64 * c + 2 * lane;
        vv[c] = dim < d ? Elem<T>::load2(vrow + dim) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float pg = __shfl_sync(kFullMask, p[g], kk);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          acc[g][c][0] = fmaf(pg, vv[c].x, acc[g][c][0]);
          acc[g][c][1] = fmaf(pg, vv[c].y, acc[g][c][1]);
        }
      }
    }
  }

  // This warp's state to shared memory: [warp][g][2 + d]
  __device__ __forceinline__ void park(float* area, int warp, int d, int lane) const {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float* dst = area + ((size_t)warp * GT + g) * (d + 2);
      if (lane == 0) { dst[0] = m[g]; dst[1] = l[g]; }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int dim = 64 * c + 2 * lane;
        if (dim < d) { dst[2 + dim] = acc[g][c][0]; dst[3 + dim] = acc[g][c][1]; }
      }
    }
  }
};

// Folds the eight warps' parked states into normalised outputs out[g][c] (G heads, d columns); all threads take part.
__device__ __forceinline__ void fold_warps(const float* area, float* out, int GT, int G, int d, int tid, int nthreads) {
  for (int e = tid; e < G * d; e += nthreads) {
    const int g = e / d, c = e - g * d;
    float M = -INFINITY;
    for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, area[((size_t)w * GT + g) * (d + 2)]);
    float L = 0.f, O = 0.f;
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float* src = area + ((size_t)w * GT + g) * (d + 2);
      const float f = src[0] == -INFINITY ? 0.f : exp2f((src[0] - M) * kLog2e);
      L = fmaf(f, src[1], L);
      O = fmaf(f, src[2 + c], O);
    }
    out[e] = L > 0.f ? O / L : 0.f;
  }
}

template <typename T, int GT>
__global__ void __launch_bounds__(kDecodeWarps * 32) decode_kernel(const DecodeParams P) {
  extern __shared__ __align__(16) float smem[];
  __shared__ int sel_idx[32];
  __shared__ int sel_count;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.x % P.kv_heads, b = blockIdx.x / P.kv_heads;
  const int G = P.q_heads / P.kv_heads, d = P.d;
  const int cpf = P.block / P.stride;
  const int cols = P.stride != P.block ? P.ncb / cpf : P.ncb;

  float* q_s = smem;                                  // un-rotated queries of the group [GT][d]
  float* qr_s = q_s + GT * d;                         // rotated queries
  float* o_s = qr_s + GT * d;                         // branch outputs [3][GT][d]
  float* area = o_s + 3 * GT * d;                     // parked warp states [8][GT][d + 2]
  float* imp_s = area + kDecodeWarps * GT * (d + 2);  // head-mean logit of every compressed block [ncb]
  float* prob_s = imp_s + P.ncb;                      // block probabilities [cols]

  for (int e = tid; e < GT * d; e += blockDim.x) {
    const int g = e / d, c = e - g * d;
    const int64_t at = ((int64_t)b * P.q_heads + kvh * G + g) * d + c;
    q_s[e] = g < G ? Elem<T>::to_float(((const T*)P.q)[at]) : 0.f;
    qr_s[e] = g < G ? Elem<T>::to_float(((const T*)P.qr)[at]) : 0.f;
  }
  __syncthreads();

  WarpSoftmax<T, GT> W;
  float logit[GT];

  // ---- 1. compressed branch: the memory slots, then every compressed block; head-mean logits kept for the selection
  if (P.ncb > 0) {
    W.init();
    const T* mk = (const T*)P.mem_k + (int64_t)kvh * P.num_mem * d;
    const T* mv = (const T*)P.mem_v + (int64_t)kvh * P.num_mem * d;
    const T* ck = (const T*)P.ck + b * P.ck_sb + (int64_t)kvh * P.ck_sh;
    const T* cv = (const T*)P.cv + b * P.cv_sb + (int64_t)kvh * P.cv_sh;
    const int mem_tiles = (P.num_mem + 31) / 32, blk_tiles = (P.ncb + 31) / 32;
    for (int t = warp; t < mem_tiles + blk_tiles; t += kDecodeWarps) {
      if (t < mem_tiles) {
        W.tile(q_s, mk, d, mv, d, t * 32, min(32, P.num_mem - t * 32), d, P.scale, lane, logit);
      } else {
        const int t0 = (t - mem_tiles) * 32, cnt = min(32, P.ncb - t0);
        W.tile(q_s, ck, P.ck_sn, cv, P.cv_sn, t0, cnt, d, P.scale, lane, logit);
        if (lane < cnt) {
          float sum = 0.f;
#pragma unroll
          for (int g = 0; g < GT; ++g) sum += g < G ? logit[g] : 0.f;
          imp_s[t0 + lane] = sum / (float)G;
        }
      }
    }
    W.park(area, warp, d, lane);
    __syncthreads();
    fold_warps(area, o_s, GT, G, d, tid, blockDim.x);
  } else {
    for (int e = tid; e < GT * d; e += blockDim.x) o_s[e] = 0.f;
  }
  __syncthreads();

  // ---- 2. selection (warp 0): mean over the compressed blocks of a selection block, sink softmax, ordered top-k
  const int k_sel = min(min(P.nsel, cols), 32);
  if (warp == 0) {
    float mx = -1000.f;   // the sink logit
    for (int j = lane; j < cols; j += 32) {
      float x;
      if (P.stride != P.block) {
        float sum = 0.f;
        for (int c = 0; c < cpf; ++c) sum += imp_s[j * cpf + c];
        x = sum / (float)cpf;
      } else {
        x = imp_s[j];
      }
      prob_s[j] = x;
      mx = fmaxf(mx, x);
    }
    mx = warp_max(mx);
    __syncwarp();
    float part = 0.f;
    for (int j = lane; j < cols; j += 32) {
      const float e = expf(prob_s[j] - mx);
      prob_s[j] = e;
      part += e;
    }
    const float z = warp_sum(part) + expf(-1000.f - mx);
    __syncwarp();
    float prev_v = INFINITY;
    int prev_i = -1, count = 0;
    for (int r = 0; r < k_sel; ++r) {
      float best_v = -INFINITY;
      int best_i = 0x7fffffff;
      for (int j = lane; j < cols; j += 32) {
        const float v = prob_s[j] / z;
        const bool eligible = v < prev_v || (v == prev_v && j > prev_i);
        if (eligible && (v > best_v || (v == best_v && j < best_i))) { best_v = v; best_i = j; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(kFullMask, best_v, o);
        const int oi = __shfl_xor_sync(kFullMask, best_i, o);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
      }
      if (best_i == 0x7fffffff) break;
      if (best_v > 1e-10f) {          // slots at or below the threshold are masked out upstream
        if (lane == 0) sel_idx[count] = best_i;
        ++count;
      }
      prev_v = best_v;
      prev_i = best_i;
    }
    if (lane == 0) sel_count = count;
  }
  __syncthreads();

  const T* kb = (const T*)P.keys + b * P.k_sb + (int64_t)kvh * P.k_sh;
  const T* vb = (const T*)P.vals + b * P.v_sb + (int64_t)kvh * P.v_sh;
  const int pos = P.T - 1;

  // ---- 3. selected blocks (whole blocks of `block` keys) and the own block up to the token
  {
    W.init();
    const int tiles_per_block = (P.block + 31) / 32;
    const int own0 = pos / P.block * P.block, own_tiles = (pos - own0 + 1 + 31) / 32;
    const int total = sel_count * tiles_per_block + own_tiles;
    for (int t = warp; t < total; t += kDecodeWarps) {
      int t0, cnt;
      if (t < sel_count * tiles_per_block) {
        const int s = t / tiles_per_block, part = t - s * tiles_per_block;
        t0 = sel_idx[s] * P.block + part * 32;
        cnt = min(32, P.block - part * 32);
        cnt = min(cnt, P.T - t0);          // (a selected block lies wholly in the past; kept as a guard)
      } else {
        t0 = own0 + (t - sel_count * tiles_per_block) * 32;
        cnt = min(32, pos + 1 - t0);
      }
      if (cnt > 0) W.tile(qr_s, kb, P.k_sn, vb, P.v_sn, t0, cnt, d, P.scale, lane, logit);
    }
    W.park(area, warp, d, lane);
    __syncthreads();
    fold_warps(area, o_s + GT * d, GT, G, d, tid, blockDim.x);
    __syncthreads();
  }

  // ---- 4. sliding window: the last window + 1 keys
  {
    W.init();
    const int first = max(0, pos - P.window);
    const int total = (pos + 1 - first + 31) / 32;
    for (int t = warp; t < total; t += kDecodeWarps) {
      const int t0 = first + t * 32;
      W.tile(qr_s, kb, P.k_sn, vb, P.v_sn, t0, min(32, pos + 1 - t0), d, P.scale, lane, logit);
    }
    W.park(area, warp, d, lane);
    __syncthreads();
    fold_warps(area, o_s + 2 * GT * d, GT, G, d, tid, blockDim.x);
    __syncthreads();
  }

  // ---- 5. gated combine into the merged row [B, Hq * d]
  for (int e = tid; e < G * d; e += blockDim.x) {
    const int g = e / d;
    const T* gate = (const T*)P.gates + ((int64_t)b * P.q_heads + kvh * G + g) * 3;
    const float v = Elem<T>::to_float(gate[0]) * o_s[e] + Elem<T>::to_float(gate[1]) * o_s[GT * d + e] +
                    Elem<T>::to_float(gate[2]) * o_s[2 * GT * d + e];
    ((T*)P.out)[((int64_t)b * P.q_heads + kvh * G) * d + e] = Elem<T>::from_float(v);
  }
}

template <typename T, int GT>
static int launch_decode_gt(const DecodeParams& P, cudaStream_t stream) {
  const int cpf = P.block / P.stride;
  const int cols = P.stride != P.block ? P.ncb / cpf : P.ncb;
  const size_t floats = (size_t)5 * GT * P.d + (size_t)kDecodeWarps * GT * (P.d + 2) + (size_t)P.ncb + (size_t)cols;
  const size_t smem = floats * sizeof(float);
  if (smem > 200 * 1024) return fail(NSA_ERR_UNSUPPORTED, "decode step: too many compressed blocks for one CTA's shared memory");
  auto kern = decode_kernel<T, GT>;
  cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  kern<<<(unsigned)(P.batch * P.kv_heads), kDecodeWarps * 32, smem, stream>>>(P);
  count_launches(1);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

template <typename T>
static int launch_decode_t(const DecodeParams& P, cudaStream_t stream) {
  const int G = P.q_heads / P.kv_heads;
  if (G == 1) return launch_decode_gt<T, 1>(P, stream);
  if (G == 2) return launch_decode_gt<T, 2>(P, stream);
  if (G <= 4) return launch_decode_gt<T, 4>(P, stream);
  if (G <= 8) return launch_decode_gt<T, 8>(P, stream);
  if (G <= 16) return launch_decode_gt<T, 16>(P, stream);
  return fail(NSA_ERR_UNSUPPORTED, "decode step: more than 16 query heads per KV head");
}

int launch_decode(const DecodeParams& P, int dtype, cudaStream_t stream) {
  if (P.batch == 0) return NSA_OK;
  return dtype == NSA_F32 ? launch_decode_t<float>(P, stream) : launch_decode_t<__nv_bfloat16>(P, stream);
}

}  // namespace nsa
