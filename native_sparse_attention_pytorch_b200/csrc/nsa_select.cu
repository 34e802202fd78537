// Block selection: per-block mean of the importance columns, own-block
// exclusion, softmax with a sink logit, and an ordered top-k -- one warp per
// query row.  Integer output; ties are broken towards the lower column index
// so the result is a pure function of the scores.

#include <limits.h>

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

__global__ void __launch_bounds__(128) select_kernel(const SelectParams P, int warps_per_block) {
  extern __shared__ float sbuf[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t task = (int64_t)blockIdx.x * warps_per_block + warp;
  if (warp >= warps_per_block || task >= (int64_t)P.rows * P.seq) return;
  const int i = (int)(task % P.seq);
  float* buf = sbuf + (size_t)warp * P.cols;
  const float* src = P.imp + task * P.ncb;
  const __nv_bfloat16* psrc = static_cast<const __nv_bfloat16*>(P.pooled) + task * P.ncb;
  const int limit = P.causal_limit ? min(P.cols, i / P.block) : P.cols;

  for (int j = lane; j < P.cols; j += 32) {
    float v;
    if (j >= limit) {
      v = P.neg_max;
    } else if (P.pooled != nullptr) {
      v = __bfloat162float(psrc[j]);
    } else if (P.cpf == 1) {
      v = src[j];
    } else {
      float sum = 0.f;
      for (int c = 0; c < P.cpf; ++c) sum += src[j * P.cpf + c];
      v = sum / (float)P.cpf;
      if (P.round_bf16) v = round_bf16(v);
    }
    if (!P.input_is_prob && P.exclude_own && j == i / P.block) v = P.neg_max;
    buf[j] = v;
  }
  __syncwarp();

  if (!P.input_is_prob) {
    float mx = -1000.f;  // the sink logit
    for (int j = lane; j < P.cols; j += 32) mx = fmaxf(mx, buf[j]);
    mx = warp_max(mx);
    float part = 0.f;
    for (int j = lane; j < P.cols; j += 32) {
      const float e = expf(buf[j] - mx);
      buf[j] = e;
      part += e;
    }
    const float z = warp_sum(part) + expf(-1000.f - mx);
    for (int j = lane; j < P.cols; j += 32) {
      float p = buf[j] / z;
      if (P.round_bf16) p = round_bf16(p);
      buf[j] = p;
    }
    __syncwarp();
  }

  // k rounds of "largest entry after the previous pick" in (value desc, index asc) order
  float prev_v = INFINITY;
  int prev_i = -1;
  for (int r = 0; r < P.k; ++r) {
    float best_v = -INFINITY;
    int best_i = INT_MAX;
    for (int j = lane; j < P.cols; j += 32) {
      const float v = buf[j];
      const bool eligible = v < prev_v || (v == prev_v && j > prev_i);
      if (eligible && (v > best_v || (v == best_v && j < best_i))) {
        best_v = v;
        best_i = j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(kFullMask, best_v, o);
      const int oi = __shfl_xor_sync(kFullMask, best_i, o);
      if (ov > best_v || (ov == best_v && oi < best_i)) {
        best_v = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      P.idx[task * P.k + r] = best_i == INT_MAX ? 0 : best_i;
      P.vals[task * P.k + r] = best_i == INT_MAX ? 0.f : best_v;
    }
    prev_v = best_v;
    prev_i = best_i;
  }
}

// The same selection with the row in registers: lane l holds columns l, l+32, ... (CPL of them), the arithmetic and its
// order are those of select_kernel (so both pick the same blocks), but every top-k round is a scan of the lane's own
// live entries, one warp-wide maximum over order-preserving integer keys and one warp-wide minimum over the column
// indices of the lanes that hold that maximum; the k results are written by k lanes at the end.  With bf16-rounded
// probabilities value and column share one word and a round is a single maximum over per-lane sorted lists.
__device__ __forceinline__ unsigned ordered_bits(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// `limit`: columns at and past it are not read, they hold probability 0 (causal_limit); `need`: columns that can
// appear among the k picks (all of them, or with a limit the first limit + k: zeros are picked in column order).
template <int CPL>
__device__ __forceinline__ void select_row(const SelectParams& P, int64_t task, int i, int lane, int limit, int need) {
  const float* src = P.imp + task * P.ncb;
  const __nv_bfloat16* psrc = static_cast<const __nv_bfloat16*>(P.pooled) + task * P.ncb;
  const bool vec4 = P.cpf == 4 && (P.ncb & 3) == 0 && (reinterpret_cast<uintptr_t>(P.imp) & 15u) == 0;
  float v[CPL];
  unsigned alive = 0;
#pragma unroll
  for (int t = 0; t < CPL; ++t) {
    const int j = lane + 32 * t;
    v[t] = 0.f;
    if (j < need) {
      alive |= 1u << t;
      float x;
      if (j >= limit) {
        x = P.neg_max;
      } else if (P.pooled != nullptr) {
        x = __bfloat162float(psrc[j]);
      } else if (P.cpf == 1) {
        x = src[j];
      } else {
        float sum = 0.f;
        if (vec4) {
          const float4 q = *reinterpret_cast<const float4*>(src + j * 4);
          sum = ((sum + q.x) + q.y) + q.z + q.w;
        } else {
          for (int c = 0; c < P.cpf; ++c) sum += src[j * P.cpf + c];
        }
        x = sum / (float)P.cpf;
        if (P.round_bf16) x = round_bf16(x);
      }
      if (!P.input_is_prob && P.exclude_own && j == i / P.block) x = P.neg_max;
      v[t] = x;
    }
  }
  if (!P.input_is_prob) {
    float mx = -1000.f;  // the sink logit
#pragma unroll
    for (int t = 0; t < CPL; ++t)
      if (alive >> t & 1) mx = fmaxf(mx, v[t]);
    mx = warp_max(mx);
    float part = 0.f;
#pragma unroll
    for (int t = 0; t < CPL; ++t) {
      if (alive >> t & 1) {
        v[t] = expf(v[t] - mx);
        part += v[t];
      }
    }
    const float z = warp_sum(part) + expf(-1000.f - mx);
#pragma unroll
    for (int t = 0; t < CPL; ++t) {
      if (alive >> t & 1) {
        float p = v[t] / z;
        if (P.round_bf16) p = round_bf16(p);
        v[t] = p;
      }
    }
  }
  int my_idx = 0;        // lane r ends up with the r-th pick
  float my_val = 0.f;
  if (P.round_bf16 && !P.input_is_prob) {
    // The probabilities were rounded to bf16, so the order-preserving key has 16 significant bits and fits one word
    // together with the column: (key << 16) | (1023 - column) is unique per entry and its maximum is the largest
    // value at the lowest column.  Each lane sorts its own entries once (bitonic network in registers); a round is
    // then one warp-wide maximum over the lanes' heads, and the lane that held it shifts its list.
    unsigned s[CPL];
#pragma unroll
    for (int t = 0; t < CPL; ++t)
      s[t] = (alive >> t & 1) ? ((ordered_bits(v[t]) & 0xffff0000u) | (1023u - (unsigned)(lane + 32 * t))) : 0u;
#pragma unroll
    for (int k = 2; k <= CPL; k <<= 1) {
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
        for (int a = 0; a < CPL; ++a) {
          const int b = a ^ j;
          if (b > a) {
            const unsigned hi = max(s[a], s[b]), lo = min(s[a], s[b]);
            if ((a & k) == 0) { s[a] = hi; s[b] = lo; } else { s[a] = lo; s[b] = hi; }   // descending overall
          }
        }
      }
    }
    for (int r = 0; r < P.k; ++r) {
      const unsigned top = __reduce_max_sync(kFullMask, s[0]);
      if (top == 0u) break;                       // fewer live entries than picks: the rest stay (0, 0.0)
      if (lane == r) {
        my_idx = (int)(1023u - (top & 1023u));
        const unsigned key = (top & 0xffff0000u) | ((top & 0x80000000u) ? 0u : 0xffffu);
        my_val = from_ordered_bits(key);
      }
      if (s[0] == top) {
#pragma unroll
        for (int t = 0; t + 1 < CPL; ++t) s[t] = s[t + 1];
        s[CPL - 1] = 0u;
      }
    }
    if (lane < P.k) {
      P.idx[task * P.k + lane] = my_idx;
      P.vals[task * P.k + lane] = my_val;
    }
    return;
  }
  unsigned key[CPL];
#pragma unroll
  for (int t = 0; t < CPL; ++t) key[t] = ordered_bits(v[t]);

  for (int r = 0; r < P.k; ++r) {
    unsigned best = 0;
    int best_t = -1;
#pragma unroll
    for (int t = 0; t < CPL; ++t) {
      if ((alive >> t & 1) && (best_t < 0 || key[t] > best)) {   // strict: the lower column wins a tie
        best = key[t];
        best_t = t;
      }
    }
    const unsigned top = __reduce_max_sync(kFullMask, best_t >= 0 ? best : 0u);
    const unsigned cand = (best_t >= 0 && best == top) ? (unsigned)(lane + 32 * best_t) : 0xffffffffu;
    const unsigned win = __reduce_min_sync(kFullMask, cand);
    if (win != 0xffffffffu) {
      if ((int)(win & 31u) == lane) alive &= ~(1u << (win >> 5));
      if (lane == r) {
        my_idx = (int)win;
        my_val = from_ordered_bits(top);
      }
    }
  }
  if (lane < P.k) {
    P.idx[task * P.k + lane] = my_idx;
    P.vals[task * P.k + lane] = my_val;
  }
}

// One warp per query row; the row takes the smallest register variant that holds the columns it needs (with a causal
// limit the early queries of a sequence need few).
template <int CPLMAX>
__global__ void __launch_bounds__(128) select_reg_kernel(const SelectParams P) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t task = (int64_t)blockIdx.x * 4 + warp;
  if (task >= (int64_t)P.rows * P.seq) return;
  const int i = (int)(task % P.seq);
  const int limit = P.causal_limit ? min(P.cols, i / P.block) : P.cols;
  const int need = P.causal_limit ? min(P.cols, limit + P.k) : P.cols;
  if (CPLMAX > 1 && need <= 32) select_row<1>(P, task, i, lane, limit, need);
  else if (CPLMAX > 2 && need <= 64) select_row<2>(P, task, i, lane, limit, need);
  else if (CPLMAX > 4 && need <= 128) select_row<4>(P, task, i, lane, limit, need);
  else if (CPLMAX > 8 && need <= 256) select_row<8>(P, task, i, lane, limit, need);
  else if (CPLMAX > 16 && need <= 512) select_row<16>(P, task, i, lane, limit, need);
  else select_row<CPLMAX>(P, task, i, lane, limit, need);
}

int launch_select(const SelectParams& P, cudaStream_t stream) {
  {
    const int64_t tasks = (int64_t)P.rows * P.seq;
    if (tasks == 0 || P.k == 0) return NSA_OK;
    const int64_t blocks = (tasks + 3) / 4;
    if (P.k <= 32 && P.cols <= 1024 && blocks <= 0x7fffffffLL) {
      const unsigned grid = (unsigned)blocks;
      if (P.cols <= 32) select_reg_kernel<1><<<grid, 128, 0, stream>>>(P);
      else if (P.cols <= 64) select_reg_kernel<2><<<grid, 128, 0, stream>>>(P);
      else if (P.cols <= 128) select_reg_kernel<4><<<grid, 128, 0, stream>>>(P);
      else if (P.cols <= 256) select_reg_kernel<8><<<grid, 128, 0, stream>>>(P);
      else if (P.cols <= 512) select_reg_kernel<16><<<grid, 128, 0, stream>>>(P);
      else select_reg_kernel<32><<<grid, 128, 0, stream>>>(P);
      count_launches(1);
      const cudaError_t err = cudaGetLastError();
      if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
      return NSA_OK;
    }
  }
  const int64_t tasks = (int64_t)P.rows * P.seq;
  if (tasks == 0 || P.k == 0) return NSA_OK;
  const size_t per_warp = (size_t)P.cols * sizeof(float);
  int warps = 4;
  while (warps > 1 && per_warp * warps > 200 * 1024) warps >>= 1;
  if (per_warp * warps > 200 * 1024) return fail(NSA_ERR_UNSUPPORTED, "too many block columns for the selection kernel");
  const size_t smem = per_warp * warps;
  cudaError_t err = cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  const int64_t blocks = (tasks + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return fail(NSA_ERR_SHAPE, "too many query rows for one launch");
  select_kernel<<<(unsigned)blocks, 128, smem, stream>>>(P, warps);
  count_launches(1);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
