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

  for (int j = lane; j < P.cols; j += 32) {
    float v;
    if (P.cpf == 1) {
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

int launch_select(const SelectParams& P, cudaStream_t stream) {
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
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
