// Gated combine of the three branch outputs with the head merge folded into
// the store, and its backward.  Pure streaming kernels (HBM bound).

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

template <typename T>
__global__ void __launch_bounds__(256) combine_fwd_kernel(const CombineParams P) {
  const int half = P.d / 2;
  const int64_t total = (int64_t)P.batch * P.seq * P.q_heads * half;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(e % half) * 2;
    const int h = (int)((e / half) % P.q_heads);
    const int n = (int)((e / ((int64_t)half * P.q_heads)) % P.seq);
    const int b = (int)(e / ((int64_t)half * P.q_heads * P.seq));
    const T* g = (const T*)P.gates + b * P.g_sb + h * P.g_sh + (int64_t)n * P.g_sn;
    float ax = 0.f, ay = 0.f;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float gs = Elem<T>::to_float(g[s]);
      const float2 v = Elem<T>::load2((const T*)P.o[s] + b * P.o_sb[s] + h * P.o_sh[s] + (int64_t)n * P.o_sn[s] + c);
      ax = fmaf(gs, v.x, ax);
      ay = fmaf(gs, v.y, ay);
    }
    Elem<T>::store2((T*)P.out + (((int64_t)b * P.seq + n) * P.q_heads + h) * P.d + c, ax, ay);
  }
}

// The same with 16-byte accesses and up to kMaxGather destinations: every destination is a [B, N, total_features]
// buffer (this GPU's own or a peer's, mapped into this process) and receives this rank's heads at feature_offset.
// With more than one destination this is the combine fused with the all-gather of the head-sharded layout: the
// merged rows never exist as a local tensor, each 16-byte piece goes straight to every rank.  Blocks start their
// round over the destinations at different ranks so that the links are used side by side.
template <typename T>
__global__ void __launch_bounds__(256) combine_gather_kernel(const CombineParams P, const GatherTargets Gt) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vpr = P.d / V;
  const int64_t total = (int64_t)P.batch * P.seq * P.q_heads * vpr;
  const int rot = (int)(blockIdx.x % (unsigned)Gt.num_outs);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(e % vpr) * V;
    const int h = (int)((e / vpr) % P.q_heads);
    const int n = (int)((e / ((int64_t)vpr * P.q_heads)) % P.seq);
    const int b = (int)(e / ((int64_t)vpr * P.q_heads * P.seq));
    const T* g = (const T*)P.gates + b * P.g_sb + h * P.g_sh + (int64_t)n * P.g_sn;
    float acc[V];
#pragma unroll
    for (int x = 0; x < V; ++x) acc[x] = 0.f;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float gs = Elem<T>::to_float(g[s]);
      const uint4 raw = *reinterpret_cast<const uint4*>((const T*)P.o[s] + b * P.o_sb[s] + h * P.o_sh[s] +
                                                       (int64_t)n * P.o_sn[s] + c);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int x = 0; x < V; ++x) acc[x] = fmaf(gs, Elem<T>::to_float(v[x]), acc[x]);
    }
    uint4 packed;
    T* pv = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int x = 0; x < V; ++x) pv[x] = Elem<T>::from_float(acc[x]);
    const int64_t at = ((int64_t)b * P.seq + n) * Gt.total_features + Gt.feature_offset + (int64_t)h * P.d + c;
    for (int r = 0; r < Gt.num_outs; ++r) {
      int k = r + rot;
      if (k >= Gt.num_outs) k -= Gt.num_outs;
      *reinterpret_cast<uint4*>((T*)Gt.outs[k] + at) = packed;
    }
  }
}

int launch_combine_gather(const CombineParams& P, const GatherTargets& Gt, int dtype, cudaStream_t stream) {
  const int V = dtype == NSA_F32 ? 4 : 8;
  const int64_t total = (int64_t)P.batch * P.q_heads * P.seq * (P.d / V);
  if (total == 0) return NSA_OK;
  const int64_t blocks = (total + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  if (dtype == NSA_F32) combine_gather_kernel<float><<<grid, 256, 0, stream>>>(P, Gt);
  else combine_gather_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(P, Gt);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

// one warp per (batch, head, position)
template <typename T>
__global__ void __launch_bounds__(128) combine_bwd_kernel(const CombineParams P) {
  const int lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (task >= (int64_t)P.batch * P.q_heads * P.seq) return;
  const int n = (int)(task % P.seq);
  const int h = (int)((task / P.seq) % P.q_heads);
  const int b = (int)(task / ((int64_t)P.seq * P.q_heads));
  const T* g = (const T*)P.gates + b * P.g_sb + h * P.g_sh + (int64_t)n * P.g_sn;
  const T* dout = (const T*)P.dout + (((int64_t)b * P.seq + n) * P.q_heads + h) * P.d;
  float gs[3], dg[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < 3; ++s) gs[s] = Elem<T>::to_float(g[s]);
  for (int c = 2 * lane; c < P.d; c += 64) {
    const float2 dy = Elem<T>::load2(dout + c);
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float2 v = Elem<T>::load2((const T*)P.o[s] + b * P.o_sb[s] + h * P.o_sh[s] + (int64_t)n * P.o_sn[s] + c);
      dg[s] += dy.x * v.x + dy.y * v.y;
      Elem<T>::store2((T*)P.d_o[s] + task * P.d + c, gs[s] * dy.x, gs[s] * dy.y);
    }
  }
#pragma unroll
  for (int s = 0; s < 3; ++s) {
    const float t = warp_sum(dg[s]);
    if (lane == 0) P.d_gates[task * 3 + s] = t;
  }
}

int launch_combine(const CombineParams& P, int dtype, bool backward, cudaStream_t stream) {
  const int64_t rows = (int64_t)P.batch * P.q_heads * P.seq;
  if (rows == 0) return NSA_OK;
  if (!backward) {
    const int64_t total = rows * (P.d / 2);
    const int64_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
    if (dtype == NSA_F32) combine_fwd_kernel<float><<<grid, 256, 0, stream>>>(P);
    else combine_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(P);
  } else {
    const int64_t blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffLL) return fail(NSA_ERR_SHAPE, "too many rows for one launch");
    if (dtype == NSA_F32) combine_bwd_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>(P);
    else combine_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(P);
  }
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
