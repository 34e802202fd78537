// Input of the compress networks: overlapping windows of the (un-rotated) keys or values plus the learned
// intra-block positions, and the backward of that step.  Upstream pads, unfolds, permutes and adds with four tensor
// operations and lets autograd invert them (an index-add and two reductions); here each direction is one pass.
//   out[b,h,w,j,:] = x[b,h,(w+1)*stride - block + j,:] (zero before the sequence start) + pos[h,j,:]

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

template <typename T>
__global__ void __launch_bounds__(256) windows_fwd_kernel(const WindowParams P) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vpr = P.d / V;
  const int64_t total = (int64_t)P.batch * P.heads * P.ncb * P.block * vpr;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const Coord4 at = split4(e, vpr, P.block, P.ncb);     // i3 = b * heads + h
    const int c = at.i0 * V, j = at.i1, w = at.i2;
    const int h = at.i3 % P.heads;
    const int64_t b = at.i3 / P.heads;
    const int tok = (w + 1) * P.stride - P.block + j;
    uint4 xraw = make_uint4(0u, 0u, 0u, 0u);
    if (tok >= 0) xraw = *reinterpret_cast<const uint4*>((const T*)P.x + b * P.x_sb + h * P.x_sh + (int64_t)tok * P.x_sn + c);
    const uint4 praw = *reinterpret_cast<const uint4*>((const T*)P.pos + ((int64_t)h * P.block + j) * P.d + c);
    const T* xv = reinterpret_cast<const T*>(&xraw);
    const T* pv = reinterpret_cast<const T*>(&praw);
    uint4 packed;
    T* ov = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int x = 0; x < V; ++x) ov[x] = Elem<T>::from_float(Elem<T>::to_float(xv[x]) + Elem<T>::to_float(pv[x]));
    *reinterpret_cast<uint4*>((T*)P.out + e * V) = packed;
  }
}

// dx[b,h,tok,:] = sum of dout over the windows that hold tok (at most ceil(block / stride) of them)
template <typename T>
__global__ void __launch_bounds__(256) windows_bwd_x_kernel(const WindowParams P) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vpr = P.d / V;
  const int64_t total = (int64_t)P.batch * P.heads * P.seq * vpr;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const Coord4 at = split4(e, vpr, P.seq, P.heads);
    const int c = at.i0 * V, tok = at.i1;
    const int64_t h = at.i2, b = at.i3, bh = b * P.heads + h;
    float acc[V];
#pragma unroll
    for (int x = 0; x < V; ++x) acc[x] = 0.f;
    const int w_lo = tok / P.stride, w_hi = min(P.ncb, (tok + P.block) / P.stride);   // windows w_lo .. w_hi - 1
    for (int w = w_lo; w < w_hi; ++w) {
      const int j = tok - (w + 1) * P.stride + P.block;
      const uint4 raw = *reinterpret_cast<const uint4*>((const T*)P.dout + ((bh * P.ncb + w) * P.block + j) * P.d + c);
      const T* dv = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int x = 0; x < V; ++x) acc[x] += Elem<T>::to_float(dv[x]);
    }
    uint4 packed;
    T* ov = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int x = 0; x < V; ++x) ov[x] = Elem<T>::from_float(acc[x]);
    *reinterpret_cast<uint4*>((T*)P.dx + b * P.dx_sb + h * P.dx_sh + (int64_t)tok * P.dx_sn + c) = packed;
  }
}

// dpos[h,j,c] = sum over (batch, window) of dout[b,h,w,j,c].  A window is block * d contiguous elements: thread t of
// blockIdx.x = (h, group of 128 sixteen-byte slots) owns one slot of the window, blockIdx.y a slice of the
// (batch, window) pairs; every slice adds its sums into the zeroed dpos.
template <typename T>
__global__ void __launch_bounds__(128) windows_bwd_pos_kernel(const WindowParams P, int slot_groups) {
  constexpr int V = 16 / (int)sizeof(T);
  const int slots = P.block * P.d / V;
  const int h = blockIdx.x / slot_groups, slot = (blockIdx.x % slot_groups) * 128 + threadIdx.x;
  if (slot >= slots) return;
  const int pairs = P.batch * P.ncb;                      // the entry point keeps this below 2^31
  const int per = (pairs + (int)gridDim.y - 1) / (int)gridDim.y;
  const int k0 = (int)blockIdx.y * per, k1 = min(k0 + per, pairs);
  const int64_t window = (int64_t)slots * V;
  const T* base = (const T*)P.dout + (int64_t)slot * V;
  auto at = [&](int k) { return base + (((int64_t)(k / P.ncb) * P.heads + h) * P.ncb + k % P.ncb) * window; };
  float acc[V];
#pragma unroll
  for (int x = 0; x < V; ++x) acc[x] = 0.f;
  int k = k0;
  for (; k + 8 <= k1; k += 8) {                            // eight independent loads in flight per thread
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(at(k + u));
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const T* dv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int x = 0; x < V; ++x) acc[x] += Elem<T>::to_float(dv[x]);
    }
  }
  for (; k < k1; ++k) {
    const uint4 raw = *reinterpret_cast<const uint4*>(at(k));
    const T* dv = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int x = 0; x < V; ++x) acc[x] += Elem<T>::to_float(dv[x]);
  }
  float* dst = P.dpos + (int64_t)h * slots * V + (int64_t)slot * V;
#pragma unroll
  for (int x = 0; x < V; ++x) atomicAdd(dst + x, acc[x]);
}

int launch_windows(const WindowParams& P, int dtype, bool backward, cudaStream_t stream) {
  const int V = dtype == NSA_F32 ? 4 : 8;
  const int64_t total = backward ? (int64_t)P.batch * P.heads * P.seq * (P.d / V)
                                 : (int64_t)P.batch * P.heads * P.ncb * P.block * (P.d / V);
  if (total > 0) {
    const int64_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    if (!backward) {
      if (dtype == NSA_F32) windows_fwd_kernel<float><<<grid, 256, 0, stream>>>(P);
      else windows_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(P);
    } else {
      if (dtype == NSA_F32) windows_bwd_x_kernel<float><<<grid, 256, 0, stream>>>(P);
      else windows_bwd_x_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(P);
    }
    count_launches(1);
  }
  if (backward && P.heads > 0 && P.block > 0) {
    const cudaError_t zerr = cudaMemsetAsync(P.dpos, 0, (size_t)P.heads * P.block * P.d * sizeof(float), stream);
    if (zerr != cudaSuccess) return fail((int)zerr, cudaGetErrorString(zerr));
    const int64_t pairs = (int64_t)P.batch * P.ncb;   // below 2^31: checked by the caller of this launcher
    const int slot_groups = (P.block * P.d / V + 127) / 128;
    const int64_t ctas = (int64_t)P.heads * slot_groups;
    int64_t slices = (148 * 3 + ctas - 1) / ctas;            // about three CTAs per SM: every slice ends in atomics
    slices = slices > pairs ? pairs : slices;
    slices = slices < 1 ? 1 : (slices > 65535 ? 65535 : slices);
    const dim3 grid((unsigned)ctas, (unsigned)slices);
    if (dtype == NSA_F32) windows_bwd_pos_kernel<float><<<grid, 128, 0, stream>>>(P, slot_groups);
    else windows_bwd_pos_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(P, slot_groups);
    count_launches(1);
  }
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
