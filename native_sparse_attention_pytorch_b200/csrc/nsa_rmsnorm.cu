// RMS normalisation of the layer input (the first step of the attention layer's forward) and its backward.
//   y = x * rstd * weight,  rstd = rsqrt(mean(x^2) + eps)
//   dx = rstd * (dy*weight - xhat * mean(dy*weight*xhat)),  dweight = sum over rows of dy * xhat,  xhat = x * rstd
// One warp per row with the row in registers (NV sixteen-byte pieces per lane), fp32 arithmetic.  The backward keeps
// the weight gradient of the rows a warp visits in registers, folds the warps of a block through shared memory and
// adds one partial per block into the zeroed fp32 output: x and dy are read once, dx written once.

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

template <typename T>
struct Piece {
  static constexpr int V = 16 / (int)sizeof(T);
  __device__ static void load(const void* base, int64_t elem, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>((const T*)base + elem);
    const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int x = 0; x < V; ++x) out[x] = Elem<T>::to_float(v[x]);
  }
  __device__ static void store(void* base, int64_t elem, const float* in) {
    uint4 raw;
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int x = 0; x < V; ++x) v[x] = Elem<T>::from_float(in[x]);
    *reinterpret_cast<uint4*>((T*)base + elem) = raw;
  }
};

// weight piece as fp32, from a weight stored in T or in fp32
template <typename T>
__device__ __forceinline__ void load_weight(const NormParams& P, int elem, float* out) {
  constexpr int V = Piece<T>::V;
  if (P.weight_f32) {
#pragma unroll
    for (int x = 0; x < V; ++x) out[x] = ((const float*)P.weight)[elem + x];
  } else {
    Piece<T>::load(P.weight, elem, out);
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const NormParams P) {
  constexpr int V = Piece<T>::V;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * 8;
  const int pieces = P.dim / V;
  float w[NV][V];
#pragma unroll
  for (int t = 0; t < NV; ++t)
    if (lane + 32 * t < pieces) load_weight<T>(P, (lane + 32 * t) * V, w[t]);
  for (int64_t row = warp; row < P.rows; row += warps) {
    float x[NV][V];
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if (lane + 32 * t < pieces) {
        Piece<T>::load(P.x, row * P.x_stride + (lane + 32 * t) * V, x[t]);
#pragma unroll
        for (int e = 0; e < V; ++e) ss += x[t][e] * x[t][e];
      }
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)P.dim + P.eps);
    if (lane == 0) P.rstd[row] = rstd;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if (lane + 32 * t < pieces) {
#pragma unroll
        for (int e = 0; e < V; ++e) x[t][e] = x[t][e] * rstd * w[t][e];
        Piece<T>::store(P.y, row * P.dim + (lane + 32 * t) * V, x[t]);
      }
    }
  }
}

// x and dy of a row stay in registers as loaded (16-byte pieces) and are decoded once for the dot product and the
// weight gradient and once more for dx; the weight sits in shared memory: registers go to the weight-gradient
// accumulators, and two or three blocks fit an SM.
template <typename T, int NV>
__global__ void __launch_bounds__(256, NV <= 4 ? 2 : 1) rmsnorm_bwd_kernel(const NormParams P) {
  constexpr int V = Piece<T>::V;
  extern __shared__ float norm_smem[];          // weight [dim], then the fold area [8][32 * V + 1]
  float* w_s = norm_smem;
  float (*fold)[32 * V + 1] = reinterpret_cast<float (*)[32 * V + 1]>(norm_smem + ((P.dim + 3) & ~3));
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * 8 + wib, warps = (int64_t)gridDim.x * 8;
  const int pieces = P.dim / V;
  for (int p = threadIdx.x; p < pieces; p += 256) {
    float tmp[V];
    load_weight<T>(P, p * V, tmp);
#pragma unroll
    for (int e = 0; e < V; ++e) w_s[p * V + e] = tmp[e];
  }
  __syncthreads();
  float dw[NV][V];
#pragma unroll
  for (int t = 0; t < NV; ++t)
#pragma unroll
    for (int e = 0; e < V; ++e) dw[t][e] = 0.f;
  for (int64_t row = warp; row < P.rows; row += warps) {
    const float rstd = P.rstd[row];
    uint4 xr[NV], gr[NV];
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if (lane + 32 * t < pieces) {
        xr[t] = *reinterpret_cast<const uint4*>((const T*)P.x + row * P.x_stride + (lane + 32 * t) * V);
        gr[t] = *reinterpret_cast<const uint4*>((const T*)P.dy + row * P.dim + (lane + 32 * t) * V);
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if (lane + 32 * t < pieces) {
        const T* xv = reinterpret_cast<const T*>(&xr[t]);
        const T* gv = reinterpret_cast<const T*>(&gr[t]);
        const float* wv = w_s + (lane + 32 * t) * V;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float xh = Elem<T>::to_float(xv[e]) * rstd, g = Elem<T>::to_float(gv[e]);
          dw[t][e] += g * xh;
          dot += (g * wv[e]) * xh;
        }
      }
    }
    const float c = warp_sum(dot) / (float)P.dim;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if (lane + 32 * t < pieces) {
        const T* xv = reinterpret_cast<const T*>(&xr[t]);
        const T* gv = reinterpret_cast<const T*>(&gr[t]);
        const float* wv = w_s + (lane + 32 * t) * V;
        float o[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float xh = Elem<T>::to_float(xv[e]) * rstd, g = Elem<T>::to_float(gv[e]);
          o[e] = rstd * (g * wv[e] - xh * c);
        }
        Piece<T>::store(P.dx, row * P.dim + (lane + 32 * t) * V, o);
      }
    }
  }
  // fold the eight warps of the block, one group of 32 pieces at a time, and add the block's partial
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < V; ++e) fold[wib][lane * V + e] = dw[t][e];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * V; i += 256) {
      const int elem = 32 * t * V + i;
      if (elem < P.dim) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += fold[k][i];
        atomicAdd(P.dweight + elem, s);
      }
    }
  }
}

template <typename T, int NV>
static void launch_one(const NormParams& P, bool backward, unsigned grid, cudaStream_t stream) {
  constexpr int V = Piece<T>::V;
  const size_t bwd_smem = (size_t)(((P.dim + 3) & ~3) + 8 * (32 * V + 1)) * sizeof(float);   // at most 16.3 KB
  if (backward) rmsnorm_bwd_kernel<T, NV><<<grid, 256, bwd_smem, stream>>>(P);
  else rmsnorm_fwd_kernel<T, NV><<<grid, 256, 0, stream>>>(P);
  count_launches(1);
}

template <typename T>
static int launch_typed(const NormParams& P, bool backward, unsigned grid, cudaStream_t stream) {
  const int per_lane = (P.dim / Piece<T>::V + 31) / 32;
  if (per_lane <= 1) launch_one<T, 1>(P, backward, grid, stream);
  else if (per_lane <= 2) launch_one<T, 2>(P, backward, grid, stream);
  else if (per_lane <= 4) launch_one<T, 4>(P, backward, grid, stream);
  else if (per_lane <= 8) launch_one<T, 8>(P, backward, grid, stream);
  else return fail(NSA_ERR_UNSUPPORTED, "model dimension above 8 sixteen-byte pieces per lane");
  return NSA_OK;
}

int launch_rmsnorm(const NormParams& P, int dtype, bool backward, cudaStream_t stream) {
  if (P.rows == 0) {
    if (backward) {
      const cudaError_t zerr = cudaMemsetAsync(P.dweight, 0, (size_t)P.dim * sizeof(float), stream);
      if (zerr != cudaSuccess) return fail((int)zerr, cudaGetErrorString(zerr));
    }
    return NSA_OK;
  }
  const int64_t blocks = (P.rows + 7) / 8;
  // the backward adds one partial per block: a few blocks per SM bound the atomics, the forward is a plain stream
  const int64_t cap = backward ? 148 * 2 : 148 * 16;   // backward: the blocks one wave holds (two per SM)
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  if (backward) {
    const cudaError_t zerr = cudaMemsetAsync(P.dweight, 0, (size_t)P.dim * sizeof(float), stream);
    if (zerr != cudaSuccess) return fail((int)zerr, cudaGetErrorString(zerr));
  }
  const int rc = dtype == NSA_F32 ? launch_typed<float>(P, backward, grid, stream)
                                  : launch_typed<__nv_bfloat16>(P, backward, grid, stream);
  if (rc != NSA_OK) return rc;
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
