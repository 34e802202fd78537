// Rotary position embedding of queries / keys in front of the selected and the sliding branch, and its backward.
// One pass over the tensor: reads the (possibly strided) head view, writes a contiguous [B, H, N, d] tensor.
// The angles come as tables cos[n][d/2], sin[n][d/2] (fp32), so the kernel holds no transcendental arithmetic
// and reproduces the elementwise formula  x * cos + rotate_pairs(x) * sin  in fp32 without contraction.

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

// 16 bytes of the row per thread: 4 fp32 / 8 bf16 values = 2 / 4 feature pairs
template <typename T>
__global__ void __launch_bounds__(256) rotary_kernel(const RotaryParams P) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vpr = P.d / V;
  const int64_t total = (int64_t)P.batch * P.heads * P.seq * vpr;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const Coord4 at = split4(e, vpr, P.seq, P.heads);
    const int c = at.i0 * V, n = at.i1, h = at.i2;
    const int64_t b = at.i3;
    const uint4 raw = *reinterpret_cast<const uint4*>((const T*)P.x + b * P.x_sb + h * P.x_sh + (int64_t)n * P.x_sn + c);
    const T* xv = reinterpret_cast<const T*>(&raw);
    const float* cs = P.cos + (int64_t)n * (P.d / 2) + c / 2;
    const float* sn = P.sin + (int64_t)n * (P.d / 2) + c / 2;
    uint4 packed;
    T* ov = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int p = 0; p < V / 2; ++p) {
      const float x0 = Elem<T>::to_float(xv[2 * p]), x1 = Elem<T>::to_float(xv[2 * p + 1]);
      const float co = cs[p], si = P.inverse ? -sn[p] : sn[p];
      // out[2m] = x[2m] cos + (-x[2m+1]) sin ; out[2m+1] = x[2m+1] cos + x[2m] sin
      ov[2 * p] = Elem<T>::from_float(__fadd_rn(__fmul_rn(x0, co), __fmul_rn(-x1, si)));
      ov[2 * p + 1] = Elem<T>::from_float(__fadd_rn(__fmul_rn(x1, co), __fmul_rn(x0, si)));
    }
    *reinterpret_cast<uint4*>((T*)P.out + b * P.o_sb + h * P.o_sh + (int64_t)n * P.o_sn + c) = packed;
  }
}

int launch_rotary(const RotaryParams& P, int dtype, cudaStream_t stream) {
  const int V = dtype == NSA_F32 ? 4 : 8;
  const int64_t total = (int64_t)P.batch * P.heads * P.seq * (P.d / V);
  if (total == 0) return NSA_OK;
  const int64_t blocks = (total + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  if (dtype == NSA_F32) rotary_kernel<float><<<grid, 256, 0, stream>>>(P);
  else rotary_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(P);
  count_launches(1);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
