// Shared device helpers for the NSA kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdint.h>

#include "nsa_b200.h"

namespace nsa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned kFullMask = 0xffffffffu;

// ---- element access: T is float or __nv_bfloat16 ---------------------------
template <typename T>
struct Elem;

template <>
struct Elem<float> {
  static constexpr int kVec = 4;  // elements in a 16-byte vector
  __device__ static __forceinline__ void load_vec(const float* p, float (&o)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
  __device__ static __forceinline__ float2 load2(const float* p) {
    return *reinterpret_cast<const float2*>(p);
  }
  __device__ static __forceinline__ void store2(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
  }
  __device__ static __forceinline__ float to_float(float v) { return v; }
  __device__ static __forceinline__ float from_float(float v) { return v; }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static __forceinline__ void load_vec(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ float2 load2(const __nv_bfloat16* p) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  __device__ static __forceinline__ void store2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
  __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Split a flat index over [d3][d2][d1][d0] (d0 fastest) into its four coordinates; with 32-bit arithmetic whenever
// the index fits (64-bit divisions cost several times more instructions, and these kernels are otherwise a few
// loads and stores per thread).
struct Coord4 { int i0, i1, i2, i3; };
__device__ __forceinline__ Coord4 split4(int64_t e, int d0, int d1, int d2) {
  Coord4 r;
  if (e < 0x7fffffffLL) {
    unsigned u = (unsigned)e;
    r.i0 = (int)(u % (unsigned)d0); u /= (unsigned)d0;
    r.i1 = (int)(u % (unsigned)d1); u /= (unsigned)d1;
    r.i2 = (int)(u % (unsigned)d2); r.i3 = (int)(u / (unsigned)d2);
  } else {
    r.i0 = (int)(e % d0); e /= d0;
    r.i1 = (int)(e % d1); e /= d1;
    r.i2 = (int)(e % d2); r.i3 = (int)(e / d2);
  }
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}

}  // namespace nsa
