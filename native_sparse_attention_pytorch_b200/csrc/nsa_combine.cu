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
// With MC the one destination is the multicast address of a symmetric buffer: a single `multimem.st` per piece and the
// NVSwitch writes every rank's copy, this rank's included, so the rank sends its heads once instead of once per peer.
template <typename T, bool MC>
__global__ void __launch_bounds__(256) combine_gather_kernel(const CombineParams P, const GatherTargets Gt) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vpr = P.d / V;
  const int64_t total = (int64_t)P.batch * P.seq * P.q_heads * vpr;
  const int rot = (int)(blockIdx.x % (unsigned)Gt.num_outs);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const Coord4 pos = split4(e, vpr, P.q_heads, P.seq);
    const int c = pos.i0 * V, h = pos.i1, n = pos.i2, b = pos.i3;
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
    if (MC) {
      asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"((T*)Gt.outs[0] + at),
                   "f"(__uint_as_float(packed.x)), "f"(__uint_as_float(packed.y)), "f"(__uint_as_float(packed.z)),
                   "f"(__uint_as_float(packed.w))
                   : "memory");
    } else {
      for (int r = 0; r < Gt.num_outs; ++r) {
        int k = r + rot;
        if (k >= Gt.num_outs) k -= Gt.num_outs;
        *reinterpret_cast<uint4*>((T*)Gt.outs[k] + at) = packed;
      }
    }
  }
  if (MC) __threadfence_system();   // the stores have left for the switch before the kernel counts as finished
}

int launch_combine_gather(const CombineParams& P, const GatherTargets& Gt, int dtype, cudaStream_t stream) {
  const int V = dtype == NSA_F32 ? 4 : 8;
  const int64_t total = (int64_t)P.batch * P.q_heads * P.seq * (P.d / V);
  if (total == 0) return NSA_OK;
  const int64_t blocks = (total + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  if (Gt.multicast) {
    if (dtype == NSA_F32) combine_gather_kernel<float, true><<<grid, 256, 0, stream>>>(P, Gt);
    else combine_gather_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(P, Gt);
  } else {
    if (dtype == NSA_F32) combine_gather_kernel<float, false><<<grid, 256, 0, stream>>>(P, Gt);
    else combine_gather_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(P, Gt);
  }
  count_launches(1);
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
    if (lane == 0) {
      P.d_gates[task * 3 + s] = t;
      if (P.delta != nullptr) P.delta[s * ((int64_t)P.batch * P.q_heads * P.seq) + task] = gs[s] * t;
    }
  }
}

// The same with 16-byte accesses: TPR threads share a (batch, head, position) row, 32 / TPR rows per warp.
template <typename T, int TPR>
__global__ void __launch_bounds__(256) combine_bwd_vec_kernel(const CombineParams P) {
  constexpr int V = 16 / (int)sizeof(T);
  const int64_t tasks = (int64_t)P.batch * P.q_heads * P.seq;
  const int64_t task = ((int64_t)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const bool live = task < tasks;
  float dg[3] = {0.f, 0.f, 0.f}, gate[3] = {0.f, 0.f, 0.f};
  if (live) {
    const Coord4 at = split4(task, P.seq, P.q_heads, 1);
    const int n = at.i0, h = at.i1, b = at.i3;
    const T* g = (const T*)P.gates + b * P.g_sb + h * P.g_sh + (int64_t)n * P.g_sn;
    const int c = part * V;
    const uint4 draw = *reinterpret_cast<const uint4*>((const T*)P.dout + (((int64_t)b * P.seq + n) * P.q_heads + h) * P.d + c);
    const T* dy = reinterpret_cast<const T*>(&draw);
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float gs = Elem<T>::to_float(g[s]);
      gate[s] = gs;
      const uint4 oraw = *reinterpret_cast<const uint4*>((const T*)P.o[s] + b * P.o_sb[s] + h * P.o_sh[s] +
                                                        (int64_t)n * P.o_sn[s] + c);
      const T* ov = reinterpret_cast<const T*>(&oraw);
      uint4 packed;
      T* pv = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int x = 0; x < V; ++x) {
        const float d = Elem<T>::to_float(dy[x]);
        dg[s] = fmaf(d, Elem<T>::to_float(ov[x]), dg[s]);
        pv[x] = Elem<T>::from_float(gs * d);
      }
      *reinterpret_cast<uint4*>((T*)P.d_o[s] + task * P.d + c) = packed;
    }
  }
#pragma unroll
  for (int s = 0; s < 3; ++s) {
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) dg[s] += __shfl_xor_sync(kFullMask, dg[s], o);
    if (live && part == 0) {
      P.d_gates[task * 3 + s] = dg[s];
      if (P.delta != nullptr) P.delta[s * tasks + task] = gate[s] * dg[s];
    }
  }
}

template <typename T>
static bool launch_combine_bwd_vec(const CombineParams& P, cudaStream_t stream) {
  constexpr int V = 16 / (int)sizeof(T);
  if (P.d % V) return false;
  const uintptr_t ptrs[5] = {(uintptr_t)P.dout, (uintptr_t)P.o[0], (uintptr_t)P.o[1], (uintptr_t)P.o[2], (uintptr_t)P.d_o[0]};
  for (uintptr_t p : ptrs)
    if (p & 15u) return false;
  if (((uintptr_t)P.d_o[1] & 15u) || ((uintptr_t)P.d_o[2] & 15u)) return false;
  for (int s = 0; s < 3; ++s)
    if (P.o_sb[s] % V || P.o_sh[s] % V || P.o_sn[s] % V) return false;
  const int tpr = P.d / V;
  const int64_t threads = (int64_t)P.batch * P.q_heads * P.seq * tpr;
  const int64_t blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffLL) return false;
  const unsigned grid = (unsigned)blocks;
  switch (tpr) {
    case 2: combine_bwd_vec_kernel<T, 2><<<grid, 256, 0, stream>>>(P); return true;
    case 4: combine_bwd_vec_kernel<T, 4><<<grid, 256, 0, stream>>>(P); return true;
    case 8: combine_bwd_vec_kernel<T, 8><<<grid, 256, 0, stream>>>(P); return true;
    case 16: combine_bwd_vec_kernel<T, 16><<<grid, 256, 0, stream>>>(P); return true;
    case 32: combine_bwd_vec_kernel<T, 32><<<grid, 256, 0, stream>>>(P); return true;
    default: return false;
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
  } else if (dtype == NSA_F32 ? launch_combine_bwd_vec<float>(P, stream) : launch_combine_bwd_vec<__nv_bfloat16>(P, stream)) {
    // 16-byte accesses served it
  } else {
    const int64_t blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffLL) return fail(NSA_ERR_SHAPE, "too many rows for one launch");
    if (dtype == NSA_F32) combine_bwd_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>(P);
    else combine_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(P);
  }
  count_launches(1);   // every path above launched exactly one kernel
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

}  // namespace nsa
