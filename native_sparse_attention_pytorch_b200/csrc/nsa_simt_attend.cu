// Generic CUDA-core kernels for the three NSA attention branches.
//
// One warp serves one (batch, head group, query) task and all query heads of
// the group, so every fetched key/value row is shared by the group (GQA).
// The key set of a task is a list of runs of consecutive key positions:
//   selected branch  : one run per visible slot + the own-block run
//   compressed branch: the memory slots, then the visible compressed blocks
//   sliding branch   : the window around the query
// Inside a run, lanes map to keys for the two dot products (q.k and do.v) and
// to feature pairs for the accumulations (p.v, ds.k, ds.q, p.do); values move
// between the two mappings with warp shuffles.  All arithmetic is fp32, which
// is what lets this family meet a 1e-4 relative bound on fp32 inputs; it also
// serves every shape the tensor-core family does not cover.

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

constexpr int kWarpsPerBlock = 4;

// Stages the G query rows (or upstream-gradient rows) of a task as fp32.
template <typename T, int GT>
__device__ __forceinline__ void stage_rows(float* dst, const T* src, int64_t head_stride, int G, int d, int lane) {
  for (int e = lane * 2; e < GT * d; e += 64) {
    const int g = e / d, c = e - g * d;
    float2 val = make_float2(0.f, 0.f);
    if (g < G) val = Elem<T>::load2(src + g * head_stride + c);
    dst[e] = val.x;
    dst[e + 1] = val.y;
  }
}

// s[g] += sum_c rows[g][c] * key[c] for this lane's key row.
template <typename T, int GT>
__device__ __forceinline__ void dot_rows(float (&s)[GT], const float* rows, const T* key, int d) {
  constexpr int V = Elem<T>::kVec;
  for (int c = 0; c < d; c += V) {
    float kv[V];
    Elem<T>::load_vec(key + c, kv);
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float* r = rows + g * d + c;
#pragma unroll
      for (int e = 0; e < V; e += 4) {
        const float4 qv = *reinterpret_cast<const float4*>(r + e);
        s[g] = fmaf(qv.x, kv[e], s[g]);
        s[g] = fmaf(qv.y, kv[e + 1], s[g]);
        s[g] = fmaf(qv.z, kv[e + 2], s[g]);
        s[g] = fmaf(qv.w, kv[e + 3], s[g]);
      }
    }
  }
}

// The runs of one task.  run(r) yields [start, end) in key-row units, whether
// rows >= valid_rows inside the run are zero keys, and whether the run is the
// "uniform" kind (all logits equal, no gradient to q and k).
struct Run {
  int start, end;
  int slot;  // selected-branch slot index, or -1
};

template <int BR>
struct TaskRuns {
  int count;
  bool uniform;   // selected branch only: the query sees no key at all
  int total_keys; // number of keys when uniform
  // selected branch: slot s is run s, own block is run nsel
  __device__ __forceinline__ void init(const AttnParams& P, int b, int grp, int i) {
    uniform = false;
    total_keys = 0;
    if (BR == BR_SEL) {
      count = P.nsel + (P.diag != NSA_DIAG_NONE ? 1 : 0);
      bool any = P.diag != NSA_DIAG_NONE;
      const int nfb = (P.seq + P.block - 1) / P.block;
      const int64_t base = (((int64_t)b * P.groups + grp) * P.seq + i) * P.nsel;
      int in_range = 0;
      for (int s = 0; s < P.nsel; ++s) {
        const int64_t blk = P.idx[base + s];
        const bool ok = blk >= 0 && blk < nfb;
        in_range += ok ? 1 : 0;
        any = any || (ok && P.mask[base + s] != 0);
      }
      uniform = !any;
      total_keys = in_range * P.block;
    } else if (BR == BR_CMP) {
      count = 2;
    } else {
      count = 1;
    }
  }
  __device__ __forceinline__ Run get(const AttnParams& P, int b, int grp, int i, int r) const {
    Run run;
    run.slot = -1;
    if (BR == BR_SEL) {
      if (r < P.nsel) {
        const int nfb = (P.seq + P.block - 1) / P.block;
        const int64_t base = (((int64_t)b * P.groups + grp) * P.seq + i) * P.nsel;
        const int64_t blk = P.idx[base + r];
        const bool ok = blk >= 0 && blk < nfb && (uniform || P.mask[base + r] != 0);
        run.start = ok ? (int)blk * P.block : 0;
        run.end = ok ? run.start + P.block : 0;
        run.slot = r;
      } else {
        const int own = i / P.block * P.block;
        run.start = own;
        run.end = P.diag == NSA_DIAG_CAUSAL ? i + 1 : own + P.block;
      }
    } else if (BR == BR_CMP) {
      if (r == 0) {
        run.start = 0;
        run.end = P.num_mem;
      } else {
        const int vis = P.causal ? min(P.ncb, i / P.stride) : P.ncb;
        run.start = P.num_mem;
        run.end = P.num_mem + vis;
      }
    } else {
      run.start = max(0, i - P.window);
      run.end = P.causal ? i + 1 : min(P.seq, i + P.window + 1);
    }
    return run;
  }
};

template <typename T, int GT, int BR>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attend_fwd_kernel(const AttnParams P) {
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t task = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t ntasks = (int64_t)P.batch * P.groups * P.seq;
  if (task >= ntasks) return;
  const int i = (int)(task % P.seq);
  const int grp = (int)((task / P.seq) % P.groups);
  const int b = (int)(task / ((int64_t)P.seq * P.groups));
  const int G = P.q_heads / P.groups;
  const int kvh = grp / (P.groups / P.kv_heads);
  const int d = P.d;
  float* q_s = smem + warp * GT * d;

  const T* qp = (const T*)P.q + b * P.q_sb + (int64_t)(grp * G) * P.q_sh + (int64_t)i * P.q_sn;
  stage_rows<T, GT>(q_s, qp, P.q_sh, G, d, lane);
  __syncwarp();
  const T* kb = (const T*)P.k + b * P.k_sb + (int64_t)kvh * P.k_sh;
  const T* vb = (const T*)P.v + b * P.v_sb + (int64_t)kvh * P.v_sh;

  float m[GT], l[GT], acc[GT][2][2];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
    acc[g][0][0] = acc[g][0][1] = acc[g][1][0] = acc[g][1][1] = 0.f;
  }

  TaskRuns<BR> runs;
  runs.init(P, b, grp, i);
  for (int r = 0; r < runs.count; ++r) {
    const Run run = runs.get(P, b, grp, i, r);
    for (int t0 = run.start; t0 < run.end; t0 += 32) {
      const int pos = t0 + lane;
      const bool present = pos < run.end;
      const bool real = present && pos < P.key_rows;  // rows past the end are zero keys
      float s[GT];
#pragma unroll
      for (int g = 0; g < GT; ++g) s[g] = 0.f;
      if (real && !runs.uniform) dot_rows<T, GT>(s, q_s, kb + (int64_t)pos * P.k_sn, d);
      if (BR == BR_CMP && r == 1 && P.importance != nullptr && present) {
        // the logit as upstream's tensor of that dtype would hold it
        const int w = pos - P.num_mem;
        float logit[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g)
          logit[g] = P.round_bf16 ? round_bf16(round_bf16(s[g]) * P.scale) : s[g] * P.scale;
        if (P.imp_heads == P.kv_heads) {
          float sum = 0.f;
#pragma unroll
          for (int g = 0; g < GT; ++g) sum += (g < G) ? logit[g] : 0.f;
          float mean = sum / (float)G;
          if (P.round_bf16) mean = round_bf16(mean);
          P.importance[(((int64_t)b * P.imp_heads + kvh) * P.seq + i) * P.ncb + w] = mean;
        } else {
#pragma unroll
          for (int g = 0; g < GT; ++g)
            if (g < G) P.importance[(((int64_t)b * P.imp_heads + kvh * G + g) * P.seq + i) * P.ncb + w] = logit[g];
        }
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) s[g] *= P.scale;
      float p[GT];
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float tile_max = warp_max(present ? s[g] : -INFINITY);
        const float m_new = fmaxf(m[g], tile_max);
        const float alpha = exp2f((m[g] - m_new) * kLog2e);
        p[g] = present ? exp2f((s[g] - m_new) * kLog2e) : 0.f;
        l[g] = l[g] * alpha + warp_sum(p[g]);
        m[g] = m_new;
        acc[g][0][0] *= alpha; acc[g][0][1] *= alpha;
        acc[g][1][0] *= alpha; acc[g][1][1] *= alpha;
      }
      const int cnt = min(32, min(run.end, P.key_rows) - t0);
      for (int kk = 0; kk < cnt; ++kk) {
        const T* vrow = vb + (int64_t)(t0 + kk) * P.v_sn;
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
  }

  if (BR == BR_CMP && P.importance != nullptr) {
    // columns the query cannot see carry the sentinel (its head mean, when shared)
    const int vis = P.causal ? min(P.ncb, i / P.stride) : P.ncb;
    float fill = P.sentinel;
    if (P.imp_heads == P.kv_heads) {
      float sum = 0.f;
      for (int g = 0; g < G; ++g) sum += P.sentinel;
      fill = sum / (float)G;
      if (P.round_bf16) fill = round_bf16(fill);
    }
    const int heads_here = P.imp_heads == P.kv_heads ? 1 : G;
    for (int hh = 0; hh < heads_here; ++hh) {
      const int ih = P.imp_heads == P.kv_heads ? kvh : kvh * G + hh;
      float* row = P.importance + (((int64_t)b * P.imp_heads + ih) * P.seq + i) * P.ncb;
      for (int w = vis + lane; w < P.ncb; w += 32) row[w] = fill;
    }
  }

  T* op = (T*)P.out + b * P.o_sb + (int64_t)(grp * G) * P.o_sh + (int64_t)i * P.o_sn;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (g >= G) break;
    const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int dim = 64 * c + 2 * lane;
      if (dim < d) Elem<T>::store2(op + g * P.o_sh + dim, acc[g][c][0] * inv, acc[g][c][1] * inv);
    }
    if (lane == 0)
      P.lse[((int64_t)b * P.q_heads + grp * G + g) * P.seq + i] = l[g] > 0.f ? m[g] + logf(l[g]) : -INFINITY;
  }
}

template <typename T, int GT, int BR>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attend_bwd_kernel(const AttnParams P) {
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t task = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t ntasks = (int64_t)P.batch * P.groups * P.seq;
  if (task >= ntasks) return;
  const int i = (int)(task % P.seq);
  const int grp = (int)((task / P.seq) % P.groups);
  const int b = (int)(task / ((int64_t)P.seq * P.groups));
  const int G = P.q_heads / P.groups;
  const int kvh = grp / (P.groups / P.kv_heads);
  const int d = P.d;
  float* q_s = smem + warp * 2 * GT * d;
  float* do_s = q_s + GT * d;

  const T* qp = (const T*)P.q + b * P.q_sb + (int64_t)(grp * G) * P.q_sh + (int64_t)i * P.q_sn;
  const T* dop = (const T*)P.dout + b * P.do_sb + (int64_t)(grp * G) * P.do_sh + (int64_t)i * P.do_sn;
  const T* op = (const T*)P.out + b * P.o_sb + (int64_t)(grp * G) * P.o_sh + (int64_t)i * P.o_sn;
  stage_rows<T, GT>(q_s, qp, P.q_sh, G, d, lane);
  stage_rows<T, GT>(do_s, dop, P.do_sh, G, d, lane);
  __syncwarp();
  const T* kb = (const T*)P.k + b * P.k_sb + (int64_t)kvh * P.k_sh;
  const T* vb = (const T*)P.v + b * P.v_sb + (int64_t)kvh * P.v_sh;
  float* dkb = P.dk + ((int64_t)b * P.kv_heads + kvh) * P.key_rows * d;
  float* dvb = P.dv + ((int64_t)b * P.kv_heads + kvh) * P.key_rows * d;

  float lse[GT], delta[GT], dq[GT][2][2];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    float part = 0.f;
    if (g < G) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int dim = 64 * c + 2 * lane;
        if (dim < d) {
          const float2 o = Elem<T>::load2(op + g * P.o_sh + dim);
          part += o.x * do_s[g * d + dim] + o.y * do_s[g * d + dim + 1];
        }
      }
    }
    delta[g] = warp_sum(part);
    lse[g] = g < G ? P.lse[((int64_t)b * P.q_heads + grp * G + g) * P.seq + i] : 0.f;
    dq[g][0][0] = dq[g][0][1] = dq[g][1][0] = dq[g][1][1] = 0.f;
  }

  TaskRuns<BR> runs;
  runs.init(P, b, grp, i);
  const float p_uniform = runs.total_keys > 0 ? 1.f / (float)runs.total_keys : 0.f;
  for (int r = 0; r < runs.count; ++r) {
    const Run run = runs.get(P, b, grp, i, r);
    float slot_part = 0.f;
    for (int t0 = run.start; t0 < run.end; t0 += 32) {
      const int pos = t0 + lane;
      const bool present = pos < run.end;
      const bool real = present && pos < P.key_rows;
      float s[GT], dp[GT], p[GT], ds[GT];
#pragma unroll
      for (int g = 0; g < GT; ++g) s[g] = dp[g] = 0.f;
      if (real) {
        if (!runs.uniform) dot_rows<T, GT>(s, q_s, kb + (int64_t)pos * P.k_sn, d);
        dot_rows<T, GT>(dp, do_s, vb + (int64_t)pos * P.v_sn, d);
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        s[g] *= P.scale;
        if (runs.uniform) {
          p[g] = present ? p_uniform : 0.f;
          ds[g] = 0.f;
        } else {
          p[g] = (present && g < G) ? exp2f((s[g] - lse[g]) * kLog2e) : 0.f;
          ds[g] = p[g] * (dp[g] - delta[g]);
          slot_part += ds[g] * s[g];
          ds[g] *= P.scale;
        }
      }
      const int cnt = min(32, min(run.end, P.key_rows) - t0);
      for (int kk = 0; kk < cnt; ++kk) {
        const int64_t row = t0 + kk;
        const T* krow = kb + row * P.k_sn;
        float2 kv[2], gk[2], gv[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int dim = 64 * c + 2 * lane;
          kv[c] = dim < d ? Elem<T>::load2(krow + dim) : make_float2(0.f, 0.f);
          gk[c] = gv[c] = make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          const float dsg = __shfl_sync(kFullMask, ds[g], kk);
          const float pg = __shfl_sync(kFullMask, p[g], kk);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int dim = 64 * c + 2 * lane;
            if (dim < d) {
              dq[g][c][0] = fmaf(dsg, kv[c].x, dq[g][c][0]);
              dq[g][c][1] = fmaf(dsg, kv[c].y, dq[g][c][1]);
              const float2 qv = *reinterpret_cast<const float2*>(q_s + g * d + dim);
              const float2 dv = *reinterpret_cast<const float2*>(do_s + g * d + dim);
              gk[c].x = fmaf(dsg, qv.x, gk[c].x);
              gk[c].y = fmaf(dsg, qv.y, gk[c].y);
              gv[c].x = fmaf(pg, dv.x, gv[c].x);
              gv[c].y = fmaf(pg, dv.y, gv[c].y);
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int dim = 64 * c + 2 * lane;
          if (dim < d) {
            if (!runs.uniform) atomicAdd(reinterpret_cast<float2*>(dkb + row * d + dim), gk[c]);
            atomicAdd(reinterpret_cast<float2*>(dvb + row * d + dim), gv[c]);
          }
        }
      }
    }
    if (BR == BR_SEL && P.slot_grads != nullptr && run.slot >= 0) {
      const float total = warp_sum(slot_part);
      if (lane == 0)
        P.slot_grads[(((int64_t)b * P.groups + grp) * P.seq + i) * P.nsel + run.slot] = total;
    }
  }

  float* dqp = P.dq + (((int64_t)b * P.q_heads + grp * G) * P.seq + i) * d;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (g >= G) break;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int dim = 64 * c + 2 * lane;
      if (dim < d)
        *reinterpret_cast<float2*>(dqp + (int64_t)g * P.seq * d + dim) = make_float2(dq[g][c][0], dq[g][c][1]);
    }
  }
}

// ---- host side --------------------------------------------------------------

template <typename T, int GT, int BR>
static int launch_one(const AttnParams& P, bool backward, cudaStream_t stream) {
  const int64_t ntasks = (int64_t)P.batch * P.groups * P.seq;
  if (ntasks == 0) return NSA_OK;
  const int64_t blocks = (ntasks + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return fail(NSA_ERR_SHAPE, "too many (batch, head, query) tasks for one launch");
  const size_t smem = (size_t)kWarpsPerBlock * GT * P.d * sizeof(float) * (backward ? 2 : 1);
  cudaError_t err;
  if (backward) {
    auto kern = attend_bwd_kernel<T, GT, BR>;
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
    kern<<<(unsigned)blocks, kWarpsPerBlock * 32, smem, stream>>>(P);
  } else {
    auto kern = attend_fwd_kernel<T, GT, BR>;
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
    kern<<<(unsigned)blocks, kWarpsPerBlock * 32, smem, stream>>>(P);
  }
  count_launches(1);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
  return NSA_OK;
}

template <typename T, int BR>
static int launch_gt(const AttnParams& P, bool backward, cudaStream_t stream) {
  const int G = P.q_heads / P.groups;
  if (G <= 1) return launch_one<T, 1, BR>(P, backward, stream);
  if (G <= 2) return launch_one<T, 2, BR>(P, backward, stream);
  if (G <= 4) return launch_one<T, 4, BR>(P, backward, stream);
  if (G <= 8) return launch_one<T, 8, BR>(P, backward, stream);
  if (G <= 16) return launch_one<T, 16, BR>(P, backward, stream);
  return fail(NSA_ERR_UNSUPPORTED, "more than 16 query heads per group");
}

int simt_attend(const AttnParams& P, int branch, int dtype, bool backward, cudaStream_t stream) {
  if (dtype == NSA_F32) {
    if (branch == BR_SEL) return launch_gt<float, BR_SEL>(P, backward, stream);
    if (branch == BR_CMP) return launch_gt<float, BR_CMP>(P, backward, stream);
    return launch_gt<float, BR_SWA>(P, backward, stream);
  }
  if (branch == BR_SEL) return launch_gt<__nv_bfloat16, BR_SEL>(P, backward, stream);
  if (branch == BR_CMP) return launch_gt<__nv_bfloat16, BR_CMP>(P, backward, stream);
  return launch_gt<__nv_bfloat16, BR_SWA>(P, backward, stream);
}

}  // namespace nsa
