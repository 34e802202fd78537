// Internal interface between the C ABI layer and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "nsa_b200.h"

namespace nsa {

enum { BR_SEL = 0, BR_CMP = 1, BR_SWA = 2 };

// Parameters of the generic attention kernels (all three branches).
struct AttnParams {
  const void *q, *k, *v, *dout;
  void* out;
  int64_t q_sb, q_sh, q_sn;
  int64_t k_sb, k_sh, k_sn;
  int64_t v_sb, v_sh, v_sn;
  int64_t o_sb, o_sh, o_sn;
  int64_t do_sb, do_sh, do_sn;
  float* lse;
  float *dq, *dk, *dv;  // contiguous fp32; dk/dv have `key_rows` rows per head
  float* slot_grads;
  int batch, q_heads, kv_heads, groups, seq, d;
  int key_rows;  // rows of k/v per head (seq, or num_mem + ncb)
  float scale;
  // selected branch
  const int64_t* idx;
  const uint8_t* mask;
  int block, nsel, diag;
  // compressed branch
  int num_mem, ncb, stride, causal, imp_heads, round_bf16;
  float sentinel;
  float* importance;
  // sliding branch
  int window;
};

struct SelectParams {
  const float* imp;
  const void* pooled;      // bf16 [rows, seq, cols], instead of imp
  int causal_limit;        // columns at and past i / block are not read: probability 0
  int64_t* idx;
  float* vals;
  int rows, seq, ncb, cpf, cols, k, block, exclude_own, input_is_prob, round_bf16;
  float neg_max;
};

struct CombineParams {
  const void *o[3], *gates, *dout;
  int64_t o_sb[3], o_sh[3], o_sn[3];
  int64_t g_sb, g_sh, g_sn;
  void* out;
  void* d_o[3];
  float* d_gates;
  float* delta;            // backward, optional: [3][batch * q_heads * seq] gate x d gate
  int batch, q_heads, seq, d;
};

constexpr int kMaxGather = NSA_MAX_GATHER;
struct GatherTargets {
  void* outs[kMaxGather];
  int num_outs, multicast;
  int64_t total_features, feature_offset;
};

struct WindowParams {
  const void *x, *pos, *dout;
  void *out, *dx;
  float* dpos;
  int64_t x_sb, x_sh, x_sn;
  int64_t dx_sb, dx_sh, dx_sn;   // strides of dx
  int batch, heads, seq, d, block, stride, ncb;
};

struct RotaryParams {
  const void* x;
  void* out;
  const float *cos, *sin;
  int64_t x_sb, x_sh, x_sn;
  int64_t o_sb, o_sh, o_sn;   // strides of out
  int batch, heads, seq, d, inverse;
};

struct NormParams {
  const void* x;      // [rows, dim] rows x_stride elements apart
  const void* weight; // [dim] in the dtype of x, or fp32 when weight_f32
  void* y;            // [rows, dim] contiguous (forward)
  float* rstd;        // [rows]: written by the forward, read by the backward
  const void* dy;     // [rows, dim] contiguous (backward)
  void* dx;           // [rows, dim] contiguous (backward)
  float* dweight;     // [dim] fp32 (backward)
  int64_t rows, x_stride;
  int dim, weight_f32;
  float eps;
};

// One decoding step (see nsa_decode.cu): the newest token's queries against the caches.
struct DecodeParams {
  const void *q, *qr;            // [B, Hq, d] contiguous: un-rotated / rotated queries of the token
  const void *keys, *vals;       // [B, Hkv, T, d]: rotated keys and values, the token included
  int64_t k_sb, k_sh, k_sn, v_sb, v_sh, v_sn;
  const void *ck, *cv;           // [B, Hkv, ncb, d]: compressed blocks, without memory slots
  int64_t ck_sb, ck_sh, ck_sn, cv_sb, cv_sh, cv_sn;
  const void *mem_k, *mem_v;     // [Hkv, num_mem, d] contiguous
  const void* gates;             // [B, Hq, 3] contiguous
  void* out;                     // [B, Hq * d]
  int batch, q_heads, kv_heads, d, T, ncb, num_mem, stride, block, nsel, window;
  float scale;
};

int fail(int code, const char* msg);

// Every host function that launches kernels of this library reports how many it launched; nsa_launch_count() returns
// the running total (a benchmark reads it before and after its timed region).
void count_launches(int n);

int simt_attend(const AttnParams& P, int branch, int dtype, bool backward, cudaStream_t stream);
int launch_select(const SelectParams& P, cudaStream_t stream);
int launch_combine(const CombineParams& P, int dtype, bool backward, cudaStream_t stream);
int launch_rotary(const RotaryParams& P, int dtype, cudaStream_t stream);
int launch_windows(const WindowParams& P, int dtype, bool backward, cudaStream_t stream);
int launch_rmsnorm(const NormParams& P, int dtype, bool backward, cudaStream_t stream);
int launch_combine_gather(const CombineParams& P, const GatherTargets& Gt, int dtype, cudaStream_t stream);
int launch_decode(const DecodeParams& P, int dtype, cudaStream_t stream);

// Tensor-core family for the selected-block branch.  Each returns
// NSA_ERR_UNSUPPORTED (without touching the error message state of a later
// successful call) when the shape is outside what it serves.
int64_t sm100_sel_workspace_bytes(const nsa_sel_fwd_args& a, bool backward);
int64_t sm100_sel_index_bytes(const nsa_sel_fwd_args& a);
int64_t sm100_swa_index_bytes(const nsa_swa_fwd_args& a);
int64_t sm100_cmp_index_bytes(const nsa_cmp_fwd_args& a);
int sm100_sel_fwd(const nsa_sel_fwd_args& a, cudaStream_t stream);
int sm100_sel_bwd(const nsa_sel_bwd_args& a, cudaStream_t stream);
int sm100_sel_fwd_static(const nsa_sel_fwd_args& a, cudaStream_t stream);
int64_t sm100_swa_workspace_bytes(const nsa_swa_fwd_args& a, bool backward);
int sm100_swa_fwd(const nsa_swa_fwd_args& a, cudaStream_t stream);
int sm100_swa_bwd(const nsa_swa_bwd_args& a, cudaStream_t stream);
int64_t sm100_cmp_workspace_bytes(const nsa_cmp_fwd_args& a, bool backward);
int sm100_cmp_fwd(const nsa_cmp_fwd_args& a, cudaStream_t stream);
bool sm100_cmp_fwd_pools(const nsa_cmp_fwd_args& a);
int sm100_sel_fwd_combine(const nsa_sel_fwd_args& a, const CombineParams& c, const GatherTargets& t, cudaStream_t stream);
int sm100_cmp_bwd(const nsa_cmp_bwd_args& a, cudaStream_t stream);
int64_t sm100_static_scratch_bytes();
int sm100_sel_static_status(int* out, cudaStream_t stream);
int sm100_wait_selftest(int* status_device, int64_t limit_cycles, cudaStream_t stream);
bool sm100_sel_bwd_overwrites_dq(const nsa_sel_fwd_args& a);
bool sm100_swa_bwd_overwrites_dq(const nsa_swa_fwd_args& a);
bool sm100_cmp_bwd_overwrites_dq(const nsa_cmp_fwd_args& a);

}  // namespace nsa
