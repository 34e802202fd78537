// extern "C" entry points: argument checks, family dispatch, launches.

#include <stdio.h>
#include <string.h>

#include <atomic>

#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

static thread_local char g_error[256] = "";

int fail(int code, const char* msg) {
  snprintf(g_error, sizeof(g_error), "%s", msg ? msg : "");
  return code;
}

static std::atomic<long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A [B,H,N,d] view is usable when rows start on 16-byte boundaries.
static int check_tensor(const nsa_tensor& t, int dtype, const char* name) {
  static thread_local char msg[128];
  if (t.ptr == nullptr) {
    snprintf(msg, sizeof(msg), "%s: NULL pointer", name);
    return fail(NSA_ERR_NULL, msg);
  }
  const int64_t per16 = dtype == NSA_F32 ? 4 : 8;
  if (!aligned16(t.ptr) || t.stride_b % per16 || t.stride_h % per16 || t.stride_n % per16) {
    snprintf(msg, sizeof(msg), "%s: pointer and strides must keep every row 16-byte aligned", name);
    return fail(NSA_ERR_ALIGN, msg);
  }
  return NSA_OK;
}

static int check_common(int dtype, int batch, int q_heads, int kv_heads, int seq, int d) {
  if (dtype != NSA_F32 && dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  if (batch < 0 || seq < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads)
    return fail(NSA_ERR_SHAPE, "batch/seq must be >= 0 and q_heads a positive multiple of kv_heads");
  if (d <= 0 || d > 128 || d % 8) return fail(NSA_ERR_SHAPE, "dim_head must be a multiple of 8, at most 128");
  return NSA_OK;
}

#define NSA_TRY(expr)            \
  do {                           \
    const int rc_ = (expr);      \
    if (rc_ != NSA_OK) return rc_; \
  } while (0)

static void set_qkvo(AttnParams& P, const nsa_tensor& q, const nsa_tensor& k, const nsa_tensor& v, const nsa_tensor& o) {
  P.q = q.ptr; P.q_sb = q.stride_b; P.q_sh = q.stride_h; P.q_sn = q.stride_n;
  P.k = k.ptr; P.k_sb = k.stride_b; P.k_sh = k.stride_h; P.k_sn = k.stride_n;
  P.v = v.ptr; P.v_sb = v.stride_b; P.v_sh = v.stride_h; P.v_sn = v.stride_n;
  P.out = o.ptr; P.o_sb = o.stride_b; P.o_sh = o.stride_h; P.o_sn = o.stride_n;
}

static void set_dout(AttnParams& P, const nsa_tensor& t) {
  P.dout = t.ptr; P.do_sb = t.stride_b; P.do_sh = t.stride_h; P.do_sn = t.stride_n;
}

static int zero_async(float* p, int64_t count, cudaStream_t stream) {
  if (count == 0) return NSA_OK;
  const cudaError_t err = cudaMemsetAsync(p, 0, (size_t)count * sizeof(float), stream);
  return err == cudaSuccess ? NSA_OK : fail((int)err, cudaGetErrorString(err));
}

// ---- selected-block branch ---------------------------------------------------

static int fill_sel(AttnParams& P, const nsa_sel_fwd_args& a) {
  NSA_TRY(check_common(a.dtype, a.batch, a.q_heads, a.kv_heads, a.seq, a.dim_head));
  if (a.sel_heads != a.kv_heads && a.sel_heads != a.q_heads)
    return fail(NSA_ERR_SHAPE, "sel_heads must equal kv_heads or q_heads");
  if (a.block <= 0 || a.nsel < 0) return fail(NSA_ERR_SHAPE, "block must be > 0 and nsel >= 0");
  if (a.diag < NSA_DIAG_NONE || a.diag > NSA_DIAG_FULL) return fail(NSA_ERR_SHAPE, "unknown diag mode");
  if (a.impl < NSA_IMPL_AUTO || a.impl > NSA_IMPL_SM100) return fail(NSA_ERR_SHAPE, "unknown impl");
  NSA_TRY(check_tensor(a.q, a.dtype, "q"));
  NSA_TRY(check_tensor(a.k, a.dtype, "k"));
  NSA_TRY(check_tensor(a.v, a.dtype, "v"));
  NSA_TRY(check_tensor(a.out, a.dtype, "out"));
  if (a.lse == nullptr) return fail(NSA_ERR_NULL, "lse: NULL pointer");
  if (a.nsel > 0 && (a.idx == nullptr || a.mask == nullptr)) return fail(NSA_ERR_NULL, "idx/mask: NULL pointer");
  memset(&P, 0, sizeof(P));
  set_qkvo(P, a.q, a.k, a.v, a.out);
  P.lse = a.lse;
  P.batch = a.batch; P.q_heads = a.q_heads; P.kv_heads = a.kv_heads; P.groups = a.sel_heads;
  P.seq = a.seq; P.d = a.dim_head; P.key_rows = a.seq; P.scale = a.scale;
  P.idx = a.idx; P.mask = a.mask; P.block = a.block; P.nsel = a.nsel; P.diag = a.diag;
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" {

int nsa_abi_version(void) { return 1; }

const char* nsa_last_error(void) { return g_error; }

int nsa_struct_size(int which) {
  switch (which) {
    case 0: return (int)sizeof(nsa_tensor);
    case 1: return (int)sizeof(nsa_sel_fwd_args);
    case 2: return (int)sizeof(nsa_sel_bwd_args);
    case 3: return (int)sizeof(nsa_cmp_fwd_args);
    case 4: return (int)sizeof(nsa_cmp_bwd_args);
    case 5: return (int)sizeof(nsa_select_args);
    case 6: return (int)sizeof(nsa_swa_fwd_args);
    case 7: return (int)sizeof(nsa_swa_bwd_args);
    case 8: return (int)sizeof(nsa_combine_fwd_args);
    case 9: return (int)sizeof(nsa_combine_bwd_args);
    case 10: return (int)sizeof(nsa_combine_gather_args);
    case 11: return (int)sizeof(nsa_rotary_args);
    case 12: return (int)sizeof(nsa_windows_fwd_args);
    case 13: return (int)sizeof(nsa_windows_bwd_args);
    case 14: return (int)sizeof(nsa_rmsnorm_fwd_args);
    case 15: return (int)sizeof(nsa_rmsnorm_bwd_args);
    case 16: return (int)sizeof(nsa_decode_args);
    default: return -1;
  }
}

int64_t nsa_sel_workspace_bytes(const nsa_sel_fwd_args* a, int backward) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  const int rc = fill_sel(P, *a);
  if (rc != NSA_OK && rc != NSA_ERR_NULL) return rc;
  if (a->impl == NSA_IMPL_SIMT) return 0;
  const int64_t need = sm100_sel_workspace_bytes(*a, backward != 0);
  if (need < 0) return a->impl == NSA_IMPL_SM100 ? need : 0;
  return need;
}

// dq_out: rows of dim_head elements in the dtype of q; only the tensor-core family at dim_head 64 writes it
static int check_dq_out(const nsa_tensor& t, int dtype, bool served) {
  if (t.ptr == nullptr) return NSA_OK;
  if (!served) return fail(NSA_ERR_UNSUPPORTED, "dq_out: this problem's backward does not store dq in one pass (see *_bwd_stores_dq)");
  return check_tensor(t, dtype, "dq_out");
}

int nsa_sel_bwd_stores_dq(const nsa_sel_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  return a->impl != NSA_IMPL_SIMT && sm100_sel_bwd_overwrites_dq(*a) ? 1 : 0;
}
int nsa_cmp_bwd_stores_dq(const nsa_cmp_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  return a->impl != NSA_IMPL_SIMT && sm100_cmp_bwd_overwrites_dq(*a) ? 1 : 0;
}
int nsa_swa_bwd_stores_dq(const nsa_swa_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  return a->impl != NSA_IMPL_SIMT && sm100_swa_bwd_overwrites_dq(*a) ? 1 : 0;
}

int64_t nsa_cmp_index_bytes(const nsa_cmp_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  return a->impl == NSA_IMPL_SIMT ? 0 : sm100_cmp_index_bytes(*a);
}
int64_t nsa_swa_index_bytes(const nsa_swa_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  return a->impl == NSA_IMPL_SIMT ? 0 : sm100_swa_index_bytes(*a);
}

int64_t nsa_sel_index_bytes(const nsa_sel_fwd_args* a) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  const int rc = fill_sel(P, *a);
  if (rc != NSA_OK && rc != NSA_ERR_NULL) return rc;
  if (a->impl == NSA_IMPL_SIMT) return 0;
  return sm100_sel_index_bytes(*a);
}

int nsa_sel_fwd(const nsa_sel_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_sel(P, *a));
  if (a->index != nullptr && (reinterpret_cast<uintptr_t>(a->index) & 15u))
    return fail(NSA_ERR_ALIGN, "index must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  if (a->impl != NSA_IMPL_SIMT) {
    const int rc = sm100_sel_fwd(*a, st);
    if (rc != NSA_ERR_UNSUPPORTED || a->impl == NSA_IMPL_SM100) return rc;
  }
  return simt_attend(P, BR_SEL, a->dtype, false, st);
}

int nsa_sel_fwd_static(const nsa_sel_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_sel(P, *a));
  return sm100_sel_fwd_static(*a, (cudaStream_t)stream);
}

int64_t nsa_sel_static_scratch_bytes(void) { return sm100_static_scratch_bytes(); }

int nsa_sel_static_status(int* out, void* stream) { return sm100_sel_static_status(out, (cudaStream_t)stream); }

int nsa_decode_step(const nsa_decode_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  NSA_TRY(check_common(a->dtype, a->batch, a->q_heads, a->kv_heads, a->cache_len, a->dim_head));
  if (a->cache_len < 1) return fail(NSA_ERR_SHAPE, "decode step: the caches hold at least the new token");
  if (a->stride < 1 || a->block < a->stride || a->block % a->stride || a->nsel < 0 || a->nsel > 32 || a->window < 0 ||
      a->ncb < 0 || a->num_mem < 1)
    return fail(NSA_ERR_SHAPE, "decode step: stride / block / nsel (<= 32) / window / ncb / num_mem out of range");
  if ((int64_t)a->ncb * a->stride > a->cache_len)
    return fail(NSA_ERR_SHAPE, "decode step: more compressed blocks than the cache length allows");
  if (!a->q || !a->qr || !a->gates || !a->out || !a->mem_k || !a->mem_v) return fail(NSA_ERR_NULL, "decode step: NULL pointer");
  NSA_TRY(check_tensor(a->keys, a->dtype, "keys"));
  NSA_TRY(check_tensor(a->vals, a->dtype, "vals"));
  if (a->ncb > 0) {
    NSA_TRY(check_tensor(a->ck, a->dtype, "ck"));
    NSA_TRY(check_tensor(a->cv, a->dtype, "cv"));
  }
  const void* small[] = {a->q, a->qr, a->mem_k, a->mem_v, a->out};
  for (const void* p : small)
    if (!aligned16(p)) return fail(NSA_ERR_ALIGN, "decode step: q, qr, mem_k, mem_v, out must be 16-byte aligned");
  DecodeParams P;
  memset(&P, 0, sizeof(P));
  P.q = a->q; P.qr = a->qr; P.gates = a->gates; P.out = a->out; P.mem_k = a->mem_k; P.mem_v = a->mem_v;
  P.keys = a->keys.ptr; P.k_sb = a->keys.stride_b; P.k_sh = a->keys.stride_h; P.k_sn = a->keys.stride_n;
  P.vals = a->vals.ptr; P.v_sb = a->vals.stride_b; P.v_sh = a->vals.stride_h; P.v_sn = a->vals.stride_n;
  P.ck = a->ck.ptr; P.ck_sb = a->ck.stride_b; P.ck_sh = a->ck.stride_h; P.ck_sn = a->ck.stride_n;
  P.cv = a->cv.ptr; P.cv_sb = a->cv.stride_b; P.cv_sh = a->cv.stride_h; P.cv_sn = a->cv.stride_n;
  P.batch = a->batch; P.q_heads = a->q_heads; P.kv_heads = a->kv_heads; P.d = a->dim_head; P.T = a->cache_len;
  P.ncb = a->ncb; P.num_mem = a->num_mem; P.stride = a->stride; P.block = a->block; P.nsel = a->nsel;
  P.window = a->window; P.scale = a->scale;
  return launch_decode(P, a->dtype, (cudaStream_t)stream);
}

int64_t nsa_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int nsa_selftest_bounded_wait(int* status_device, int64_t limit_cycles, void* stream) {
  return sm100_wait_selftest(status_device, limit_cycles, (cudaStream_t)stream);
}

int nsa_sel_bwd(const nsa_sel_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_sel(P, a->fwd));
  NSA_TRY(check_tensor(a->dout, a->fwd.dtype, "dout"));
  // dk and dv are accumulated into; dq too, unless the kernels that will run store every row of it
  const bool dq_stored = a->fwd.impl != NSA_IMPL_SIMT && sm100_sel_bwd_overwrites_dq(a->fwd);
  NSA_TRY(check_dq_out(a->dq_out, a->fwd.dtype, dq_stored));
  if ((!a->dq && !a->dq_out.ptr) || !a->dk || !a->dv) return fail(NSA_ERR_NULL, "dq/dk/dv: NULL pointer");
  if (a->index != nullptr && (reinterpret_cast<uintptr_t>(a->index) & 15u))
    return fail(NSA_ERR_ALIGN, "index must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t d = a->fwd.dim_head, n = a->fwd.seq, b = a->fwd.batch;
  if (!dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * n * d, st));
  NSA_TRY(zero_async(a->dk, b * a->fwd.kv_heads * n * d, st));
  NSA_TRY(zero_async(a->dv, b * a->fwd.kv_heads * n * d, st));
  if (a->fwd.impl != NSA_IMPL_SIMT) {
    const int rc = sm100_sel_bwd(*a, st);
    if (rc != NSA_ERR_UNSUPPORTED || a->fwd.impl == NSA_IMPL_SM100) return rc;
    if (a->dq == nullptr) return fail(NSA_ERR_UNSUPPORTED, "the tensor-core kernels could not take these tensors; pass an fp32 dq");
    if (dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * n * d, st));
  }
  set_dout(P, a->dout);
  P.dq = a->dq; P.dk = a->dk; P.dv = a->dv; P.slot_grads = a->slot_grads;
  return simt_attend(P, BR_SEL, a->fwd.dtype, true, st);
}

// ---- compressed branch -------------------------------------------------------

static int fill_cmp(AttnParams& P, const nsa_cmp_fwd_args& a) {
  NSA_TRY(check_common(a.dtype, a.batch, a.q_heads, a.kv_heads, a.seq, a.dim_head));
  if (a.sel_heads != a.kv_heads && a.sel_heads != a.q_heads)
    return fail(NSA_ERR_SHAPE, "sel_heads must equal kv_heads or q_heads");
  if (a.num_mem < 1 || a.ncb < 0 || a.stride <= 0) return fail(NSA_ERR_SHAPE, "need num_mem >= 1, ncb >= 0, stride > 0");
  NSA_TRY(check_tensor(a.q, a.dtype, "q"));
  NSA_TRY(check_tensor(a.ck, a.dtype, "ck"));
  NSA_TRY(check_tensor(a.cv, a.dtype, "cv"));
  NSA_TRY(check_tensor(a.out, a.dtype, "out"));
  if (a.lse == nullptr) return fail(NSA_ERR_NULL, "lse: NULL pointer");
  memset(&P, 0, sizeof(P));
  set_qkvo(P, a.q, a.ck, a.cv, a.out);
  P.lse = a.lse;
  P.batch = a.batch; P.q_heads = a.q_heads; P.kv_heads = a.kv_heads; P.groups = a.kv_heads;
  P.seq = a.seq; P.d = a.dim_head; P.key_rows = a.num_mem + a.ncb; P.scale = a.scale;
  P.num_mem = a.num_mem; P.ncb = a.ncb; P.stride = a.stride; P.causal = a.causal;
  P.imp_heads = a.sel_heads; P.round_bf16 = a.dtype == NSA_BF16; P.sentinel = a.sentinel;
  P.importance = a.importance;
  return NSA_OK;
}

int64_t nsa_cmp_workspace_bytes(const nsa_cmp_fwd_args* a, int backward) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  if (a->impl == NSA_IMPL_SIMT) return 0;
  const int64_t need = sm100_cmp_workspace_bytes(*a, backward != 0);
  if (need < 0) return a->impl == NSA_IMPL_SM100 ? need : 0;
  return need;
}

int nsa_cmp_fwd_pools(const nsa_cmp_fwd_args* a) {
  if (a == nullptr) return 0;
  return sm100_cmp_fwd_pools(*a) ? 1 : 0;
}

int nsa_cmp_fwd(const nsa_cmp_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_cmp(P, *a));
  if (a->pooled != nullptr) {
    if (a->importance != nullptr) return fail(NSA_ERR_SHAPE, "pass importance or pooled, not both");
    if (reinterpret_cast<uintptr_t>(a->pooled) & 1u) return fail(NSA_ERR_ALIGN, "pooled must be 2-byte aligned");
    if (!sm100_cmp_fwd_pools(*a))
      return fail(NSA_ERR_UNSUPPORTED, "pooled: not served for these arguments (nsa_cmp_fwd_pools); pass importance");
  }
  if (a->impl != NSA_IMPL_SIMT) {
    const int rc = sm100_cmp_fwd(*a, (cudaStream_t)stream);
    if (rc != NSA_ERR_UNSUPPORTED) return rc;
    if (a->impl == NSA_IMPL_SM100) return fail(NSA_ERR_UNSUPPORTED, "compressed branch: shape outside the tensor-core family");
  }
  return simt_attend(P, BR_CMP, a->dtype, false, (cudaStream_t)stream);
}

int nsa_cmp_bwd(const nsa_cmp_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_cmp(P, a->fwd));
  NSA_TRY(check_tensor(a->dout, a->fwd.dtype, "dout"));
  const bool dq_stored = a->fwd.impl != NSA_IMPL_SIMT && sm100_cmp_bwd_overwrites_dq(a->fwd);
  NSA_TRY(check_dq_out(a->dq_out, a->fwd.dtype, dq_stored));
  if ((!a->dq && !a->dq_out.ptr) || !a->dck || !a->dcv) return fail(NSA_ERR_NULL, "dq/dck/dcv: NULL pointer");
  if (a->index != nullptr && (reinterpret_cast<uintptr_t>(a->index) & 15u))
    return fail(NSA_ERR_ALIGN, "index must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t d = a->fwd.dim_head, rows = a->fwd.num_mem + a->fwd.ncb, b = a->fwd.batch;
  if (!dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * a->fwd.seq * d, st));
  NSA_TRY(zero_async(a->dck, b * a->fwd.kv_heads * rows * d, st));
  NSA_TRY(zero_async(a->dcv, b * a->fwd.kv_heads * rows * d, st));
  if (a->fwd.impl != NSA_IMPL_SIMT) {
    const int rc = sm100_cmp_bwd(*a, st);
    if (rc != NSA_ERR_UNSUPPORTED) return rc;
    if (a->fwd.impl == NSA_IMPL_SM100) return fail(NSA_ERR_UNSUPPORTED, "compressed branch: shape outside the tensor-core family");
    if (a->dq == nullptr) return fail(NSA_ERR_UNSUPPORTED, "the tensor-core kernels could not take these tensors; pass an fp32 dq");
    if (dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * a->fwd.seq * d, st));
  }
  set_dout(P, a->dout);
  P.importance = nullptr;
  P.dq = a->dq; P.dk = a->dck; P.dv = a->dcv;
  return simt_attend(P, BR_CMP, a->fwd.dtype, true, st);
}

// ---- selection -----------------------------------------------------------------

int nsa_select(const nsa_select_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  if (a->dtype != NSA_F32 && a->dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  if (a->rows < 0 || a->seq < 0 || a->ncb < 0 || a->cpf < 1 || a->block <= 0 || a->k < 0)
    return fail(NSA_ERR_SHAPE, "negative size, cpf < 1 or block <= 0");
  const int cols = a->ncb / a->cpf;
  if (a->k > cols) return fail(NSA_ERR_SHAPE, "k exceeds the number of block columns");
  if (a->input_is_prob && a->cpf != 1) return fail(NSA_ERR_SHAPE, "input_is_prob needs cpf == 1");
  if ((!a->importance && !a->pooled) || !a->idx || !a->vals) return fail(NSA_ERR_NULL, "importance/idx/vals: NULL pointer");
  if (a->pooled != nullptr && (a->importance != nullptr || a->cpf != 1 || a->input_is_prob))
    return fail(NSA_ERR_SHAPE, "pooled excludes importance and input_is_prob and needs cpf == 1");
  SelectParams P;
  P.imp = a->importance; P.idx = a->idx; P.vals = a->vals;
  P.pooled = a->pooled; P.causal_limit = (a->pooled != nullptr || a->causal_limit) ? 1 : 0;
  P.rows = a->rows; P.seq = a->seq; P.ncb = a->ncb; P.cpf = a->cpf; P.cols = cols; P.k = a->k;
  P.block = a->block; P.exclude_own = a->exclude_own; P.input_is_prob = a->input_is_prob;
  P.round_bf16 = a->dtype == NSA_BF16;
  P.neg_max = a->dtype == NSA_BF16 ? -3.3895313892515355e38f : -FLT_MAX;
  return launch_select(P, (cudaStream_t)stream);
}

// ---- sliding window ------------------------------------------------------------

static int fill_swa(AttnParams& P, const nsa_swa_fwd_args& a) {
  NSA_TRY(check_common(a.dtype, a.batch, a.q_heads, a.kv_heads, a.seq, a.dim_head));
  if (a.window < 0) return fail(NSA_ERR_SHAPE, "window must be >= 0");
  NSA_TRY(check_tensor(a.q, a.dtype, "q"));
  NSA_TRY(check_tensor(a.k, a.dtype, "k"));
  NSA_TRY(check_tensor(a.v, a.dtype, "v"));
  NSA_TRY(check_tensor(a.out, a.dtype, "out"));
  if (a.lse == nullptr) return fail(NSA_ERR_NULL, "lse: NULL pointer");
  memset(&P, 0, sizeof(P));
  set_qkvo(P, a.q, a.k, a.v, a.out);
  P.lse = a.lse;
  P.batch = a.batch; P.q_heads = a.q_heads; P.kv_heads = a.kv_heads; P.groups = a.kv_heads;
  P.seq = a.seq; P.d = a.dim_head; P.key_rows = a.seq; P.scale = a.scale;
  P.window = a.window; P.causal = a.causal;
  return NSA_OK;
}

int64_t nsa_swa_workspace_bytes(const nsa_swa_fwd_args* a, int backward) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  if (a->impl == NSA_IMPL_SIMT) return 0;
  const int64_t need = sm100_swa_workspace_bytes(*a, backward != 0);
  if (need < 0) return a->impl == NSA_IMPL_SM100 ? need : 0;
  return need;
}

int nsa_swa_fwd(const nsa_swa_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_swa(P, *a));
  if (a->impl != NSA_IMPL_SIMT) {
    const int rc = sm100_swa_fwd(*a, (cudaStream_t)stream);
    if (rc != NSA_ERR_UNSUPPORTED) return rc;
    if (a->impl == NSA_IMPL_SM100) return fail(NSA_ERR_UNSUPPORTED, "sliding branch: shape outside the tensor-core family");
  }
  return simt_attend(P, BR_SWA, a->dtype, false, (cudaStream_t)stream);
}

int nsa_swa_bwd(const nsa_swa_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  AttnParams P;
  NSA_TRY(fill_swa(P, a->fwd));
  NSA_TRY(check_tensor(a->dout, a->fwd.dtype, "dout"));
  const bool dq_stored = a->fwd.impl != NSA_IMPL_SIMT && sm100_swa_bwd_overwrites_dq(a->fwd);
  NSA_TRY(check_dq_out(a->dq_out, a->fwd.dtype, dq_stored));
  if ((!a->dq && !a->dq_out.ptr) || !a->dk || !a->dv) return fail(NSA_ERR_NULL, "dq/dk/dv: NULL pointer");
  if (a->index != nullptr && (reinterpret_cast<uintptr_t>(a->index) & 15u))
    return fail(NSA_ERR_ALIGN, "index must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t d = a->fwd.dim_head, n = a->fwd.seq, b = a->fwd.batch;
  if (!dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * n * d, st));
  NSA_TRY(zero_async(a->dk, b * a->fwd.kv_heads * n * d, st));
  NSA_TRY(zero_async(a->dv, b * a->fwd.kv_heads * n * d, st));
  if (a->fwd.impl != NSA_IMPL_SIMT) {
    const int rc = sm100_swa_bwd(*a, st);
    if (rc != NSA_ERR_UNSUPPORTED) return rc;
    if (a->fwd.impl == NSA_IMPL_SM100) return fail(NSA_ERR_UNSUPPORTED, "sliding branch: shape outside the tensor-core family");
    if (a->dq == nullptr) return fail(NSA_ERR_UNSUPPORTED, "the tensor-core kernels could not take these tensors; pass an fp32 dq");
    if (dq_stored) NSA_TRY(zero_async(a->dq, b * a->fwd.q_heads * n * d, st));
  }
  set_dout(P, a->dout);
  P.dq = a->dq; P.dk = a->dk; P.dv = a->dv;
  return simt_attend(P, BR_SWA, a->fwd.dtype, true, st);
}

// ---- combine ---------------------------------------------------------------------

static int fill_combine(CombineParams& P, const nsa_combine_fwd_args& a) {
  if (a.dtype != NSA_F32 && a.dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  if (a.batch < 0 || a.seq < 0 || a.q_heads <= 0 || a.dim_head <= 0 || a.dim_head % 2)
    return fail(NSA_ERR_SHAPE, "negative size or odd dim_head");
  const nsa_tensor* o[3] = {&a.o_cmp, &a.o_sel, &a.o_swa};
  memset(&P, 0, sizeof(P));
  for (int s = 0; s < 3; ++s) {
    if (o[s]->ptr == nullptr) return fail(NSA_ERR_NULL, "branch output: NULL pointer");
    if ((reinterpret_cast<uintptr_t>(o[s]->ptr) & 7u) || o[s]->stride_b % 2 || o[s]->stride_h % 2 || o[s]->stride_n % 2)
      return fail(NSA_ERR_ALIGN, "branch outputs must keep feature pairs aligned");
    P.o[s] = o[s]->ptr; P.o_sb[s] = o[s]->stride_b; P.o_sh[s] = o[s]->stride_h; P.o_sn[s] = o[s]->stride_n;
  }
  if (a.gates.ptr == nullptr) return fail(NSA_ERR_NULL, "gates: NULL pointer");
  P.gates = a.gates.ptr; P.g_sb = a.gates.stride_b; P.g_sh = a.gates.stride_h; P.g_sn = a.gates.stride_n;
  P.batch = a.batch; P.q_heads = a.q_heads; P.seq = a.seq; P.d = a.dim_head;
  return NSA_OK;
}

int nsa_combine_fwd(const nsa_combine_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  CombineParams P;
  NSA_TRY(fill_combine(P, *a));
  if (a->out == nullptr) return fail(NSA_ERR_NULL, "out: NULL pointer");
  P.out = a->out;
  // 16-byte pieces when everything is aligned for them (the usual case), feature pairs otherwise
  const int V = a->dtype == NSA_F32 ? 4 : 8;
  bool vec = a->dim_head % V == 0 && (reinterpret_cast<uintptr_t>(a->out) & 15u) == 0;
  const nsa_tensor* o[3] = {&a->o_cmp, &a->o_sel, &a->o_swa};
  for (int s = 0; s < 3; ++s)
    vec = vec && (reinterpret_cast<uintptr_t>(o[s]->ptr) & 15u) == 0 && o[s]->stride_b % V == 0 &&
          o[s]->stride_h % V == 0 && o[s]->stride_n % V == 0;
  if (vec) {
    GatherTargets Gt;
    memset(&Gt, 0, sizeof(Gt));
    Gt.outs[0] = a->out;
    Gt.num_outs = 1;
    Gt.total_features = (int64_t)a->q_heads * a->dim_head;
    Gt.feature_offset = 0;
    return launch_combine_gather(P, Gt, a->dtype, (cudaStream_t)stream);
  }
  return launch_combine(P, a->dtype, false, (cudaStream_t)stream);
}

// checks of a gather call shared by nsa_combine_fwd_gather and nsa_sel_fwd_combine_gather (`skip`: a branch whose
// tensor the caller does not pass because the call computes it)
static int fill_gather(CombineParams& P, GatherTargets& Gt, const nsa_combine_gather_args& a, int skip) {
  nsa_combine_fwd_args f = a.fwd;
  nsa_tensor* o[3] = {&f.o_cmp, &f.o_sel, &f.o_swa};
  if (skip >= 0) *o[skip] = *o[(skip + 1) % 3];      // stands in for the checks only
  NSA_TRY(fill_combine(P, f));
  const int V = f.dtype == NSA_F32 ? 4 : 8;
  if (a.num_outs < 1 || a.num_outs > NSA_MAX_GATHER) return fail(NSA_ERR_SHAPE, "num_outs must be 1..NSA_MAX_GATHER");
  if (f.dim_head % V) return fail(NSA_ERR_ALIGN, "dim_head must be a multiple of 16 bytes");
  if (a.feature_offset < 0 || a.feature_offset % V || a.total_features % V ||
      a.feature_offset + (int64_t)f.q_heads * f.dim_head > a.total_features)
    return fail(NSA_ERR_SHAPE, "feature_offset / total_features do not hold these heads in 16-byte pieces");
  for (int s = 0; s < 3; ++s)
    if ((reinterpret_cast<uintptr_t>(o[s]->ptr) & 15u) || o[s]->stride_b % V || o[s]->stride_h % V || o[s]->stride_n % V)
      return fail(NSA_ERR_ALIGN, "branch outputs must keep 16-byte pieces aligned");
  memset(&Gt, 0, sizeof(Gt));
  for (int r = 0; r < a.num_outs; ++r) {
    if (a.outs[r] == nullptr) return fail(NSA_ERR_NULL, "outs: NULL pointer");
    if (reinterpret_cast<uintptr_t>(a.outs[r]) & 15u) return fail(NSA_ERR_ALIGN, "outs must be 16-byte aligned");
    Gt.outs[r] = a.outs[r];
  }
  if (a.multicast != 0 && a.num_outs != 1)
    return fail(NSA_ERR_SHAPE, "a multicast destination is the only destination (num_outs == 1)");
  Gt.num_outs = a.num_outs;
  Gt.multicast = a.multicast != 0;
  Gt.total_features = a.total_features;
  Gt.feature_offset = a.feature_offset;
  return NSA_OK;
}

int nsa_sel_fwd_combine_gather(const nsa_sel_fwd_args* s, const nsa_combine_gather_args* c, void* stream) {
  if (s == nullptr || c == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  if (s->impl == NSA_IMPL_SIMT) return fail(NSA_ERR_UNSUPPORTED, "the fused merge is part of the tensor-core family");
  nsa_sel_fwd_args sel = *s;
  if (sel.out.ptr == nullptr) sel.out = sel.q;       // never written by this call: any tensor of the shape passes the checks
  AttnParams A;
  NSA_TRY(fill_sel(A, sel));
  if (sel.index != nullptr && (reinterpret_cast<uintptr_t>(sel.index) & 15u))
    return fail(NSA_ERR_ALIGN, "index must be 16-byte aligned");
  if (c->fwd.dtype != NSA_BF16 || s->dtype != NSA_BF16) return fail(NSA_ERR_UNSUPPORTED, "the fused merge serves bf16");
  if (c->fwd.batch != s->batch || c->fwd.q_heads != s->q_heads || c->fwd.seq != s->seq || c->fwd.dim_head != s->dim_head)
    return fail(NSA_ERR_SHAPE, "the combine's sizes must be those of the selected-block call");
  CombineParams P;
  GatherTargets Gt;
  NSA_TRY(fill_gather(P, Gt, *c, 1));
  P.o[1] = nullptr;
  const int rc = sm100_sel_fwd_combine(sel, P, Gt, (cudaStream_t)stream);
  if (rc == NSA_ERR_UNSUPPORTED) return fail(NSA_ERR_UNSUPPORTED, "selected branch: shape outside the tensor-core family");
  return rc;
}

int nsa_combine_fwd_gather(const nsa_combine_gather_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  CombineParams P;
  GatherTargets Gt;
  NSA_TRY(fill_gather(P, Gt, *a, -1));
  const nsa_combine_fwd_args& f = a->fwd;
  return launch_combine_gather(P, Gt, f.dtype, (cudaStream_t)stream);
}

int nsa_combine_bwd(const nsa_combine_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  CombineParams P;
  NSA_TRY(fill_combine(P, a->fwd));
  if (!a->dout || !a->d_cmp || !a->d_sel || !a->d_swa || !a->d_gates) return fail(NSA_ERR_NULL, "gradient buffer: NULL pointer");
  P.dout = a->dout;
  P.d_o[0] = a->d_cmp; P.d_o[1] = a->d_sel; P.d_o[2] = a->d_swa;
  P.d_gates = a->d_gates;
  P.delta = a->delta;
  return launch_combine(P, a->fwd.dtype, true, (cudaStream_t)stream);
}

int nsa_rotary(const nsa_rotary_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  if (a->dtype != NSA_F32 && a->dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  const int V = a->dtype == NSA_F32 ? 4 : 8;
  if (a->batch < 0 || a->heads < 0 || a->seq < 0 || a->dim_head <= 0 || a->dim_head % V)
    return fail(NSA_ERR_SHAPE, "negative size, or dim_head not a multiple of 16 bytes");
  if ((int64_t)a->batch * a->heads * a->seq == 0) return NSA_OK;
  if (!a->x.ptr || !a->out || !a->cos_table || !a->sin_table) return fail(NSA_ERR_NULL, "tensor: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a->x.ptr) & 15u) || (reinterpret_cast<uintptr_t>(a->out) & 15u) ||
      a->x.stride_b % V || a->x.stride_h % V || a->x.stride_n % V)
    return fail(NSA_ERR_ALIGN, "x and out must keep 16-byte pieces aligned");
  RotaryParams P;
  P.x = a->x.ptr; P.out = a->out; P.cos = a->cos_table; P.sin = a->sin_table;
  P.x_sb = a->x.stride_b; P.x_sh = a->x.stride_h; P.x_sn = a->x.stride_n;
  P.batch = a->batch; P.heads = a->heads; P.seq = a->seq; P.d = a->dim_head; P.inverse = a->inverse;
  if (a->out_stride_b == 0 && a->out_stride_h == 0 && a->out_stride_n == 0) {
    P.o_sn = a->dim_head; P.o_sh = P.o_sn * a->seq; P.o_sb = P.o_sh * a->heads;
  } else {
    if (a->out_stride_b % V || a->out_stride_h % V || a->out_stride_n % V || a->out_stride_n < a->dim_head)
      return fail(NSA_ERR_ALIGN, "out strides must keep rows apart and 16-byte aligned");
    P.o_sb = a->out_stride_b; P.o_sh = a->out_stride_h; P.o_sn = a->out_stride_n;
  }
  return launch_rotary(P, a->dtype, (cudaStream_t)stream);
}

static int fill_windows(WindowParams& P, const nsa_windows_fwd_args& a) {
  if (a.dtype != NSA_F32 && a.dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  const int V = a.dtype == NSA_F32 ? 4 : 8;
  if (a.batch < 0 || a.heads < 0 || a.seq < 0 || a.ncb < 0 || a.dim_head <= 0 || a.dim_head % V || a.dim_head > 256 ||
      a.block <= 0 || a.stride <= 0 || a.block < a.stride)
    return fail(NSA_ERR_SHAPE, "sizes: negative, dim_head not a multiple of 16 bytes (or above 256), or block < stride");
  if ((int64_t)a.ncb * a.stride > a.seq) return fail(NSA_ERR_SHAPE, "ncb windows do not fit the sequence");
  if ((int64_t)a.batch * a.ncb > 0x7fffffffLL) return fail(NSA_ERR_SHAPE, "batch * ncb must stay below 2^31");
  memset(&P, 0, sizeof(P));
  P.batch = a.batch; P.heads = a.heads; P.seq = a.seq; P.d = a.dim_head; P.block = a.block; P.stride = a.stride;
  P.ncb = a.ncb;
  return NSA_OK;
}

int nsa_windows_fwd(const nsa_windows_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  WindowParams P;
  NSA_TRY(fill_windows(P, *a));
  if ((int64_t)a->batch * a->heads * a->ncb == 0) return NSA_OK;
  const int V = a->dtype == NSA_F32 ? 4 : 8;
  if (!a->x.ptr || !a->pos || !a->out) return fail(NSA_ERR_NULL, "tensor: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a->x.ptr) & 15u) || (reinterpret_cast<uintptr_t>(a->pos) & 15u) ||
      (reinterpret_cast<uintptr_t>(a->out) & 15u) || a->x.stride_b % V || a->x.stride_h % V || a->x.stride_n % V)
    return fail(NSA_ERR_ALIGN, "x, pos and out must keep 16-byte pieces aligned");
  P.x = a->x.ptr; P.x_sb = a->x.stride_b; P.x_sh = a->x.stride_h; P.x_sn = a->x.stride_n;
  P.pos = a->pos; P.out = a->out;
  return launch_windows(P, a->dtype, false, (cudaStream_t)stream);
}

int nsa_windows_bwd(const nsa_windows_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  WindowParams P;
  NSA_TRY(fill_windows(P, a->fwd));
  if (!a->dout || !a->dx || !a->dpos) return fail(NSA_ERR_NULL, "gradient buffer: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a->dout) & 15u) || (reinterpret_cast<uintptr_t>(a->dx) & 15u))
    return fail(NSA_ERR_ALIGN, "dout and dx must be 16-byte aligned");
  P.dout = a->dout; P.dx = a->dx; P.dpos = a->dpos;
  if (a->dx_stride_b == 0 && a->dx_stride_h == 0 && a->dx_stride_n == 0) {
    P.dx_sn = a->fwd.dim_head; P.dx_sh = P.dx_sn * a->fwd.seq; P.dx_sb = P.dx_sh * a->fwd.heads;
  } else {
    const int V = a->fwd.dtype == NSA_F32 ? 4 : 8;
    if (a->dx_stride_b % V || a->dx_stride_h % V || a->dx_stride_n % V || a->dx_stride_n < a->fwd.dim_head)
      return fail(NSA_ERR_ALIGN, "dx strides must keep rows apart and 16-byte aligned");
    P.dx_sb = a->dx_stride_b; P.dx_sh = a->dx_stride_h; P.dx_sn = a->dx_stride_n;
  }
  return launch_windows(P, a->fwd.dtype, true, (cudaStream_t)stream);
}

static int fill_norm(NormParams& P, const nsa_rmsnorm_fwd_args& a) {
  if (a.dtype != NSA_F32 && a.dtype != NSA_BF16) return fail(NSA_ERR_DTYPE, "dtype must be NSA_F32 or NSA_BF16");
  const int V = a.dtype == NSA_F32 ? 4 : 8;
  if (a.rows < 0 || a.dim <= 0 || a.dim % V || a.dim / V > 256 || a.x_stride < a.dim)
    return fail(NSA_ERR_SHAPE, "rows negative, dim not a multiple of 16 bytes or above 256 such pieces, or rows overlap");
  if (a.x_stride % V) return fail(NSA_ERR_ALIGN, "rows of x must start on 16-byte boundaries");
  memset(&P, 0, sizeof(P));
  P.rows = a.rows; P.x_stride = a.x_stride; P.dim = a.dim; P.weight_f32 = a.weight_f32 != 0; P.eps = a.eps;
  if (a.rows == 0) return NSA_OK;
  if (!a.x || !a.weight || !a.rstd) return fail(NSA_ERR_NULL, "tensor: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.weight) & 15u))
    return fail(NSA_ERR_ALIGN, "x and weight must be 16-byte aligned");
  P.x = a.x; P.weight = a.weight; P.rstd = a.rstd;
  return NSA_OK;
}

int nsa_rmsnorm_fwd(const nsa_rmsnorm_fwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  NormParams P;
  NSA_TRY(fill_norm(P, *a));
  if (a->rows == 0) return NSA_OK;
  if (!a->y) return fail(NSA_ERR_NULL, "y: NULL pointer");
  if (reinterpret_cast<uintptr_t>(a->y) & 15u) return fail(NSA_ERR_ALIGN, "y must be 16-byte aligned");
  P.y = a->y;
  return launch_rmsnorm(P, a->dtype, false, (cudaStream_t)stream);
}

int nsa_rmsnorm_bwd(const nsa_rmsnorm_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(NSA_ERR_NULL, "args: NULL pointer");
  NormParams P;
  NSA_TRY(fill_norm(P, a->fwd));
  if (!a->dweight) return fail(NSA_ERR_NULL, "dweight: NULL pointer");
  if (a->fwd.rows > 0) {
    if (!a->dy || !a->dx) return fail(NSA_ERR_NULL, "gradient buffer: NULL pointer");
    if ((reinterpret_cast<uintptr_t>(a->dy) & 15u) || (reinterpret_cast<uintptr_t>(a->dx) & 15u))
      return fail(NSA_ERR_ALIGN, "dy and dx must be 16-byte aligned");
  }
  P.dy = a->dy; P.dx = a->dx; P.dweight = a->dweight;
  return launch_rmsnorm(P, a->fwd.dtype, true, (cudaStream_t)stream);
}

}  // extern "C"
