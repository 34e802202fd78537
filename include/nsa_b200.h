/*
 * nsa_b200.h -- C ABI of the B200 (sm_100a) Native Sparse Attention hot path.
 *
 * Every entry point replaces one piece of upstream's Python/Triton hot path;
 * the piece is cited beside each declaration as
 *   NSA:<line>  native_sparse_attention_pytorch/native_sparse_attention.py
 *   TRI:<line>  native_sparse_attention_pytorch/triton_native_sparse_attention.py
 *
 * Conventions
 *   - All pointers are DEVICE pointers owned by the caller.  Nothing here
 *     allocates or frees; work buffers are passed in and sized with
 *     nsa_sel_workspace_bytes() / nsa_cmp_workspace_bytes() / nsa_swa_workspace_bytes().
 *   - Every call is asynchronous on the given CUDA stream (a cudaStream_t
 *     passed as void*, NULL = default stream).
 *   - Return value: 0 on success; a negative NSA_ERR_* for an argument the
 *     library rejects (nothing was launched); a positive value is a CUDA
 *     runtime error code from a launch.  nsa_last_error() returns a static
 *     message for the last non-zero return on the calling thread.
 *   - 4-D activations are described by nsa_tensor: logical shape
 *     [batch, heads, seq, dim_head], last axis contiguous, the other three
 *     strides given in ELEMENTS, so the "b n (h d)" views produced by a fused
 *     qkv projection are consumed without a copy.
 *   - dtype is NSA_F32 or NSA_BF16 and applies to q/k/v/out/do; statistics
 *     (lse), scores, gradients accumulated across queries (dq, dk, dv) and
 *     work buffers are always fp32; block indices are int64 as in upstream.
 *   - Head grouping everywhere: query head = group * G + g (NSA:164, NSA:805).
 */
#ifndef NSA_B200_H
#define NSA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { NSA_F32 = 0, NSA_BF16 = 1 };

enum {
  NSA_OK = 0,
  NSA_ERR_NULL = -1,        /* a required pointer is NULL                     */
  NSA_ERR_SHAPE = -2,       /* sizes inconsistent or outside supported range  */
  NSA_ERR_DTYPE = -3,       /* dtype is neither NSA_F32 nor NSA_BF16          */
  NSA_ERR_ALIGN = -4,       /* pointer or stride breaks the 16-byte rule      */
  NSA_ERR_WORKSPACE = -5,   /* work buffer missing or too small               */
  NSA_ERR_UNSUPPORTED = -6, /* valid request that this build cannot serve     */
  NSA_ERR_DEVICE = -7       /* a kernel reported a bounded wait that ran out  */
};

/* own-block ("diagonal") handling of the selected-block branch */
enum {
  NSA_DIAG_NONE = 0,   /* non-causal: only the selected blocks (NSA:769-770)            */
  NSA_DIAG_CAUSAL = 1, /* causal: keys floor(i/sel)*sel..i of the own block (NSA:754-767) */
  NSA_DIAG_FULL = 2    /* the whole zero-padded own block (non-causal NSA:821-837)       */
};

/* kernel family */
enum {
  NSA_IMPL_AUTO = 0,  /* tensor-core (tcgen05/TMA) kernels where the shape allows, else SIMT */
  NSA_IMPL_SIMT = 1,  /* generic fp32-accumulate CUDA-core kernels                            */
  NSA_IMPL_SM100 = 2  /* tensor-core kernels only; NSA_ERR_UNSUPPORTED if the shape does not fit */
};

typedef struct {
  void* ptr;
  int64_t stride_b, stride_h, stride_n; /* in elements; the dim_head axis has stride 1 */
} nsa_tensor;

/* ------------------------------------------------------------------------
 * Selected-block attention, forward.
 * Replaces native_sparse_attend -> NSA.forward -> native_sparse_attn_forward
 * -> forward_kernel (TRI:1938-1987, 1826-1872, 599-694, 494-597) and the
 * gather formulation NSA:741-819; with nsel == 0 and a diagonal mode it is
 * the no-selection fallback NSA:821-837.
 *
 * Query i of selection head hs (there are sel_heads of them, sel_heads ==
 * kv_heads when the query heads of a KV head share one selection, == q_heads
 * otherwise) attends, for every slot s with mask[b,hs,i,s] != 0, the `block`
 * keys of block idx[b,hs,i,s], plus its own block as `diag` says.  Keys at
 * positions >= seq inside a selected block count as zero keys with zero
 * values (upstream zero-pads K and V).  Slots whose mask is 0 carry the logit
 * -FLT_MAX, so a query with no visible key gets the plain average of the
 * values its slots point at, as upstream's masked_fill + softmax does.
 * ---------------------------------------------------------------------- */
typedef struct {
  nsa_tensor q;          /* [B, q_heads, N, d]  (rotary already applied)      */
  nsa_tensor k, v;       /* [B, kv_heads, N, d]                               */
  nsa_tensor out;        /* [B, q_heads, N, d]  written                       */
  const int64_t* idx;    /* [B, sel_heads, N, nsel] contiguous                */
  const uint8_t* mask;   /* [B, sel_heads, N, nsel] contiguous, 0 / non-zero  */
  float* lse;            /* [B, q_heads, N] natural-log sum-exp, written      */
  int32_t batch, q_heads, kv_heads, sel_heads, seq, dim_head;
  int32_t block;         /* selection_block_size                              */
  int32_t nsel;          /* slots per query, may be 0                         */
  int32_t diag;          /* NSA_DIAG_*                                        */
  int32_t dtype;         /* NSA_F32 / NSA_BF16                                */
  int32_t impl;          /* NSA_IMPL_*                                        */
  float scale;           /* logit scale, upstream uses dim_head^-0.5          */
  void* workspace;       /* nsa_sel_workspace_bytes(args, 0) bytes, may be NULL if that is 0 */
  int64_t workspace_bytes;
  const void* index;     /* optional, forward only: the first nsa_sel_index_bytes(args) bytes of the work buffer of
                            an earlier nsa_sel_fwd call with the same idx, mask and sizes (q_heads / kv_heads
                            included); the call then skips its index pre-pass.  16-byte aligned.  A copy that does
                            not fit the sizes is detected on the device (status 2, nothing computed).  Ignored
                            inside nsa_sel_bwd_args, which has an index field of its own                          */
  int64_t index_bytes;
} nsa_sel_fwd_args;

int nsa_sel_fwd(const nsa_sel_fwd_args* args, void* stream);

/* ------------------------------------------------------------------------
 * Selected-block attention, backward.
 * Replaces NSA.backward -> native_sparse_attn_backward -> backward_preprocess_do_o_dot,
 * backward_kernel (TRI:1874-1925, 1646-1818, 696-756, 1427-1644).
 * dq [B,q_heads,N,d], dk, dv [B,kv_heads,N,d] are contiguous fp32 and are
 * zeroed by the call before accumulation (upstream returns fp32 too,
 * TRI:1900-1902).  slot_grads, if not NULL, receives for every slot the
 * gradient of a multiplier of 1 on that slot's logits (TRI:1061-1080), fp32
 * [B, sel_heads, N, nsel].
 * The tensor-core kernels walk an index of which queries attend which key
 * block, built from idx and mask at the start of each call into the first
 * nsa_sel_index_bytes(args) bytes of the work buffer.  A caller that kept a
 * copy of those bytes from the forward call over the same idx, mask and
 * sizes may pass it as `index` (read only, 16-byte aligned, index_bytes ==
 * nsa_sel_index_bytes): the backward then skips rebuilding it.  NULL = build.
 * ---------------------------------------------------------------------- */
typedef struct {
  nsa_sel_fwd_args fwd;  /* same tensors as the forward call; out and lse are read */
  nsa_tensor dout;       /* [B, q_heads, N, d]                                */
  float* dq;             /* [B, q_heads, N, d]  contiguous fp32, written      */
  float* dk;             /* [B, kv_heads, N, d] contiguous fp32, written      */
  float* dv;             /* [B, kv_heads, N, d] contiguous fp32, written      */
  float* slot_grads;     /* optional                                          */
  const void* index;     /* optional: the forward's index, see above          */
  int64_t index_bytes;
  nsa_tensor dq_out;     /* optional (ptr NULL = unused): dq in the dtype of q with these strides, see nsa_sel_bwd_stores_dq */
  const float* delta;    /* optional [B, q_heads, N] fp32: sum over d of out * dout for every row, for a caller that
                            has it already (the gated combine's backward forms it: gate * d gate); NULL = computed */
} nsa_sel_bwd_args;

int nsa_sel_bwd(const nsa_sel_bwd_args* args, void* stream);

/* Bytes at the start of the forward's work buffer that hold the index the
 * backward can reuse; 0 when the generic kernels serve the problem. */
int64_t nsa_sel_index_bytes(const nsa_sel_fwd_args* args);

/* 1 when the backward of this problem stores every row of dq in one ordered
 * pass (the tensor-core family at dim_head 64) instead of adding into it, 0
 * otherwise, negative = NSA_ERR_*.  Where it is 1 the caller may set
 * `dq_out` (rows of dim_head contiguous elements in the dtype of q, 16-byte
 * aligned, any batch / head / row strides -- for instance the layout of q
 * itself) and pass dq = NULL: dq is then written there, already rounded, and
 * no fp32 dq exists.  With dq_out set on a problem that is not served this
 * way the call returns NSA_ERR_UNSUPPORTED and writes nothing.  The same
 * holds for nsa_cmp_bwd / nsa_swa_bwd with their *_stores_dq functions. */
int nsa_sel_bwd_stores_dq(const nsa_sel_fwd_args* args);

/* Bytes of work buffer the selected-block kernels need for this problem
 * (backward != 0: for nsa_sel_bwd).  0 when the SIMT family serves it.
 * Negative = NSA_ERR_*. */
int64_t nsa_sel_workspace_bytes(const nsa_sel_fwd_args* args, int backward);

/* ------------------------------------------------------------------------
 * Selected-block attention, forward, on the library's built-in scratch area.
 * (No counterpart in upstream: there PyTorch's allocator provides every
 * buffer.)
 *
 * For callers that cannot allocate device memory at the point of the call --
 * a serving loop that must not enter the CUDA allocator, a host application
 * whose memory pool is closed to plug-ins, an embedder that forbids
 * cudaMalloc after start-up.  Same arguments, results and error codes as
 * nsa_sel_fwd with the tensor-core kernels (impl is ignored; `workspace` and
 * `workspace_bytes` are ignored), but the work buffer is a fixed area of
 * nsa_sel_static_scratch_bytes() bytes inside the library image, which every
 * GPU that loads the library keeps reserved until the process exits.
 *   - Only shapes the tensor-core family serves are accepted (bf16, block 64,
 *     dim_head 64 or 128, sel_heads == kv_heads, diag != NSA_DIAG_NONE);
 *     others return NSA_ERR_UNSUPPORTED.
 *   - A problem whose work buffer (nsa_sel_workspace_bytes(args, 0)) exceeds
 *     the area returns NSA_ERR_WORKSPACE; nothing is launched.
 *   - The call itself allocates nothing and frees nothing.  The first call on
 *     a device looks up the area's device address; make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one area and it keeps the previous
 *     call's contents; the call re-initialises what it needs.  Two calls that
 *     overlap on the GPU (different streams, or the same stream before the
 *     first has finished being consumed) race on it: keep them ordered.
 * ---------------------------------------------------------------------- */
int nsa_sel_fwd_static(const nsa_sel_fwd_args* args, void* stream);
int64_t nsa_sel_static_scratch_bytes(void);

/* The device status of the last nsa_sel_fwd_static call on the current
 * device: 0 = its kernels ran to the end, 1 = one of them gave up on a bounded
 * wait (the outputs are invalid), 2 = internal index mismatch.  The word
 * lives at the start of the built-in area; this copies it to `out` -- host
 * memory (pinned, for a copy that does not block the host) or device memory --
 * in the order of `stream`, so issue it on the stream of the forward call
 * and read `out` once that stream has reached it.  Allocates nothing.  (No
 * counterpart in upstream, which checks nothing on the device.) */
int nsa_sel_static_status(int* out, void* stream);

/* ------------------------------------------------------------------------
 * Compressed-KV attention with the importance reduction fused in.
 * Replaces NSA:621-639 + attend NSA:153-184 and the first half of the
 * selection chain NSA:652-680, without materialising the logits tensor.
 *
 * ck, cv hold num_mem memory slots followed by ncb compressed blocks
 * ([B, kv_heads, num_mem + ncb, d]).  Causal: compressed block w is visible
 * to query i iff (w+1)*stride-1 < i; memory slots always are.
 * importance, if not NULL, receives [B, sel_heads, N, ncb] fp32: the logits
 * of the ncb block columns, invisible ones replaced by `sentinel` (upstream's
 * finite (-max)//10 in the tensor dtype, NSA:171), averaged over the
 * q_heads / sel_heads query heads of a selection head (NSA:659-662).  With
 * dtype NSA_BF16 every intermediate is rounded to bf16 where upstream's bf16
 * tensors would be (product, scaled logit, mean).
 * ---------------------------------------------------------------------- */
typedef struct {
  nsa_tensor q;          /* [B, q_heads, N, d]  NOT rotated                   */
  nsa_tensor ck, cv;     /* [B, kv_heads, num_mem + ncb, d]                   */
  nsa_tensor out;        /* [B, q_heads, N, d]  written                       */
  float* lse;            /* [B, q_heads, N]     written                       */
  float* importance;     /* [B, sel_heads, N, ncb] or NULL                    */
  int32_t batch, q_heads, kv_heads, sel_heads, seq, dim_head;
  int32_t num_mem, ncb;
  int32_t stride;        /* compress_block_sliding_stride                     */
  int32_t causal;
  int32_t dtype;
  int32_t impl;
  float scale;
  float sentinel;        /* value an invisible logit is replaced by            */
  void* workspace;       /* nsa_cmp_workspace_bytes(args, 0) bytes, may be NULL if that is 0 */
  int64_t workspace_bytes;
  void* pooled;          /* optional, instead of importance: see nsa_cmp_fwd_pools */
  int32_t pool;          /* block columns per selection block (selection_block_size / stride) */
} nsa_cmp_fwd_args;

int nsa_cmp_fwd(const nsa_cmp_fwd_args* args, void* stream);

/* The second step of the selection chain (NSA:672-680: the mean over the
 * `pool` block columns of every selection block) inside the forward: with
 * `pooled` set (and importance NULL) the call writes [B, sel_heads, N,
 * ncb / pool] bf16 instead of the importance matrix, 1 / (2 * pool) of its
 * bytes: entry (i, c) is the mean of the head-averaged logits of columns
 * c*pool .. c*pool+pool-1, rounded to bf16 as upstream's bf16 tensor would be,
 * for the selection blocks c < i / (pool * stride) that lie wholly before the
 * query's own block.  The other entries are NOT written: under the causal
 * mask those blocks hold a masked column or are the own block, and the
 * selection gives them probability 0 whatever their value, which is what
 * nsa_select assumes when it is handed this tensor (`pooled` there).
 * Returns 1 when nsa_cmp_fwd would serve `pooled` for these arguments (tensor-
 * core family, bf16, causal, 4 / 8 / 16 query heads per KV head, pool a power
 * of two up to 16, num_mem <= 64), else 0: pass importance instead. */
int nsa_cmp_fwd_pools(const nsa_cmp_fwd_args* args);

/* Bytes of work buffer nsa_cmp_fwd (backward != 0: nsa_cmp_bwd) needs; 0 when
 * the SIMT family serves the problem.  The tensor-core family serves bf16,
 * causal, dim_head 64/128, sel_heads == kv_heads, q_heads/kv_heads a power of
 * two up to 16. */
int64_t nsa_cmp_workspace_bytes(const nsa_cmp_fwd_args* args, int backward);

/* Backward of the compressed branch (autograd of NSA:621-639 in upstream).
 * dq [B,q_heads,N,d], dck, dcv [B,kv_heads,num_mem+ncb,d] contiguous fp32,
 * zeroed by the call.  The importance output carries no gradient. */
typedef struct {
  nsa_cmp_fwd_args fwd;
  nsa_tensor dout;
  float* dq;
  float* dck;
  float* dcv;
  nsa_tensor dq_out;     /* optional, as in nsa_sel_bwd_args */
  const void* index;     /* optional, see nsa_cmp_index_bytes */
  int64_t index_bytes;
  const float* delta;    /* optional, as in nsa_sel_bwd_args */
} nsa_cmp_bwd_args;

int nsa_cmp_bwd(const nsa_cmp_bwd_args* args, void* stream);
int nsa_cmp_bwd_stores_dq(const nsa_cmp_fwd_args* args);
/* The tensor-core backward walks an index of which queries attend which block of compressed keys.  Here it depends on
 * the sizes only (batch, heads, seq, num_mem, ncb, stride), not on any tensor: after a backward call the first
 * nsa_cmp_index_bytes(args) bytes of its work buffer hold it, and a caller may keep a copy and pass it as `index`
 * (16-byte aligned, index_bytes as reported) to later calls with the same sizes, which then skip building it.
 * 0 = the generic kernels serve the problem.  A copy that does not fit the sizes is detected on the device: the
 * kernels do nothing and set status 2 in the first word of the work buffer. */
int64_t nsa_cmp_index_bytes(const nsa_cmp_fwd_args* args);

/* ------------------------------------------------------------------------
 * Block selection: per-block mean, own-block exclusion, sink softmax, top-k.
 * Replaces NSA:672-713.
 * importance [rows, N, ncb] fp32 (as written by nsa_cmp_fwd).  For every
 * query: the first cols*cpf columns are averaged in runs of cpf (NSA:672-680,
 * cols = ncb / cpf; cpf == 1 leaves them as they are); if exclude_own, column
 * i / block is overwritten with -max of `dtype` (NSA:686-691); a sink logit
 * of -1000 joins the softmax and is then dropped (NSA:693-695); the k <= cols
 * largest probabilities are written in descending order with their column
 * indices; equal values are ordered by ascending index.  With input_is_prob
 * != 0 (and cpf == 1) the input is ranked as it is, no mean and no softmax.
 * With dtype NSA_BF16 the mean and the probabilities are rounded to bf16 as
 * upstream's bf16 tensors would be.
 * ---------------------------------------------------------------------- */
typedef struct {
  const float* importance;
  int64_t* idx;          /* [rows, N, k] written                              */
  float* vals;           /* [rows, N, k] written                              */
  int32_t rows;          /* B * sel_heads                                     */
  int32_t seq, ncb, cpf, k;
  int32_t block;         /* selection_block_size (for the own-block column)   */
  int32_t exclude_own;
  int32_t input_is_prob;
  int32_t dtype;         /* dtype whose rounding the probabilities follow     */
  const void* pooled;    /* optional, instead of importance: [rows, N, ncb] bf16 as written by nsa_cmp_fwd
                            (`pooled` there; ncb here = its column count, cpf = 1): column c of query i is read
                            only for c < i / block, every other column has probability 0                         */
  int32_t causal_limit;  /* with importance: likewise read only the columns c < i / block of the averaged row   */
} nsa_select_args;

int nsa_select(const nsa_select_args* args, void* stream);

/* ------------------------------------------------------------------------
 * Sliding-window attention.  Replaces the LocalAttention call NSA:841-850.
 * Causal: keys j with 0 <= i-j <= window; otherwise |i-j| <= window.
 * ---------------------------------------------------------------------- */
typedef struct {
  nsa_tensor q;          /* [B, q_heads, N, d]                                */
  nsa_tensor k, v;       /* [B, kv_heads, N, d]  (not repeated over groups)   */
  nsa_tensor out;        /* written                                           */
  float* lse;            /* [B, q_heads, N] written                           */
  int32_t batch, q_heads, kv_heads, seq, dim_head;
  int32_t window, causal, dtype, impl;
  float scale;
  void* workspace;       /* nsa_swa_workspace_bytes(args, 0) bytes, may be NULL if that is 0 */
  int64_t workspace_bytes;
} nsa_swa_fwd_args;

int nsa_swa_fwd(const nsa_swa_fwd_args* args, void* stream);

/* Bytes of work buffer nsa_swa_fwd (backward != 0: nsa_swa_bwd) needs; 0 when
 * the SIMT family serves the problem (tensor-core family: bf16, causal,
 * dim_head 64/128, q_heads/kv_heads a power of two up to 16). */
int64_t nsa_swa_workspace_bytes(const nsa_swa_fwd_args* args, int backward);

typedef struct {
  nsa_swa_fwd_args fwd;
  nsa_tensor dout;
  float* dq;             /* contiguous fp32, zeroed by the call               */
  float* dk;
  float* dv;
  nsa_tensor dq_out;     /* optional, as in nsa_sel_bwd_args */
  const void* index;     /* optional, see nsa_swa_index_bytes */
  int64_t index_bytes;
  const float* delta;    /* optional, as in nsa_sel_bwd_args */
} nsa_swa_bwd_args;

int nsa_swa_bwd(const nsa_swa_bwd_args* args, void* stream);
int nsa_swa_bwd_stores_dq(const nsa_swa_fwd_args* args);
/* As nsa_cmp_index_bytes: the sliding backward's index depends on batch, heads, seq and window only. */
int64_t nsa_swa_index_bytes(const nsa_swa_fwd_args* args);

/* ------------------------------------------------------------------------
 * Gated combine of the three branches and head merge.
 * Replaces NSA:854-860: out[b,n,h*d+c] = sum_s gates[b,h,n,s] * o_s[b,h,n,c],
 * s = compressed, selected, sliding.  gates is a strided [B,q_heads,N,3] view.
 * ---------------------------------------------------------------------- */
typedef struct {
  nsa_tensor o_cmp, o_sel, o_swa; /* [B, q_heads, N, d]                       */
  nsa_tensor gates;               /* [B, q_heads, N, 3]                       */
  void* out;                      /* [B, N, q_heads*d] contiguous, written    */
  int32_t batch, q_heads, seq, dim_head, dtype;
} nsa_combine_fwd_args;

int nsa_combine_fwd(const nsa_combine_fwd_args* args, void* stream);

/* Backward of the combine: d_o_s = gates_s * dout, d_gates_s = sum_c dout * o_s. */
typedef struct {
  nsa_combine_fwd_args fwd;       /* out is unused                            */
  const void* dout;               /* [B, N, q_heads*d] contiguous             */
  void* d_cmp;                    /* [B, q_heads, N, d] contiguous, dtype     */
  void* d_sel;
  void* d_swa;
  float* d_gates;                 /* [B, q_heads, N, 3] contiguous fp32       */
  float* delta;                   /* optional, [3, B, q_heads, N] fp32: gates_s * d_gates_s, which is the row sum
                                     sum_c o_s * d_o_s every branch backward starts from (`delta` there)        */
} nsa_combine_bwd_args;

int nsa_combine_bwd(const nsa_combine_bwd_args* args, void* stream);

/* Gated combine fused with the all-gather of the head-sharded layout.  Replaces the same upstream lines as
 * nsa_combine_fwd (NSA:854-860) for a rank that holds only its own heads: the merged rows of these heads are written
 * at `feature_offset` into every buffer of `outs`, each a [B, N, total_features] tensor -- this GPU's own and the
 * peers' (their device memory mapped into this process, e.g. CUDA IPC or symmetric memory), so no local copy of the
 * merged rows and no separate collective are needed.  Upstream runs on one GPU and has no counterpart of the gather;
 * the partition (KV-head groups per GPU, output all-gathered) is the one this library is specified with.
 * With `multicast` set, outs[0] is instead the multicast address of a buffer that every rank has bound to one NVLink
 * multicast object (symmetric memory): each piece is stored once with multimem.st and the switch writes all ranks'
 * copies, the caller's own included, so a rank sends its heads once instead of once per peer.
 * The caller orders the call against the other ranks (a barrier before the buffers are reused, one after the call
 * before they are read).  Pointers, strides and dim_head must keep 16-byte pieces aligned. */
#define NSA_MAX_GATHER 8
typedef struct {
  nsa_combine_fwd_args fwd;       /* fwd.out is not used                      */
  void* outs[NSA_MAX_GATHER];     /* destinations, own buffer included        */
  int32_t num_outs;               /* 1 .. NSA_MAX_GATHER                      */
  int32_t multicast;              /* 1: outs[0] is a multicast address (num_outs == 1) */
  int64_t total_features;         /* features per position in the destinations */
  int64_t feature_offset;         /* first feature of this rank's heads       */
} nsa_combine_gather_args;

int nsa_combine_fwd_gather(const nsa_combine_gather_args* args, void* stream);

/* The selected-block forward (nsa_sel_fwd, NSA:723-730) with the gated combine, the head merge and the gather
 * (NSA:854-860) in its last kernel: the kernel that merges the partial results of a query's selected blocks also
 * reads the compressed and the sliding row and the gates, and stores the combined row into every destination.  For
 * the branch that runs last this saves the selected output's round trip through memory and the combine's own
 * launch, and the peer stores leave from a kernel that is already streaming.  `sel`: as for nsa_sel_fwd (out may be
 * NULL, it is not written; lse is); `combine`: as for nsa_combine_fwd_gather, fwd.o_sel ignored.  Same bytes as the
 * two calls one after the other.  Tensor-core family only (bf16, block 64, ...): NSA_ERR_UNSUPPORTED otherwise, and
 * the caller makes the two calls.  (No counterpart in upstream, which combines in PyTorch.) */
int nsa_sel_fwd_combine_gather(const nsa_sel_fwd_args* sel, const nsa_combine_gather_args* combine, void* stream);

/* Rotary position embedding of the queries / keys that feed the selected and the sliding branch: replaces the calls
 * into the third-party rotary_embedding_torch package at NSA:643 (rotate_queries_with_cached_keys) and NSA:384-385
 * (rotate_queries_or_keys).  out[b,h,n,2m]   = x[2m] cos[n,m] - x[2m+1] sin[n,m],
 *                        out[b,h,n,2m+1] = x[2m+1] cos[n,m] + x[2m] sin[n,m]   (fp32 arithmetic, no contraction);
 * `inverse` != 0 rotates by the negative angle, which is the backward of the forward rotation.  The tables hold the
 * angles of the positions the caller wants (an offset for cached keys is the caller's choice of table rows). */
typedef struct {
  nsa_tensor x;                   /* [B, H, N, d] view, last axis contiguous, rows 16-byte aligned */
  void* out;                      /* [B, H, N, d], same dtype, written; contiguous unless out_stride_* say otherwise */
  const float* cos_table;         /* [N, d/2] fp32                                                 */
  const float* sin_table;         /* [N, d/2] fp32                                                 */
  int32_t batch, heads, seq, dim_head, dtype, inverse;
  int64_t out_stride_b, out_stride_h, out_stride_n; /* in elements, multiples of 16 bytes; all 0 = contiguous out.
                                                     * The backward can thus write in the layout of the forward's
                                                     * input, e.g. a [B, N, H, d] buffer seen as [B, H, N, d].       */
} nsa_rotary_args;

int nsa_rotary(const nsa_rotary_args* args, void* stream);

/* Input of the compress networks (NSA:589-614): the windows of `block` rows taken every `stride` rows of the un-rotated
 * keys or values -- window w holds rows (w+1)*stride - block .. (w+1)*stride - 1, zero before the sequence start, what
 * upstream gets from pad + unfold (NSA:270-275) -- plus the intra-block position embedding (NSA:600-601):
 *   out[b,h,w,j,:] = x[b,h,(w+1)*stride - block + j,:] + pos[h,j,:].
 * The backward writes dx (zero for rows no window holds) and dpos = sum over batch and windows of dout. */
typedef struct {
  nsa_tensor x;                   /* [B, H, N, d] view, last axis contiguous, rows 16-byte aligned      */
  const void* pos;                /* [H, block, d] contiguous, same dtype                               */
  void* out;                      /* [B, H, ncb, block, d] contiguous, same dtype, written              */
  int32_t batch, heads, seq, dim_head, block, stride, ncb, dtype;
} nsa_windows_fwd_args;

int nsa_windows_fwd(const nsa_windows_fwd_args* args, void* stream);

typedef struct {
  nsa_windows_fwd_args fwd;       /* sizes as in the forward; x, pos and out are not read               */
  const void* dout;               /* [B, H, ncb, block, d] contiguous                                   */
  void* dx;                       /* [B, H, N, d], same dtype, written; contiguous unless dx_stride_* say otherwise */
  float* dpos;                    /* [H, block, d] contiguous fp32, written                             */
  int64_t dx_stride_b, dx_stride_h, dx_stride_n; /* in elements, multiples of 16 bytes; all 0 = contiguous dx   */
} nsa_windows_bwd_args;

int nsa_windows_bwd(const nsa_windows_bwd_args* args, void* stream);

/* RMS normalisation of the layer input, the first step of the layer's forward (NSA:579 and NSA:369 `inp = self.norm(inp)`, an
 * nn.RMSNorm built at NSA:230; the same module normalises the feed-forward input and the final tokens of the
 * language model, transformer.py:134, 210):  y = x * rsqrt(mean(x^2, last axis) + eps) * weight, fp32 arithmetic, one rounding.
 * The forward also writes the reciprocal root per row, which the backward reads:
 *   dx = rstd * (dy*weight - xhat * mean(dy*weight*xhat)),  dweight = sum over rows of dy * xhat,  xhat = x * rstd.
 * dim must be a multiple of 16 bytes and at most 256 sixteen-byte pieces (2048 bf16 / 1024 fp32 elements). */
typedef struct {
  const void* x;                  /* [rows, dim], rows x_stride elements apart, 16-byte aligned rows     */
  const void* weight;             /* [dim] in the dtype of x, or fp32 when weight_f32 != 0              */
  void* y;                        /* [rows, dim] contiguous, dtype of x, written                          */
  float* rstd;                    /* [rows] fp32, written                                                 */
  int64_t rows, x_stride;
  int32_t dim, dtype, weight_f32, reserved;
  float eps, reserved2;
} nsa_rmsnorm_fwd_args;

int nsa_rmsnorm_fwd(const nsa_rmsnorm_fwd_args* args, void* stream);

typedef struct {
  nsa_rmsnorm_fwd_args fwd;       /* x, weight, rstd and the sizes as in the forward; y is not read        */
  const void* dy;                 /* [rows, dim] contiguous, dtype of x                                   */
  void* dx;                       /* [rows, dim] contiguous, dtype of x, written                          */
  float* dweight;                 /* [dim] fp32, written                                                  */
} nsa_rmsnorm_bwd_args;

int nsa_rmsnorm_bwd(const nsa_rmsnorm_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------
 * One decoding step of the hot path in a single launch.  Replaces the
 * attention part of upstream's forward_inference (NSA:387-547): for the
 * newest token at position T-1,
 *   - compressed attention over the ncb blocks compressed so far, with the
 *     num_mem memory slots in front (none of it when ncb == 0, as upstream),
 *     un-rotated queries;
 *   - block selection from the compressed logits: mean over the heads of a KV
 *     head and over the block/stride compressed blocks of a selection block,
 *     softmax with the -1000 sink, top-nsel, slots with probability <= 1e-10
 *     dropped (no own-block exclusion: upstream's decode path has none);
 *   - attention of the rotated queries over the selected blocks plus keys
 *     (T-1)/block*block .. T-1 of the own block;
 *   - sliding window over keys max(0, T-1-window) .. T-1;
 *   - out[b, (h d)] = sum_s gates[b,h,s] * branch_s.
 * One selection per KV head (query_heads_share_selected_kv).  q, qr, gates,
 * mem_k, mem_v and out are contiguous; keys, vals, ck, cv take strides in
 * elements (rows 16-byte aligned).  fp32 arithmetic; dtype as elsewhere.
 * Limits: q_heads / kv_heads <= 16, dim_head <= 128, nsel <= 32, and
 * ncb + ncb / (block / stride) block logits must fit one CTA's shared memory
 * (NSA_ERR_UNSUPPORTED beyond, about 20000 compressed blocks).
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;          /* [B, q_heads, d] un-rotated queries of the token  */
  const void* qr;         /* [B, q_heads, d] rotated queries                   */
  nsa_tensor keys;        /* [B, kv_heads, T, d] rotated keys, token included  */
  nsa_tensor vals;        /* [B, kv_heads, T, d]                               */
  nsa_tensor ck;          /* [B, kv_heads, ncb, d] (ptr may be NULL if ncb==0) */
  nsa_tensor cv;
  const void* mem_k;      /* [kv_heads, num_mem, d]                            */
  const void* mem_v;
  const void* gates;      /* [B, q_heads, 3]: compressed, selected, sliding    */
  void* out;              /* [B, q_heads * d]                                  */
  int32_t batch, q_heads, kv_heads, dim_head;
  int32_t cache_len;      /* T                                                 */
  int32_t ncb, num_mem, stride, block, nsel, window;
  int32_t dtype;
  float scale;
  int32_t reserved;
} nsa_decode_args;

int nsa_decode_step(const nsa_decode_args* args, void* stream);

/* ------------------------------------------------------------------------
 * Housekeeping (no counterparts in upstream).
 * ---------------------------------------------------------------------- */

/* Kernels this library has launched in this process so far, all entry points
 * and threads together.  A benchmark reads it before and after its timed
 * region. */
int64_t nsa_launch_count(void);

/* Self-test of the bounded waits every tensor-core kernel uses: launches one
 * block that allocates tensor memory and waits, for at most `limit_cycles` SM
 * clock cycles, on a barrier nobody arrives on; it must give up, free its
 * tensor memory and leave 1 in *status_device (device memory, cleared first),
 * the way a kernel that lost a hand-over would.  Returns at once; nothing
 * traps or spins without a bound. */
int nsa_selftest_bounded_wait(int* status_device, int64_t limit_cycles, void* stream);

/* Library information.  nsa_struct_size(i) is sizeof() of the i-th argument
 * struct in declaration order (0 nsa_tensor, 1 sel_fwd, 2 sel_bwd, 3 cmp_fwd,
 * 4 cmp_bwd, 5 select, 6 swa_fwd, 7 swa_bwd, 8 combine_fwd, 9 combine_bwd, 10 combine_gather,
 * 11 rotary, 12 windows_fwd, 13 windows_bwd, 14 rmsnorm_fwd, 15 rmsnorm_bwd, 16 decode), so
 * a foreign-function binding can verify its own layout; -1 for other i. */
const char* nsa_last_error(void);
int nsa_abi_version(void);
int nsa_struct_size(int which);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H */
