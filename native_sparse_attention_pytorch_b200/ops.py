"""PyTorch operators over the C-ABI kernels: one autograd Function per NSA
branch plus the block selection and the gated combine.  Tensors stay owned by
PyTorch's allocator; the library only sees device pointers, sizes and the
current CUDA stream."""
import ctypes as C
import threading

import torch
from torch.autograd import Function

from . import _lib as L


def _empty_like_rows(t):
    """Contiguous [B,H,N,d] buffer of t's dtype."""
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)


# --------------------------------------------------------------------------
# selected-block attention (replaces upstream's Triton NSA Function, TRI:1824-1927)
# --------------------------------------------------------------------------

def _sel_args(q, k, v, out, idx, mask, lse, block, diag, impl, scale):
    b, hq, n, d = q.shape
    hkv = k.shape[1]
    nsel = 0 if idx is None else idx.shape[-1]
    hs = hkv if idx is None else idx.shape[1]
    return L.SelFwdArgs(q=L.t4(q), k=L.t4(k), v=L.t4(v), out=L.t4(out), idx=L.ptr(idx), mask=L.ptr(mask),
                        lse=L.ptr(lse), batch=b, q_heads=hq, kv_heads=hkv, sel_heads=hs, seq=n, dim_head=d,
                        block=block, nsel=nsel, diag=diag, dtype=L.dtype_code(q), impl=impl, scale=scale,
                        workspace=None, workspace_bytes=0)


# Device status of the tensor-core kernels.  Every such kernel reports through the first word of its work buffer:
# 0 = fine, 1 = a bounded wait ran out (results invalid), 2 = it was handed an index built for another problem.  The
# words are folded, in stream order, into one int32 per device (bitwise or), so nothing is lost however many kernels
# run between two checks.  The autograd engine calls the backward functions from its own thread: one lock guards the
# tables below.
_state_lock = threading.Lock()
_status_acc = {}      # device index -> int32[1] device tensor
_status_polls = {}    # device index -> (pinned int32[1], event) of the copy issued by the last poll


def _with_workspace(args, backward, device, sizer='nsa_sel_workspace_bytes'):
    lib = L.load()
    need = getattr(lib, sizer)(C.byref(args), int(backward))
    if need < 0:
        L.check(int(need))
    ws = None
    if need > 0:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
    return ws


def _keep_status(ws):
    """Fold the status word of a work buffer into the device's accumulator (one tiny stream-ordered kernel)."""
    if ws is None:
        return
    key = ws.device.index
    with _state_lock:
        acc = _status_acc.get(key)
        if acc is None:
            acc = _status_acc[key] = torch.zeros(1, dtype=torch.int32, device=ws.device)
    acc.bitwise_or_(ws[:4].view(torch.int32))


def _raise_for(code):
    if code & 2:
        raise L.NsaError('a tensor-core kernel was given an index that was not built for its problem; '
                         'its results are invalid')
    if code != 0:
        raise L.NsaError('a tensor-core kernel gave up on a bounded wait; its results are invalid')


def check_device_status():
    """Synchronise and raise if any tensor-core kernel launched since the last check gave up on a wait (status 1) or
    was handed an index that was not built for its problem (status 2)."""
    with _state_lock:
        accs = list(_status_acc.values())
        _status_polls.clear()
    code = 0
    for acc in accs:
        code |= int(acc.item())
        acc.zero_()
    _raise_for(code)


def poll_device_status(device):
    """The same check without a synchronisation, one call late: looks at the status copy the previous poll started
    (if it has landed) and starts the next one.  `SparseAttention.forward` calls this, so a training loop learns of
    an invalid step at its next forward without any host wait on the hot path."""
    if torch.cuda.is_current_stream_capturing():
        return                          # a CUDA graph is being recorded: nothing here may touch the host
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    with _state_lock:
        acc = _status_acc.get(key)
        pending = _status_polls.get(key)
    if acc is None:
        return
    if pending is not None:
        host, event = pending
        if not event.query():
            return                      # the previous copy is still in flight: look again at the next call
        code = int(host.item())
        if code != 0:
            acc.zero_()
            with _state_lock:
                _status_polls.pop(key, None)
            _raise_for(code)
    host = pending[0] if pending is not None else torch.zeros(1, dtype=torch.int32).pin_memory()
    host.copy_(acc, non_blocking=True)
    event = torch.cuda.Event()
    event.record(torch.cuda.current_stream(acc.device))
    with _state_lock:
        _status_polls[key] = (host, event)


def dim_order(t):
    """The dimensions of t from outermost to innermost in memory (the last one stays last)."""
    return tuple(sorted(range(t.dim() - 1), key=lambda i: (-t.stride(i), i))) + (t.dim() - 1,)


def empty_in_order(shape, order, dtype, device):
    """Uninitialised dense tensor of `shape` whose dimensions lie in memory in `order`."""
    buf = torch.empty([shape[i] for i in order], dtype=dtype, device=device)
    return buf.permute([order.index(i) for i in range(len(shape))])


def _empty_in_order_of(t):
    """Uninitialised tensor of t's shape and dtype whose dimensions lie in memory in the order t's do: a [b, h, n, d]
    view of a [b, n, (h d)] projection output gives a [b, n, h, d] buffer seen as [b, h, n, d], so that the gradient
    of the view that made t is a view again instead of a copy."""
    return empty_in_order(t.shape, dim_order(t), t.dtype, t.device)


def _dq_buffers(lib, query, fwd, q, need_fp32=False):
    """(fp32 dq, None), or (None, dq in q's dtype and layout) where the backward stores whole rows of dq itself."""
    if not need_fp32 and q.dtype == torch.bfloat16 and getattr(lib, query)(C.byref(fwd)) == 1:
        return None, _empty_in_order_of(q)
    return torch.empty(q.shape, dtype=torch.float32, device=q.device), None


def _handed_over_delta(dout, shape):
    """The row sums sum_d out * dout that the gated combine's backward attached to the branch gradient it returned
    (delta = gate * d gate, see GatedCombine.backward), when `dout` is that very tensor; else None and the backward
    computes them itself."""
    delta = getattr(dout, '_nsa_delta', None)
    if delta is None or tuple(delta.shape) != tuple(shape) or delta.dtype != torch.float32 or not delta.is_contiguous() \
            or delta.device != dout.device:
        return None
    return delta


def _call_bwd(fn, make_args, q, stream):
    """Run a backward entry point; when the tensor-core kernels decline the tensors at run time although the direct
    dq was offered, run it again with an fp32 dq."""
    args, dq, dq_out = make_args(True)
    rc = fn(C.byref(args), stream)
    if rc == L.NSA_ERR_UNSUPPORTED and dq_out is not None:
        args, dq, dq_out = make_args(False)
        rc = fn(C.byref(args), stream)
    L.check(rc)
    return dq_out if dq_out is not None else dq.to(q.dtype)


# The index the sliding and the compressed backward walk depends on the sizes only: built once per shape and device
# (by the first backward call, inside its work buffer), then handed to later calls.  A few MB per entry.
_shape_index = {}
_SHAPE_INDEX_ENTRIES = 8


def _cached_index(key):
    if not REUSE_INDEX:
        return None
    with _state_lock:
        return _shape_index.get(key)


def _keep_index(key, ws, nbytes):
    if not (REUSE_INDEX and ws is not None and nbytes > 0):
        return
    with _state_lock:
        if key in _shape_index:
            return
        while len(_shape_index) >= _SHAPE_INDEX_ENTRIES:
            _shape_index.pop(next(iter(_shape_index)))
        _shape_index[key] = ws[:nbytes].clone()


REUSE_INDEX = True     # the selected-block backward takes the index the forward built instead of rebuilding it
HAND_OVER_DELTA = True # the gated combine's backward hands the row sums out * d out to the three branch backwards


class SelectedAttention(Function):
    """out, lse = f(q, k, v, idx, mask, slot_scale, block, diag, impl, index_cache)."""

    @staticmethod
    def forward(ctx, q, k, v, idx, mask, slot_scale, block, diag, impl, index_cache=None):
        L.require_cuda(q, k, v, idx, mask)
        lib = L.load()
        q, k, v = L.rowwise(q), L.rowwise(k), L.rowwise(v)
        if idx is not None:
            idx = idx.to(torch.int64).contiguous()
            mask = mask.to(torch.bool).contiguous().view(torch.uint8)
        b, hq, n, d = q.shape
        out = _empty_like_rows(q)
        lse = torch.empty(b, hq, n, dtype=torch.float32, device=q.device)
        scale = d ** -0.5
        with torch.cuda.device(q.device):
            args = _sel_args(q, k, v, out, idx, mask, lse, block, diag, impl, scale)
            ws = _with_workspace(args, False, q.device)
            # `index_cache`: a dict the caller owns while it calls several times with the SAME idx and mask (runs of
            # query heads of one KV head); the first call of a shape leaves its index there, the later ones take it
            cache_key = (tuple(q.shape), tuple(k.shape), None if idx is None else tuple(idx.shape), block, diag, impl)
            shared = index_cache.get(cache_key) if index_cache is not None else None
            if shared is not None:
                args.index, args.index_bytes = shared.data_ptr(), shared.numel()
            L.check(lib.nsa_sel_fwd(C.byref(args), L.stream_of(q)))
            # the index of which queries attend which key block: a few MB the backward need not rebuild
            keep = ws is not None and ((REUSE_INDEX and any(ctx.needs_input_grad[:3])) or
                                       (index_cache is not None and shared is None))
            index_bytes = int(lib.nsa_sel_index_bytes(C.byref(args))) if keep else 0
        ctx.index = shared if shared is not None else (ws[:index_bytes].clone() if index_bytes > 0 else None)
        if index_cache is not None and shared is None and ctx.index is not None:
            index_cache[cache_key] = ctx.index
        _keep_status(ws)
        del ws
        ctx.save_for_backward(q, k, v, idx, mask, out, lse)
        ctx.cfg = (block, diag, impl, scale, None if slot_scale is None else slot_scale.dtype)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, idx, mask, out, lse = ctx.saved_tensors
        block, diag, impl, scale, slot_dtype = ctx.cfg
        want_slot_grads = slot_dtype is not None
        lib = L.load()
        delta = _handed_over_delta(dout, lse.shape)
        dout = L.rowwise(dout)
        dk = torch.empty(k.shape, dtype=torch.float32, device=q.device)
        dv = torch.empty(v.shape, dtype=torch.float32, device=q.device)
        slot = torch.zeros(idx.shape, dtype=torch.float32, device=q.device) if want_slot_grads else None
        with torch.cuda.device(q.device):
            fwd = _sel_args(q, k, v, out, idx, mask, lse, block, diag, impl, scale)
            ws = _with_workspace(fwd, True, q.device)
            index = ctx.index

            def make_args(direct):
                dq, dq_out = _dq_buffers(lib, 'nsa_sel_bwd_stores_dq', fwd, q, need_fp32=not direct)
                return L.SelBwdArgs(fwd=fwd, dout=L.t4(dout), dq=L.ptr(dq), dk=L.ptr(dk), dv=L.ptr(dv),
                                    slot_grads=L.ptr(slot), index=L.ptr(index),
                                    index_bytes=0 if index is None else index.numel(),
                                    dq_out=L.t4(dq_out) if dq_out is not None else L.Tensor4(),
                                    delta=L.ptr(delta)), dq, dq_out
            dq = _call_bwd(lib.nsa_sel_bwd, make_args, q, L.stream_of(q))
        _keep_status(ws)
        del ws
        return (dq, dk.to(k.dtype), dv.to(v.dtype), None, None,
                None if slot is None else slot.to(slot_dtype), None, None, None, None)


def native_sparse_attend(fq, fk, fv, block_size, selected_block_indices, fmask, sel_scale=None,
                         include_block_causal=True, return_lse=False, block_dk_dv_use_dot=False,
                         return_sliding_window_out=False, impl='auto', index_cache=None):
    """Drop-in for upstream's ``native_sparse_attend`` (TRI:1938-1987): selected-
    block attention with GQA head grouping.  fq [b,qh,n,d]; fk, fv [b,kh,n,d];
    indices / mask / sel_scale [b,kh,n,sel] or [b,qh,n,sel].  ``sel_scale`` must
    be all ones (TRI:1860-1861) and only adds a gradient output for it.
    ``block_dk_dv_use_dot`` is accepted and ignored (a Triton tuning switch).
    ``return_sliding_window_out`` adds upstream's second output (TRI:199-201, 273-277,
    1975-1987): causal attention over the last ``block_size`` keys and the query's own
    position, here one more call of the sliding-window kernels; out and lse then
    are pairs, as upstream's.  Unlike upstream there is no block_size >= 16
    or fp16 restriction, and float32 inputs are computed in float32.  ``index_cache``:
    a dict a caller passes to several calls that share ``selected_block_indices`` and
    ``fmask`` (and the shapes); the first call leaves its index of which queries attend
    which key block there and the later ones skip building it."""
    if return_sliding_window_out and not include_block_causal:
        raise ValueError('return_sliding_window_out needs include_block_causal: upstream computes the sliding output '
                         'in the pass over the causal own block')
    q_heads, kv_heads, sel_heads = fq.shape[1], fk.shape[1], selected_block_indices.shape[1]
    assert q_heads % kv_heads == 0
    assert sel_heads in (q_heads, kv_heads)
    diag = L.DIAG_CAUSAL if include_block_causal else L.DIAG_NONE
    out, lse = SelectedAttention.apply(fq, fk, fv, selected_block_indices, fmask, sel_scale, block_size, diag,
                                       L.IMPL_BY_NAME[impl], index_cache)
    if return_sliding_window_out:
        sliding_out, sliding_lse = SlidingAttention.apply(fq, fk, fv, block_size, True, L.IMPL_BY_NAME[impl])
        out, lse = (out, sliding_out), (lse, sliding_lse)
    return (out, lse) if return_lse else out


def block_diagonal_attend(fq, fk, fv, block_size, causal, impl='auto'):
    """The no-selection fallback (NSA:821-837): every query attends its own block only."""
    diag = L.DIAG_CAUSAL if causal else L.DIAG_FULL
    out, _ = SelectedAttention.apply(fq, fk, fv, None, None, None, block_size, diag, L.IMPL_BY_NAME[impl])
    return out


# --------------------------------------------------------------------------
# compressed attention + importance (replaces NSA:621-639, 652-662)
# --------------------------------------------------------------------------

def mask_sentinel(dtype):
    """The finite value upstream writes over invisible logits: (-finfo.max)//10 stored in `dtype` (NSA:168-171)."""
    return torch.tensor(-torch.finfo(dtype).max // 10, dtype=dtype).float().item()


def _cmp_args(q, ck, cv, out, lse, imp, sel_heads, num_mem, stride, causal, impl, scale, pooled=None, pool=0):
    b, hq, n, d = q.shape
    return L.CmpFwdArgs(pooled=L.ptr(pooled), pool=pool, q=L.t4(q), ck=L.t4(ck), cv=L.t4(cv), out=L.t4(out), lse=L.ptr(lse), importance=L.ptr(imp),
                        batch=b, q_heads=hq, kv_heads=ck.shape[1], sel_heads=sel_heads, seq=n, dim_head=d,
                        num_mem=num_mem, ncb=ck.shape[2] - num_mem, stride=stride, causal=int(causal),
                        dtype=L.dtype_code(q), impl=impl, scale=scale, sentinel=mask_sentinel(q.dtype), workspace=None,
                        workspace_bytes=0)


class CompressedAttention(Function):
    """out, importance = f(q, ck, cv, num_mem, stride, causal, sel_heads, want_importance, impl, pool);
    ck, cv carry the memory slots in front.  importance is [B, sel_heads, N, ncb] fp32, no gradient; with pool > 0,
    where the library can (nsa_cmp_fwd_pools), it is instead the bf16 tensor [B, sel_heads, N, ncb // pool] of
    per-selection-block means that `select_blocks` recognises by its dtype."""

    @staticmethod
    def forward(ctx, q, ck, cv, num_mem, stride, causal, sel_heads, want_importance, impl, pool=0):
        L.require_cuda(q, ck, cv)
        lib = L.load()
        q, ck, cv = L.rowwise(q), L.rowwise(ck), L.rowwise(cv)
        b, hq, n, d = q.shape
        ncb = ck.shape[2] - num_mem
        out = _empty_like_rows(q)
        lse = torch.empty(b, hq, n, dtype=torch.float32, device=q.device)
        scale = d ** -0.5
        pooled = None
        if want_importance and pool > 0:
            probe = _cmp_args(q, ck, cv, out, lse, None, sel_heads, num_mem, stride, causal, impl, scale, None, pool)
            if lib.nsa_cmp_fwd_pools(C.byref(probe)):
                # entries at and past a query's own block are never written nor read
                pooled = torch.empty(b, sel_heads, n, ncb // pool, dtype=torch.bfloat16, device=q.device)
        imp = torch.empty(b, sel_heads, n, ncb, dtype=torch.float32, device=q.device) \
            if want_importance and pooled is None else None
        with torch.cuda.device(q.device):
            args = _cmp_args(q, ck, cv, out, lse, imp, sel_heads, num_mem, stride, causal, impl, scale, pooled,
                             pool if pooled is not None else 0)
            ws = _with_workspace(args, False, q.device, 'nsa_cmp_workspace_bytes')
            L.check(lib.nsa_cmp_fwd(C.byref(args), L.stream_of(q)))
            _keep_status(ws)
            del ws
        ctx.save_for_backward(q, ck, cv, out, lse)
        ctx.cfg = (num_mem, stride, causal, sel_heads, impl, scale)
        ctx.set_materialize_grads(False)   # no gradient through the importance unless the top-k is differentiable
        if pooled is not None:
            imp = pooled
            ctx.mark_non_differentiable(imp)
        elif imp is None:
            imp = torch.empty(0, device=q.device)
            ctx.mark_non_differentiable(imp)
        return out, imp

    @staticmethod
    def backward(ctx, dout, dimp):
        q, ck, cv, out, lse = ctx.saved_tensors
        num_mem, stride, causal, sel_heads, impl, scale = ctx.cfg
        lib = L.load()
        delta = None if dout is None else _handed_over_delta(dout, lse.shape)
        dout = torch.zeros_like(out) if dout is None else L.rowwise(dout)
        dck = torch.empty(ck.shape, dtype=torch.float32, device=q.device)
        dcv = torch.empty(cv.shape, dtype=torch.float32, device=q.device)
        # a gradient through the importance output (differentiable top-k) is added to the fp32 dq afterwards
        with_dimp = dimp is not None and dimp.numel() > 0 and ctx.needs_input_grad[0]
        with torch.cuda.device(q.device):
            fwd = _cmp_args(q, ck, cv, out, lse, None, sel_heads, num_mem, stride, causal, impl, scale)
            ws = _with_workspace(fwd, True, q.device, 'nsa_cmp_workspace_bytes')
            key = ('cmp', q.device.index, tuple(q.shape), tuple(ck.shape), num_mem, stride, bool(causal), impl)
            index = _cached_index(key)

            def make_args(direct):
                dq, dq_out = _dq_buffers(lib, 'nsa_cmp_bwd_stores_dq', fwd, q, need_fp32=with_dimp or not direct)
                return L.CmpBwdArgs(fwd=fwd, dout=L.t4(dout), dq=L.ptr(dq), dck=L.ptr(dck), dcv=L.ptr(dcv),
                                    dq_out=L.t4(dq_out) if dq_out is not None else L.Tensor4(), index=L.ptr(index),
                                    index_bytes=0 if index is None else index.numel(), delta=L.ptr(delta)), dq, dq_out
            if with_dimp:
                args, dq32, _ = make_args(False)
                L.check(lib.nsa_cmp_bwd(C.byref(args), L.stream_of(q)))
                _importance_backward(dimp, q, ck, dq32, dck, num_mem, stride, causal, sel_heads, scale)
                dq = dq32.to(q.dtype)
            else:
                dq = _call_bwd(lib.nsa_cmp_bwd, make_args, q, L.stream_of(q))
            if index is None:
                _keep_index(key, ws, int(lib.nsa_cmp_index_bytes(C.byref(fwd))))
            _keep_status(ws)
            del ws
        return dq, dck.to(ck.dtype), dcv.to(cv.dtype), None, None, None, None, None, None, None


def _importance_backward(dimp, q, ck, dq, dck, num_mem, stride, causal, sel_heads, scale):
    """Adds the gradient that arrives through the importance output (differentiable top-k, upstream NSA:715) to dq and
    dck.  importance[b,s,i,c] is the mean over the heads of selection head s of the visible logit
    scale * q[b,h,i] . ck[b,kv(h),num_mem+c]; rounding steps pass the gradient through.  Two plain batched GEMMs per
    KV head (library GEMMs: this path is off unless use_diff_topk is set)."""
    b, hq, n, d = q.shape
    hkv = ck.shape[1]
    ncb = ck.shape[2] - num_mem
    g_sel = hq // sel_heads                      # query heads averaged into one importance row
    dlog = dimp.float() * (scale / g_sel)        # d logit of every head of the selection head, [B, Hs, N, ncb]
    if causal:
        visible = torch.arange(ncb, device=q.device)[None, :] < (torch.arange(n, device=q.device) // stride)[:, None]
        dlog = dlog * visible
    per_kv = hq // hkv
    ckc = ck[:, :, num_mem:].float()             # [B, Hkv, ncb, d]
    # every query head h gets dlog of its selection head times the compressed keys of its KV head
    dlog_h = dlog.repeat_interleave(g_sel, dim=1) if g_sel > 1 else dlog        # [B, Hq, N, ncb]
    ck_h = ckc.repeat_interleave(per_kv, dim=1) if per_kv > 1 else ckc          # [B, Hq, ncb, d]
    dq += torch.matmul(dlog_h, ck_h)
    dck_part = torch.matmul(dlog_h.transpose(-1, -2), q.float())                # [B, Hq, ncb, d]
    dck[:, :, num_mem:] += dck_part.view(b, hkv, per_kv, ncb, d).sum(dim=2)


def compressed_attend(q, ck, cv, num_mem, stride, causal, sel_heads=None, want_importance=True, impl='auto', pool=0):
    """Compressed attention and, with `want_importance`, the head-averaged logits [B, sel_heads, N, ncb] in fp32.
    `pool` = block columns per selection block (selection_block_size // stride) lets the kernel do the per-block mean
    of the selection chain as well, where it can: the second result is then a bf16 tensor [B, sel_heads, N,
    ncb // pool] (defined before each query's own block only, no gradient) for `select_blocks`; callers that need the
    full matrix or its gradient leave pool at 0."""
    sel_heads = ck.shape[1] if sel_heads is None else sel_heads
    out, imp = CompressedAttention.apply(q, ck, cv, num_mem, stride, causal, sel_heads, want_importance,
                                         L.IMPL_BY_NAME[impl], pool)
    return (out, imp) if want_importance else out


# --------------------------------------------------------------------------
# block selection (replaces NSA:672-713); integer output, no gradient
# --------------------------------------------------------------------------

class _SelectValuesGrad(Function):
    """Identity on the selected values that carries their gradient back to the importance matrix (the differentiable
    top-k of upstream NSA:715: the picked probabilities are a gather out of a softmax).  The forward values and
    indices come from the selection kernel; the backward recomputes the softmax in PyTorch."""

    @staticmethod
    def forward(ctx, importance, vals, idx, block, stride):
        ctx.save_for_backward(importance, idx)
        ctx.cfg = (block, stride)
        return vals.clone()

    @staticmethod
    def backward(ctx, dvals):
        importance, idx = ctx.saved_tensors
        block, stride = ctx.cfg
        b, hs, n, ncb = importance.shape
        cpf = block // stride
        cols = ncb // cpf
        x = importance.float()
        own = None
        if cpf > 1:
            x = x[..., : cols * cpf].reshape(b, hs, n, cols, cpf).mean(dim=-1)
            own = (torch.arange(n, device=x.device) // block)[:, None] == torch.arange(cols, device=x.device)[None, :]
            x = x.masked_fill(own, -torch.finfo(torch.float32).max)
        p = torch.nn.functional.pad(x, (1, 0), value=-1e3).softmax(dim=-1)[..., 1:]
        dp = torch.zeros_like(p).scatter_add_(-1, idx, dvals.float())
        dx = p * (dp - (p * dp).sum(dim=-1, keepdim=True))        # the sink has no incoming gradient
        if cpf > 1:
            dx = dx.masked_fill(own, 0.)
            dimp = torch.zeros_like(importance, dtype=torch.float32)
            dimp[..., : cols * cpf] = (dx / cpf).repeat_interleave(cpf, dim=-1)
        else:
            dimp = dx
        return dimp.to(importance.dtype), None, None, None, None


def select_blocks(importance, block, stride, nsel, dtype=torch.float32, input_is_prob=False):
    """As `_select_blocks`; when `importance` requires grad, the returned values carry it (differentiable top-k).
    A bf16 `importance` is the pooled tensor of `compressed_attend(..., pool=block // stride)`."""
    vals, idx = _select_blocks(importance.detach(), block, stride, nsel, dtype, input_is_prob)
    if torch.is_grad_enabled() and importance.requires_grad and not input_is_prob and vals.numel() > 0:
        vals = _SelectValuesGrad.apply(importance, vals, idx, block, stride)
    return vals, idx


@torch.no_grad()
def _select_blocks(importance, block, stride, nsel, dtype=torch.float32, input_is_prob=False):
    """importance [B, Hs, N, ncb] fp32 -> (values [B,Hs,N,k] in `dtype`, int64 indices [B,Hs,N,k]),
    k = min(nsel, ncb // (block // stride)).  See nsa_select in include/nsa_b200.h."""
    L.require_cuda(importance)
    lib = L.load()
    pooled = importance.dtype == torch.bfloat16 and not input_is_prob
    importance = importance.contiguous() if pooled else importance.contiguous().float()
    b, hs, n, ncb = importance.shape
    cpf = 1 if input_is_prob or pooled else block // stride
    cols = ncb // cpf
    k = min(nsel, cols)
    idx = torch.empty(b, hs, n, k, dtype=torch.int64, device=importance.device)
    vals = torch.empty(b, hs, n, k, dtype=torch.float32, device=importance.device)
    if k > 0 and idx.numel() > 0:
        code = L.NSA_BF16 if dtype == torch.bfloat16 else L.NSA_F32
        args = L.SelectArgs(importance=None if pooled else L.ptr(importance), idx=L.ptr(idx), vals=L.ptr(vals),
                            rows=b * hs, seq=n, ncb=ncb, cpf=cpf, k=k, block=block,
                            exclude_own=int(block != stride and not input_is_prob),
                            input_is_prob=int(input_is_prob), dtype=code,
                            pooled=L.ptr(importance) if pooled else None, causal_limit=int(pooled))
        with torch.cuda.device(importance.device):
            L.check(lib.nsa_select(C.byref(args), L.stream_of(importance)))
    return vals.to(dtype), idx


@torch.no_grad()
def selected_attend_combine_gather(fq, fk, fv, block_size, idx, fmask, o_cmp, o_swa, gates, out_ptrs, total_features,
                                   feature_offset, include_block_causal=True, multicast=False, impl='auto',
                                   index_cache=None):
    """Forward only: the selected branch for `fq`'s heads with the gated combine, the head merge and the stores into
    every [B, N, total_features] buffer of `out_ptrs` done by its last kernel (nsa_sel_fwd_combine_gather) -- what
    `native_sparse_attend` followed by `gated_combine_gather` gives, byte for byte, without the selected output's
    round trip.  Returns False, having done nothing, where the tensor-core family does not serve the shapes: the
    caller then makes the two calls."""
    L.require_cuda(fq, fk, fv, idx, fmask, o_cmp, o_swa, gates)
    lib = L.load()
    if fq.dtype != torch.bfloat16 or impl == 'simt' or idx.shape[1] != fk.shape[1]:
        return False
    q, k, v = L.rowwise(fq), L.rowwise(fk), L.rowwise(fv)
    idx = idx.to(torch.int64).contiguous()
    mask = fmask.to(torch.bool).contiguous().view(torch.uint8)
    o_cmp, o_swa = (t if _vec_ok(t) else t.contiguous() for t in (o_cmp, o_swa))
    if gates.stride(-1) != 1:
        gates = gates.contiguous()
    b, hq, n, d = q.shape
    lse = torch.empty(b, hq, n, dtype=torch.float32, device=q.device)
    diag = L.DIAG_CAUSAL if include_block_causal else L.DIAG_NONE
    with torch.cuda.device(q.device):
        args = _sel_args(q, k, v, q, idx, mask, lse, block_size, diag, L.IMPL_BY_NAME[impl], d ** -0.5)
        args.out = L.Tensor4()
        need = lib.nsa_sel_workspace_bytes(C.byref(args), 0)
        if need <= 0:
            return False
        ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
        cache_key = (tuple(q.shape), tuple(k.shape), tuple(idx.shape), block_size, diag, L.IMPL_BY_NAME[impl])
        shared = index_cache.get(cache_key) if index_cache is not None else None
        if shared is not None:
            args.index, args.index_bytes = shared.data_ptr(), shared.numel()
        fwd = L.CombineFwdArgs(o_cmp=L.t4(o_cmp), o_sel=L.Tensor4(), o_swa=L.t4(o_swa), gates=L.t4(gates), out=None,
                               batch=b, q_heads=hq, seq=n, dim_head=d, dtype=L.dtype_code(q))
        outs = (C.c_void_p * L.MAX_GATHER)(*[int(p) for p in out_ptrs])
        cargs = L.CombineGatherArgs(fwd=fwd, outs=outs, num_outs=len(out_ptrs), multicast=int(bool(multicast)),
                                    total_features=total_features, feature_offset=feature_offset)
        rc = lib.nsa_sel_fwd_combine_gather(C.byref(args), C.byref(cargs), L.stream_of(q))
        if rc == L.NSA_ERR_UNSUPPORTED:
            return False
        L.check(rc)
        if index_cache is not None and shared is None:
            index_cache[cache_key] = ws[:int(lib.nsa_sel_index_bytes(C.byref(args)))].clone()
        _keep_status(ws)
    return True


# --------------------------------------------------------------------------
# sliding window (replaces the LocalAttention call NSA:841-850)
# --------------------------------------------------------------------------

def _swa_args(q, k, v, out, lse, window, causal, impl, scale):
    b, hq, n, d = q.shape
    return L.SwaFwdArgs(q=L.t4(q), k=L.t4(k), v=L.t4(v), out=L.t4(out), lse=L.ptr(lse), batch=b, q_heads=hq,
                        kv_heads=k.shape[1], seq=n, dim_head=d, window=window, causal=int(causal),
                        dtype=L.dtype_code(q), impl=impl, scale=scale, workspace=None, workspace_bytes=0)


class SlidingAttention(Function):
    @staticmethod
    def forward(ctx, q, k, v, window, causal, impl):
        L.require_cuda(q, k, v)
        lib = L.load()
        q, k, v = L.rowwise(q), L.rowwise(k), L.rowwise(v)
        b, hq, n, d = q.shape
        out = _empty_like_rows(q)
        lse = torch.empty(b, hq, n, dtype=torch.float32, device=q.device)
        scale = d ** -0.5
        with torch.cuda.device(q.device):
            args = _swa_args(q, k, v, out, lse, window, causal, impl, scale)
            ws = _with_workspace(args, False, q.device, 'nsa_swa_workspace_bytes')
            L.check(lib.nsa_swa_fwd(C.byref(args), L.stream_of(q)))
            _keep_status(ws)
            del ws
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (window, causal, impl, scale)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse = ctx.saved_tensors
        window, causal, impl, scale = ctx.cfg
        lib = L.load()
        delta = _handed_over_delta(dout, lse.shape)
        dout = L.rowwise(dout)
        dk = torch.empty(k.shape, dtype=torch.float32, device=q.device)
        dv = torch.empty(v.shape, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            fwd = _swa_args(q, k, v, out, lse, window, causal, impl, scale)
            ws = _with_workspace(fwd, True, q.device, 'nsa_swa_workspace_bytes')
            key = ('swa', q.device.index, tuple(q.shape), tuple(k.shape), window, bool(causal), impl)
            index = _cached_index(key)

            def make_args(direct):
                dq, dq_out = _dq_buffers(lib, 'nsa_swa_bwd_stores_dq', fwd, q, need_fp32=not direct)
                return L.SwaBwdArgs(fwd=fwd, dout=L.t4(dout), dq=L.ptr(dq), dk=L.ptr(dk), dv=L.ptr(dv),
                                    dq_out=L.t4(dq_out) if dq_out is not None else L.Tensor4(), index=L.ptr(index),
                                    index_bytes=0 if index is None else index.numel(), delta=L.ptr(delta)), dq, dq_out
            dq = _call_bwd(lib.nsa_swa_bwd, make_args, q, L.stream_of(q))
            if index is None:
                _keep_index(key, ws, int(lib.nsa_swa_index_bytes(C.byref(fwd))))
            _keep_status(ws)
            del ws
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def sliding_window_attend(q, k, v, window, causal, impl='auto', return_lse=False):
    """q [b,qh,n,d]; k, v [b,kh,n,d] (not repeated over the query-head groups)."""
    out, lse = SlidingAttention.apply(q, k, v, window, causal, L.IMPL_BY_NAME[impl])
    return (out, lse) if return_lse else out


# --------------------------------------------------------------------------
# gated combine + head merge (replaces NSA:854-860)
# --------------------------------------------------------------------------

def _pairwise(t):
    ok = t.stride(-1) == 1 and t.data_ptr() % 8 == 0 and all(s % 2 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


class GatedCombine(Function):
    """merged [B,N,H*d] = sum_s gates[...,s] * branch_s; gates [B,H,N,3] (any strides)."""

    @staticmethod
    def forward(ctx, o_cmp, o_sel, o_swa, gates):
        L.require_cuda(o_cmp, o_sel, o_swa, gates)
        lib = L.load()
        o_cmp, o_sel, o_swa = _pairwise(o_cmp), _pairwise(o_sel), _pairwise(o_swa)
        if gates.stride(-1) != 1:
            gates = gates.contiguous()
        b, h, n, d = o_cmp.shape
        out = torch.empty(b, n, h * d, dtype=o_cmp.dtype, device=o_cmp.device)
        args = L.CombineFwdArgs(o_cmp=L.t4(o_cmp), o_sel=L.t4(o_sel), o_swa=L.t4(o_swa), gates=L.t4(gates),
                                out=L.ptr(out), batch=b, q_heads=h, seq=n, dim_head=d, dtype=L.dtype_code(o_cmp))
        with torch.cuda.device(out.device):
            L.check(lib.nsa_combine_fwd(C.byref(args), L.stream_of(out)))
        ctx.save_for_backward(o_cmp, o_sel, o_swa, gates)
        return out

    @staticmethod
    def backward(ctx, dout):
        o_cmp, o_sel, o_swa, gates = ctx.saved_tensors
        lib = L.load()
        dout = dout.contiguous()
        b, h, n, d = o_cmp.shape
        d_cmp, d_sel, d_swa = (torch.empty(b, h, n, d, dtype=o_cmp.dtype, device=o_cmp.device) for _ in range(3))
        d_gates = torch.empty(b, h, n, 3, dtype=torch.float32, device=o_cmp.device)
        # Every branch backward starts from delta = sum_d out_s * d out_s of each row.  With d out_s = gate_s * dout
        # that is gate_s * (sum_d out_s * dout) = gate_s * d gate_s, which this kernel forms anyway: it writes it out,
        # the branch receives it through the gradient tensor it is about to get, and skips its own pass.
        deltas = torch.empty(3, b, h, n, dtype=torch.float32, device=o_cmp.device) if HAND_OVER_DELTA else None
        fwd = L.CombineFwdArgs(o_cmp=L.t4(o_cmp), o_sel=L.t4(o_sel), o_swa=L.t4(o_swa), gates=L.t4(gates),
                               out=None, batch=b, q_heads=h, seq=n, dim_head=d, dtype=L.dtype_code(o_cmp))
        args = L.CombineBwdArgs(fwd=fwd, dout=L.ptr(dout), d_cmp=L.ptr(d_cmp), d_sel=L.ptr(d_sel),
                                d_swa=L.ptr(d_swa), d_gates=L.ptr(d_gates), delta=L.ptr(deltas))
        with torch.cuda.device(dout.device):
            L.check(lib.nsa_combine_bwd(C.byref(args), L.stream_of(dout)))
        if deltas is not None:
            for s_, t_ in enumerate((d_cmp, d_sel, d_swa)):
                t_._nsa_delta = deltas[s_]
        return d_cmp, d_sel, d_swa, d_gates.to(gates.dtype)


def gated_combine(o_cmp, o_sel, o_swa, gates):
    return GatedCombine.apply(o_cmp, o_sel, o_swa, gates)


def _vec_ok(t):
    v = 16 // t.element_size()
    return t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % v == 0 for s in t.stride()[:-1])


def gated_combine_gather(o_cmp, o_sel, o_swa, gates, out_ptrs, total_features, feature_offset, multicast=False):
    """Forward-only gated combine of this rank's heads, written at `feature_offset` into every [B, N, total_features]
    buffer whose device address is listed in `out_ptrs` (own buffer and the peers' mappings): the combine fused with
    the all-gather of the head-sharded layout.  With `multicast`, `out_ptrs` is the one multicast address of the
    symmetric buffer and every piece is stored once (multimem.st), the switch writing all ranks' copies.  The caller
    synchronises the ranks around the call."""
    L.require_cuda(o_cmp, o_sel, o_swa, gates)
    lib = L.load()
    o_cmp, o_sel, o_swa = (t if _vec_ok(t) else t.contiguous() for t in (o_cmp, o_sel, o_swa))
    if gates.stride(-1) != 1:
        gates = gates.contiguous()
    b, h, n, d = o_cmp.shape
    if not 1 <= len(out_ptrs) <= L.MAX_GATHER:
        raise ValueError(f'between 1 and {L.MAX_GATHER} destinations, got {len(out_ptrs)}')
    fwd = L.CombineFwdArgs(o_cmp=L.t4(o_cmp), o_sel=L.t4(o_sel), o_swa=L.t4(o_swa), gates=L.t4(gates), out=None,
                           batch=b, q_heads=h, seq=n, dim_head=d, dtype=L.dtype_code(o_cmp))
    outs = (C.c_void_p * L.MAX_GATHER)(*[int(p) for p in out_ptrs])
    args = L.CombineGatherArgs(fwd=fwd, outs=outs, num_outs=len(out_ptrs), multicast=int(bool(multicast)),
                               total_features=total_features, feature_offset=feature_offset)
    with torch.cuda.device(o_cmp.device):
        L.check(lib.nsa_combine_fwd_gather(C.byref(args), L.stream_of(o_cmp)))


# --------------------------------------------------------------------------
# one decoding step (replaces the attention part of upstream's forward_inference, NSA:387-547)
# --------------------------------------------------------------------------

@torch.no_grad()
def decode_step(q, qr, keys, vals, ck, cv, mem_k, mem_v, gates, *, stride, block, num_selected, window):
    """The newest token against the caches, one kernel launch.  q, qr [B, Hq, d]: un-rotated / rotated queries of
    the token; keys, vals [B, Hkv, T, d]: rotated keys and values with the token appended; ck, cv [B, Hkv, ncb, d]:
    the blocks compressed so far (without memory slots, ncb may be 0); mem_k, mem_v [Hkv, M, d]; gates [B, Hq, 3]
    (compressed, selected, sliding).  Returns the merged row [B, Hq * d].  See nsa_decode_step in include/nsa_b200.h."""
    L.require_cuda(q, qr, keys, vals, ck, cv, mem_k, mem_v, gates)
    lib = L.load()
    dt = q.dtype
    q, qr, gates = q.contiguous(), qr.to(dt).contiguous(), gates.to(dt).contiguous()
    mem_k, mem_v = mem_k.to(dt).contiguous(), mem_v.to(dt).contiguous()
    keys, vals = L.rowwise(keys.to(dt)), L.rowwise(vals.to(dt))
    b, hq, d = q.shape
    ncb = ck.shape[2]
    if ncb > 0:
        ck, cv = L.rowwise(ck.to(dt)), L.rowwise(cv.to(dt))
    out = torch.empty(b, hq * d, dtype=dt, device=q.device)
    args = L.DecodeArgs(q=L.ptr(q), qr=L.ptr(qr), keys=L.t4(keys), vals=L.t4(vals),
                        ck=L.t4(ck) if ncb > 0 else L.Tensor4(), cv=L.t4(cv) if ncb > 0 else L.Tensor4(),
                        mem_k=L.ptr(mem_k), mem_v=L.ptr(mem_v), gates=L.ptr(gates), out=L.ptr(out), batch=b,
                        q_heads=hq, kv_heads=keys.shape[1], dim_head=d, cache_len=keys.shape[2], ncb=ncb,
                        num_mem=mem_k.shape[1], stride=stride, block=block, nsel=num_selected, window=window,
                        dtype=L.dtype_code(q), scale=d ** -0.5, reserved=0)
    with torch.cuda.device(q.device):
        L.check(lib.nsa_decode_step(C.byref(args), L.stream_of(q)))
    return out


# --------------------------------------------------------------------------
# input of the compress networks: windows + intra-block positions (NSA:589-614)
# --------------------------------------------------------------------------

class CompressWindows(Function):
    """out[b,h,w,j,:] = x[b,h,(w+1)*stride - block + j,:] (zero before the start) + pos[h,j,:], w < ncb."""

    @staticmethod
    def forward(ctx, x, pos, block, stride, ncb):
        L.require_cuda(x, pos)
        lib = L.load()
        if not _vec_ok(x):
            x = x.contiguous()
        pos = pos.contiguous()
        b, h, n, d = x.shape
        out = torch.empty(b, h, ncb, block, d, dtype=x.dtype, device=x.device)
        args = L.WindowsFwdArgs(x=L.t4(x), pos=L.ptr(pos), out=L.ptr(out), batch=b, heads=h, seq=n, dim_head=d,
                                block=block, stride=stride, ncb=ncb, dtype=L.dtype_code(x))
        with torch.cuda.device(x.device):
            L.check(lib.nsa_windows_fwd(C.byref(args), L.stream_of(x)))
        ctx.cfg = (b, h, n, d, block, stride, ncb, x.dtype, pos.dtype, dim_order(x))
        return out

    @staticmethod
    def backward(ctx, dout):
        b, h, n, d, block, stride, ncb, xdtype, pdtype, order = ctx.cfg
        lib = L.load()
        dout = dout.contiguous()
        dx = empty_in_order((b, h, n, d), order, xdtype, dout.device)   # in the layout of x: see _empty_in_order_of
        dpos = torch.empty(h, block, d, dtype=torch.float32, device=dout.device)
        fwd = L.WindowsFwdArgs(x=L.Tensor4(), pos=None, out=None, batch=b, heads=h, seq=n, dim_head=d, block=block,
                               stride=stride, ncb=ncb, dtype=L.dtype_code(dout))
        args = L.WindowsBwdArgs(fwd=fwd, dout=L.ptr(dout), dx=L.ptr(dx), dpos=L.ptr(dpos), dx_stride_b=dx.stride(0),
                                dx_stride_h=dx.stride(1), dx_stride_n=dx.stride(2))
        with torch.cuda.device(dout.device):
            L.check(lib.nsa_windows_bwd(C.byref(args), L.stream_of(dout)))
        return dx, dpos.to(pdtype), None, None, None


def compress_windows(x, pos, block, stride, ncb):
    """Windows of `block` rows every `stride` rows of x [B,H,N,d] plus the intra-block positions pos [H,block,d]:
    the input of the compress networks, [B,H,ncb,block,d]."""
    return CompressWindows.apply(x, pos, block, stride, ncb)


def compress_windows_supported(x):
    v = 16 // x.element_size()
    d = x.shape[-1]
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and d % v == 0 and d <= 256 and 256 % d == 0
