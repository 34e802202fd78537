"""CPU oracle for the Native Sparse Attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch ops that run on the host, the algorithm of
the upstream pure-PyTorch ``SparseAttention.forward`` path
(native_sparse_attention_pytorch/native_sparse_attention.py, cited below as
NSA:<line>) and of the kernel-level reference ``regular_attend``
(test_triton_nsa.py:32-133).  It is the checker the CUDA kernels are compared
with; nothing in the shipped package imports it.  Only the tests, the smoke
entry and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the unmodified
upstream library (with three small stand-ins for packages that are not
installed) and stores its outputs, gradients and intermediate tensors on
seeded inputs; ``tests/test_oracle_golden.py`` checks every function here
against those stored vectors.  One convention is not pinned by upstream's own
tests: the rotary embedding layout (adjacent feature pairs, base 10000), which
only affects tensors produced before the hot path.

Every function is written for clarity, not speed, and works in the dtype of
its inputs exactly like the upstream code (so a bf16 run reproduces upstream's
rounding chain).  Gradients come from autograd over these functions.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


def neg_max(t: torch.Tensor) -> float:
    """Most negative finite value of t's dtype (NSA:131-132)."""
    return -torch.finfo(t.dtype).max


# --------------------------------------------------------------------------
# producers of the hot path's inputs (kept as PyTorch in the product as well)
# --------------------------------------------------------------------------

def rotary(t: torch.Tensor, offset: int = 0, theta: float = 10000.0) -> torch.Tensor:
    """Rotary position embedding on the last two axes (positions offset..offset+n-1).

    Call sites NSA:643 and NSA:384-385.  Convention: inverse frequency
    theta^(-2m/d) on the adjacent feature pair (2m, 2m+1); angles in fp32;
    result cast back to t.dtype.
    """
    n, d = t.shape[-2:]
    inv_freq = theta ** (-torch.arange(0, d, 2, device=t.device).float() / d)
    pos = torch.arange(n, device=t.device).float() + offset
    ang = pos[:, None] * inv_freq[None, :]
    cos = ang.cos().repeat_interleave(2, dim=-1)
    sin = ang.sin().repeat_interleave(2, dim=-1)
    x = t.float()
    even, odd = x[..., 0::2], x[..., 1::2]
    rotated = torch.stack((-odd, even), dim=-1).flatten(-2)
    return (x * cos + rotated * sin).to(t.dtype)


def compress_windows(t: torch.Tensor, cbs: int, st: int) -> torch.Tensor:
    """[B,H,N,d] -> [B,H,ncb,cbs,d]: window w holds tokens (w+1)*st-cbs .. (w+1)*st-1,
    zeros where the position is negative (NSA:270-275, 589-595)."""
    b, h, n, d = t.shape
    ncb = n // st
    if ncb == 0:
        return t.new_zeros(b, h, 0, cbs, d)
    t = F.pad(t[:, :, : ncb * st], (0, 0, cbs - st, 0))
    return t.unfold(2, cbs, st).permute(0, 1, 2, 4, 3)


# --------------------------------------------------------------------------
# branch 1: attention over the compressed keys, returning its logits
# --------------------------------------------------------------------------

def compressed_attend(q, ck, cv, mem_k, mem_v, st: int, causal: bool, rows=None):
    """NSA:621-639 with ``attend`` NSA:153-184.

    q [B,Hq,N,d] (not rotated); ck, cv [B,Hkv,ncb,d]; mem_k, mem_v [Hkv,M,d].
    Returns (out [B,Hq,N,d], csim [B,Hq,N,M+ncb]).  Compressed key w is visible
    to a causal query i iff (w+1)*st-1 < i; memory slots are always visible.
    Invisible logits are *replaced* by (-finfo.max)//10, a finite sentinel.
    ``rows`` (1-D int64) restricts the computation to those query positions
    (used to check samples of large cases); N in the results is then len(rows).
    """
    b, hq, _, d = q.shape
    hkv, m = mem_k.shape[0], mem_k.shape[1]
    g = hq // hkv
    pos = torch.arange(q.shape[2], device=q.device) if rows is None else rows
    if rows is not None:
        q = q[:, :, rows]
    n = pos.numel()
    keys = torch.cat((mem_k.expand(b, -1, -1, -1), ck), dim=-2)
    vals = torch.cat((mem_v.expand(b, -1, -1, -1), cv), dim=-2)
    qg = q.reshape(b, hkv, g, n, d)
    sim = torch.einsum('bhgid,bhjd->bhgij', qg, keys) * (d ** -0.5)
    if causal:
        last_token = (torch.arange(ck.shape[-2], device=q.device) + 1) * st - 1
        last_token = F.pad(last_token, (m, 0), value=-1)
        visible = last_token[None, :] < pos[:, None]
        sim = sim.masked_fill(~visible, neg_max(sim) // 10)
    attn = sim.softmax(dim=-1)
    out = torch.einsum('bhgij,bhjd->bhgid', attn, vals)
    return out.reshape(b, hq, n, d), sim.reshape(b, hq, n, -1)


# --------------------------------------------------------------------------
# selection: importance reduction and top-k
# --------------------------------------------------------------------------

def importance_scores(csim, num_mem: int, hkv: int, st: int, sel: int, share_heads: bool = True, rows=None):
    """NSA:652-695.  csim [B,Hq,N,M+ncb] -> probabilities [B,Hsel,N,cols].

    Steps, each rounded to the tensor dtype as upstream does: drop the memory
    columns; mean over the G query heads of a KV head (if shared); if st != sel
    truncate to a multiple of cpf = sel//st columns, mean over each cpf
    consecutive columns and overwrite the query's own block column with
    -finfo.max; prepend a sink column of -1000; softmax; drop the sink.
    ``rows`` gives the query positions when csim holds a subset of the queries.
    """
    imp = csim[..., num_mem:]
    b, hq, n, _ = imp.shape
    if share_heads:
        imp = imp.reshape(b, hkv, hq // hkv, n, -1).mean(dim=2)
    if st != sel:
        cpf = sel // st
        cols = imp.shape[-1] // cpf
        imp = imp[..., : cols * cpf]
        if imp.numel() > 0:
            imp = imp.reshape(*imp.shape[:-1], cols, cpf).mean(dim=-1)
            own = (torch.arange(n, device=imp.device) if rows is None else rows) // sel
            diag = own[:, None] == torch.arange(cols, device=imp.device)[None, :]
            imp = imp.masked_fill(diag, neg_max(csim))
    imp = F.pad(imp, (1, 0), value=-1e3)
    return imp.softmax(dim=-1)[..., 1:]


def select_blocks(probs, nsel: int):
    """NSA:703-713: top-k over the block probabilities; k is clipped to the
    number of columns.  Returns (values, int64 indices), sorted by value."""
    k = min(nsel, probs.shape[-1])
    return probs.topk(k, dim=-1)


# --------------------------------------------------------------------------
# branch 2: attention over the selected blocks
# --------------------------------------------------------------------------

def selected_attend(fq, fk, fv, sel: int, idx, fmask, causal: bool, gates=None,
                    rows=None, return_lse: bool = False):
    """Gather formulation of the selected-block branch, NSA:741-819 (and the
    equivalent kernel-level statement test_triton_nsa.py:32-133).

    fq [B,Hq,N,d]; fk, fv [B,Hkv,N,d]; idx (int64), fmask (bool), gates
    [B,Hs,N,nsel] with Hs == Hkv (shared) or Hq.  Query i of head group h
    attends the ``sel`` keys of every block idx[b,h,i,s] whose fmask is true
    and, when ``causal``, keys floor(i/sel)*sel..i of its own block.  K and V
    are zero-padded to a multiple of ``sel``; padded keys inside a selected
    block take part with logit 0 exactly as upstream's padding does.  Slots
    with fmask false get logit -finfo.max (not -inf), so a row with no visible
    key at all is a uniform average.  ``gates`` multiplies the keys of a slot
    (differentiable top-k, NSA:793-797).  ``rows`` (1-D int64) restricts the
    computation to those query positions (used to check samples of large cases).
    """
    b, hq, n, d = fq.shape
    hkv, hs = fk.shape[1], idx.shape[1]
    if hs != hkv:  # per-query-head selection: every query head is its own group
        rep = hq // hkv
        fk = fk.repeat_interleave(rep, dim=1)
        fv = fv.repeat_interleave(rep, dim=1)
        hkv = hq
    g = hq // hkv
    nfb = math.ceil(n / sel)
    pad = nfb * sel - n
    kb = F.pad(fk, (0, 0, 0, pad)).reshape(b, hkv, nfb, sel, d)
    vb = F.pad(fv, (0, 0, 0, pad)).reshape(b, hkv, nfb, sel, d)

    pos = torch.arange(n, device=fq.device) if rows is None else rows
    r = pos.numel()
    q = fq[:, :, pos].reshape(b, hkv, g, r, d)
    idx_r = idx[:, :, pos]
    keep = fmask[:, :, pos][..., None].expand(-1, -1, -1, -1, sel)   # b h r s j
    if gates is not None:
        gates = gates[:, :, pos]
    if causal:
        own = (pos // sel)[None, None, :, None].expand(b, hkv, r, 1)
        idx_r = torch.cat((idx_r, own), dim=-1)
        tri = (torch.arange(sel, device=fq.device)[None, :] <= (pos % sel)[:, None])
        keep = torch.cat((keep, tri[None, None, :, None, :].expand(b, hkv, r, 1, sel)), dim=3)
        if gates is not None:
            gates = F.pad(gates, (0, 1), value=1.)
    ns = idx_r.shape[-1]
    bi = torch.arange(b, device=fq.device)[:, None, None, None]
    hi = torch.arange(hkv, device=fq.device)[None, :, None, None]
    gk = kb[bi, hi, idx_r]            # b h r s j d
    gv = vb[bi, hi, idx_r]
    if gates is not None:
        gk = gk * gates[..., None, None]
    gk = gk.reshape(b, hkv, r, ns * sel, d)
    gv = gv.reshape(b, hkv, r, ns * sel, d)
    keep = keep.reshape(b, hkv, 1, r, ns * sel)
    sim = torch.einsum('bhgid,bhijd->bhgij', q, gk) * (d ** -0.5)
    sim = sim.masked_fill(~keep, neg_max(sim))
    out = torch.einsum('bhgij,bhijd->bhgid', sim.softmax(dim=-1), gv).reshape(b, hq, r, d)
    if not return_lse:
        return out
    return out, sim.logsumexp(dim=-1).reshape(b, hq, r)


def block_diagonal_attend(fq, fk, fv, sel: int, causal: bool):
    """NSA:821-837: when nothing can be selected, every query attends only its
    own ``sel``-block (lower-triangular if causal, the whole zero-padded block
    otherwise)."""
    b, hq, n, d = fq.shape
    hkv = fk.shape[1]
    g = hq // hkv
    nfb = math.ceil(n / sel)
    pad = nfb * sel - n
    q = F.pad(fq, (0, 0, 0, pad)).reshape(b, hkv, g, nfb, sel, d)
    k = F.pad(fk, (0, 0, 0, pad)).reshape(b, hkv, nfb, sel, d)
    v = F.pad(fv, (0, 0, 0, pad)).reshape(b, hkv, nfb, sel, d)
    sim = torch.einsum('bhgwid,bhwjd->bhgwij', q, k) * (d ** -0.5)
    if causal:
        tri = torch.ones(sel, sel, dtype=torch.bool, device=fq.device).tril()
        sim = sim.masked_fill(~tri, neg_max(sim) // 10)
    out = torch.einsum('bhgwij,bhwjd->bhgwid', sim.softmax(dim=-1), v)
    return out.reshape(b, hq, nfb * sel, d)[:, :, :n]


# --------------------------------------------------------------------------
# branch 3: sliding window, and the gated combine
# --------------------------------------------------------------------------

def sliding_attend(q, k, v, window: int, causal: bool, rows=None):
    """NSA:841-850.  Causal: keys j with 0 <= i-j <= window (window+1 keys,
    cf. NSA:524-530); non-causal: |i-j| <= window (NSA:46-56).  ``rows``
    restricts the computation to those query positions."""
    b, hq, _, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    kpos = torch.arange(k.shape[2], device=q.device)
    pos = kpos if rows is None else rows
    if rows is not None:
        q = q[:, :, rows]
    n = pos.numel()
    dist = pos[:, None] - kpos[None, :]
    visible = (dist <= window) & (dist >= (0 if causal else -window))
    sim = torch.einsum('bhgid,bhjd->bhgij', q.reshape(b, hkv, g, n, d), k) * (d ** -0.5)
    sim = sim.masked_fill(~visible, neg_max(sim))
    return torch.einsum('bhgij,bhjd->bhgid', sim.softmax(dim=-1), v).reshape(b, hq, n, d)


def combine(o_cmp, o_sel, o_swa, gates):
    """NSA:854-860: out[b,n,(h d)] = sum_s gates[b,h,n,s] * branch_s[b,h,n,:],
    branch order (compressed, selected, sliding)."""
    out = (gates[..., 0:1] * o_cmp + gates[..., 1:2] * o_sel + gates[..., 2:3] * o_swa)
    b, h, n, d = out.shape
    return out.permute(0, 2, 1, 3).reshape(b, n, h * d)


# --------------------------------------------------------------------------
# the whole layer (same parameter names as upstream, NSA:189-336)
# --------------------------------------------------------------------------

class OracleSparseAttention(nn.Module):
    """Restatement of ``SparseAttention`` (NSA:188-336, forward NSA:549-867,
    parallel mode only) built from the functions above.  Parameters are created
    in upstream's order so that the same seed gives the same weights, and carry
    upstream's names so a state_dict can be exchanged."""

    def __init__(self, dim, dim_head, heads, sliding_window_size, compress_block_size,
                 compress_block_sliding_stride, selection_block_size, num_selected_blocks,
                 kv_heads=None, num_compressed_mem_kv=1, causal=False, norm=True,
                 use_diff_topk=False, query_heads_share_selected_kv=True,
                 compress_mlp_expand_factor=1.):
        super().__init__()
        kv_heads = heads if kv_heads is None else kv_heads
        self.heads, self.kv_heads, self.dim_head = heads, kv_heads, dim_head
        self.causal = causal
        self.window = sliding_window_size
        self.cbs, self.st = compress_block_size, compress_block_sliding_stride
        self.sel, self.nsel = selection_block_size, num_selected_blocks
        self.use_diff_topk = use_diff_topk
        self.share = query_heads_share_selected_kv
        self.num_mem = num_compressed_mem_kv
        self.norm = nn.RMSNorm(dim) if norm else nn.Identity()
        self.qkv_split = (dim_head * heads, dim_head * kv_heads, dim_head * kv_heads)
        self.to_qkv = nn.Linear(dim, sum(self.qkv_split), bias=False)
        self.compress_mem_kv = nn.Parameter(torch.zeros(2, kv_heads, num_compressed_mem_kv, dim_head))
        self.k_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))
        self.v_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))
        cdim = compress_block_size * dim_head
        hidden = int(compress_mlp_expand_factor * cdim)
        mlp = nn.Sequential(nn.Flatten(-2), nn.Linear(cdim, hidden), nn.ReLU(), nn.Linear(hidden, dim_head))
        import copy
        self.k_compress, self.v_compress = copy.deepcopy(mlp), copy.deepcopy(mlp)
        gate = nn.Linear(dim, 3 * heads)
        nn.init.zeros_(gate.weight)
        gate.bias.data.copy_(torch.tensor([-2., -2., 2.] * heads))
        self.to_strategy_combine = nn.Sequential(gate, nn.Sigmoid())
        self.combine_heads = nn.Linear(dim_head * heads, dim, bias=False)

    def forward(self, inp, return_intermediates: bool = False, forced_selection=None):
        """``forced_selection`` = (idx, fmask) replaces the layer's own block selection (the tests use it to compare
        two precisions of the layer on identical blocks)."""
        b, n, _ = inp.shape
        h, hkv, d = self.heads, self.kv_heads, self.dim_head
        x = self.norm(inp)
        q, k, v = self.to_qkv(x).split(self.qkv_split, dim=-1)
        q, k, v = (t.reshape(b, n, -1, d).transpose(1, 2) for t in (q, k, v))

        kw = compress_windows(k, self.cbs, self.st)
        vw = compress_windows(v, self.cbs, self.st)
        if kw.numel() > 0:
            kw = kw + self.k_intrablock_positions[None, :, None]
            vw = vw + self.v_intrablock_positions[None, :, None]
        ck, cv = self.k_compress(kw), self.v_compress(vw)

        o_cmp, csim = compressed_attend(q, ck, cv, self.compress_mem_kv[0], self.compress_mem_kv[1],
                                        self.st, self.causal)
        qr, kr = rotary(q), rotary(k)

        ncb = n // self.st
        num_selected = min(self.nsel, ncb)
        probs = None
        if num_selected > 0:
            probs = importance_scores(csim, self.num_mem, hkv, self.st, self.sel, self.share)
            num_selected = min(num_selected, probs.shape[-1])
        vals = idx = fmask = None
        if num_selected > 0:
            vals, idx = select_blocks(probs, num_selected)
            fmask = vals > 1e-10
            if forced_selection is not None:
                idx, fmask = forced_selection
            gates_topk = (vals + (1. - vals).detach()) if self.use_diff_topk else None
            o_sel = selected_attend(qr, kr, v, self.sel, idx, fmask, self.causal, gates=gates_topk)
        else:
            o_sel = block_diagonal_attend(qr, kr, v, self.sel, self.causal)

        o_swa = sliding_attend(qr, kr, v, self.window, self.causal)
        gates = self.to_strategy_combine(x).reshape(b, n, h, 3).transpose(1, 2)
        merged = combine(o_cmp, o_sel, o_swa, gates)
        out = self.combine_heads(merged)
        if not return_intermediates:
            return out
        return out, dict(q=q, k=k, v=v, ck=ck, cv=cv, qr=qr, kr=kr, csim=csim, probs=probs,
                         vals=vals, idx=idx, fmask=fmask, o_cmp=o_cmp, o_sel=o_sel, o_swa=o_swa,
                         gates=gates, merged=merged)
