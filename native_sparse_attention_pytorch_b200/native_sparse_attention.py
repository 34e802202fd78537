"""Drop-in ``SparseAttention`` layer whose hot path -- compressed attention,
block selection, selected-block attention, sliding window and the gated
combine -- runs on the B200 kernels of libnsa_b200.so.

Constructor arguments, parameter names and the forward signature follow
upstream's module (NSA:189-209, NSA:549-557), so a state_dict moves between
the two.  Only the accelerated path exists here: the layer must be built with
``use_triton_kernel=True`` (upstream's name for "use the fused kernel", kept
for compatibility) and called on CUDA tensors; anything else raises instead of
silently computing somewhere else."""
from copy import deepcopy

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import Module

from . import ops
from .norm import RMSNorm
from .rotary import RotaryEmbedding


class _Windows(Module):
    """[B,H,N,d] -> [B,H,ncb,cbs,d]: window w holds tokens (w+1)*stride-cbs .. (w+1)*stride-1,
    zero where that is negative (same result as upstream's pad + unfold, NSA:270-275)."""

    def __init__(self, block, stride):
        super().__init__()
        self.block, self.stride = block, stride

    def forward(self, t):
        t = F.pad(t, (0, 0, self.block - self.stride, 0))
        return t.unfold(2, self.block, self.stride).permute(0, 1, 2, 4, 3)


class SparseAttention(Module):
    def __init__(
        self,
        dim,
        dim_head,
        heads,
        sliding_window_size,
        compress_block_size,
        compress_block_sliding_stride,
        selection_block_size,
        num_selected_blocks,
        kv_heads=None,
        num_compressed_mem_kv=1,
        causal=False,
        norm=True,
        use_diff_topk=False,
        use_triton_kernel=False,
        query_heads_share_selected_kv=True,
        compress_mlp: Module | None = None,
        compress_mlp_expand_factor=1.,
        strategy_combine_mlp: Module | None = None,
        kernel_impl='auto',
    ):
        super().__init__()
        kv_heads = heads if kv_heads is None else kv_heads
        assert kv_heads <= heads and heads % kv_heads == 0
        self.heads, self.kv_heads, self.dim_head = heads, kv_heads, dim_head
        self.num_grouped_queries = heads // kv_heads
        self.scale = dim_head ** -0.5
        self.causal = causal
        self.kernel_impl = kernel_impl

        self.norm = RMSNorm(dim) if norm else nn.Identity()
        self.rotary_emb = RotaryEmbedding(dim_head)
        self.qkv_split = (dim_head * heads, dim_head * kv_heads, dim_head * kv_heads)
        self.to_qkv = nn.Linear(dim, sum(self.qkv_split), bias=False)

        self.sliding_window_size = sliding_window_size

        self.compress_block_size = compress_block_size
        self.compress_block_sliding_stride = compress_block_sliding_stride
        assert compress_block_size >= compress_block_sliding_stride, 'compress_block_size must be >= compress_block_sliding_stride'
        assert compress_block_sliding_stride > 0, 'compress_block_sliding_stride must be greater than 0'
        assert selection_block_size % compress_block_sliding_stride == 0, \
            f'selection_block_size {selection_block_size} must be divisible by compress_block_sliding_stride {compress_block_sliding_stride}'
        self.split_compress_window = _Windows(compress_block_size, compress_block_sliding_stride)

        assert num_compressed_mem_kv > 0
        self.num_mem_compress_kv = num_compressed_mem_kv
        self.compress_mem_kv = nn.Parameter(torch.zeros(2, kv_heads, num_compressed_mem_kv, dim_head))
        self.k_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))
        self.v_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))

        if compress_mlp is None:
            compress_dim = compress_block_size * dim_head
            hidden = int(compress_mlp_expand_factor * compress_dim)
            # index 0 flattens (n d) so the Linear layers sit at indices 1 and 3 as upstream's do
            compress_mlp = nn.Sequential(nn.Flatten(-2), nn.Linear(compress_dim, hidden), nn.ReLU(),
                                         nn.Linear(hidden, dim_head))
        self.k_compress = deepcopy(compress_mlp)
        self.v_compress = deepcopy(compress_mlp)

        self.use_diff_topk = use_diff_topk
        self.query_heads_share_selected_kv = query_heads_share_selected_kv
        self.selection_block_size = selection_block_size
        assert num_selected_blocks >= 0
        if num_selected_blocks == 0:
            print('`num_selected_blocks` should be set greater than 0, unless if you are ablating it for experimental purposes')
        self.num_selected_blocks = num_selected_blocks
        self.use_triton_kernel = use_triton_kernel

        if strategy_combine_mlp is None:
            strategy_combine_mlp = nn.Linear(dim, 3 * heads)
            nn.init.zeros_(strategy_combine_mlp.weight)
            strategy_combine_mlp.bias.data.copy_(torch.tensor([-2., -2., 2.] * heads))
        self.to_strategy_combine = nn.Sequential(strategy_combine_mlp, nn.Sigmoid())

        self.combine_heads = nn.Linear(dim_head * heads, dim, bias=False)

    def _split_heads(self, t):
        b, n, _ = t.shape
        return t.view(b, n, -1, self.dim_head).transpose(1, 2)   # a view: the kernels take the strides

    def forward_inference(self, inp, cache, return_cache=True):
        """One decoding step (upstream NSA:338-547): `inp` is the newest token [B, 1, dim], `cache` what the previous
        call returned: ((rotated keys, values), ((compressed keys, compressed values), (keys, values of the window
        that is being filled for the next compressed block, un-rotated))).  The attention part -- compressed branch,
        block selection, selected blocks plus the own block, sliding window, gated combine -- is one kernel launch
        (`ops.decode_step`, all (batch, KV head) units in its grid); the projections, the rotary kernel and the
        compress network of a window that has just filled up stay tensor operations.  It keeps upstream's behaviour,
        including that the memory slots are attended only once a compressed block exists."""
        assert self.causal, 'inference only relevant for autoregressive'
        if not self.query_heads_share_selected_kv:
            raise NotImplementedError('decoding with per-query-head selection is not built (upstream gathers K/V with '
                                      'indices of the wrong head count in that case)')
        (past_k, past_v), ((ck, cv), (run_k, run_v)) = cache
        b = inp.shape[0]
        h, d = self.heads, self.dim_head
        st, cbs, sel = self.compress_block_sliding_stride, self.compress_block_size, self.selection_block_size
        pos = past_k.shape[-2]                       # position of the new token
        x = self.norm(inp)
        q, k, v = (self._split_heads(t).contiguous() for t in self.to_qkv(x).split(self.qkv_split, dim=-1))
        run_k, run_v = torch.cat((run_k, k), dim=-2), torch.cat((run_v, v), dim=-2)   # compression sees un-rotated k, v
        qr = self.rotary_emb.rotate_queries_or_keys(q, offset=pos)
        keys = torch.cat((past_k, self.rotary_emb.rotate_queries_or_keys(k, offset=pos)), dim=-2)
        vals = torch.cat((past_v, v), dim=-2)

        gates = self.to_strategy_combine(x).view(b, h, 3)
        merged = ops.decode_step(q.view(b, h, d), qr.view(b, h, d), keys, vals, ck, cv, self.compress_mem_kv[0],
                                 self.compress_mem_kv[1], gates, stride=st, block=sel,
                                 num_selected=self.num_selected_blocks, window=self.sliding_window_size)

        # the window that was being filled is complete: compress it and keep its overlap with the next one (the step
        # above attended the blocks that existed before this token, as upstream's does)
        if run_k.shape[-2] % cbs == 0:
            ck = torch.cat((ck, self.k_compress((run_k + self.k_intrablock_positions)[:, :, None])), dim=-2)
            cv = torch.cat((cv, self.v_compress((run_v + self.v_intrablock_positions)[:, :, None])), dim=-2)
            keep = cbs - st
            run_k, run_v = run_k[..., run_k.shape[-2] - keep:, :], run_v[..., run_v.shape[-2] - keep:, :]

        out = self.combine_heads(merged.view(b, 1, h * d))
        if not return_cache:
            return out
        return out, ((keys, vals), ((ck, cv), (run_k, run_v)))

    def forward(
        self,
        inp,
        cache=None,
        disable_triton_kernel=False,
        sliding_window_flex_mask=None,
        fine_selection_flex_mask=None,
        return_cache=False,
        return_intermediates=False,
        forced_selection=None,
    ):
        """Upstream's signature (NSA:549-557) plus two keyword arguments of this package: ``return_intermediates``
        also returns the tensors at the boundaries of the hot path, and ``forced_selection`` = (block indices,
        mask), both [B, Hs, N, k], replaces the layer's own block selection (used to compare two precisions of the
        layer on identical blocks).  A tensor-core kernel of an earlier call that gave up on a bounded wait is
        reported here, one call late and without synchronising (`ops.poll_device_status`)."""
        if inp.is_cuda:
            ops.poll_device_status(inp.device)
        if cache is not None:
            if not inp.is_cuda:
                raise RuntimeError('SparseAttention (B200 kernels) needs CUDA tensors; there is no CPU path here')
            return self.forward_inference(inp, cache, return_cache=return_cache)
        if not self.use_triton_kernel or disable_triton_kernel:
            raise RuntimeError('this package implements only the fused-kernel path: construct SparseAttention with '
                               'use_triton_kernel=True and do not pass disable_triton_kernel')
        if sliding_window_flex_mask is not None or fine_selection_flex_mask is not None:
            raise RuntimeError('flex-attention masks select another backend upstream; this package has one backend')
        if not inp.is_cuda:
            raise RuntimeError('SparseAttention (B200 kernels) needs CUDA tensors; there is no CPU path here')
        assert not (not self.causal and return_cache)

        b, n, _ = inp.shape
        h, hkv, d = self.heads, self.kv_heads, self.dim_head
        st, sel = self.compress_block_sliding_stride, self.selection_block_size
        impl = self.kernel_impl
        ncb = n // st

        x = self.norm(inp)
        q, k, v = self.to_qkv(x).split(self.qkv_split, dim=-1)
        q, k, v = map(self._split_heads, (q, k, v))

        # compressed keys / values: plug-in networks on un-rotated k, v (NSA:589-614)
        if ncb > 0 and ops.compress_windows_supported(k):
            kw = ops.compress_windows(k, self.k_intrablock_positions, self.compress_block_size, st, ncb)
            vw = ops.compress_windows(v, self.v_intrablock_positions, self.compress_block_size, st, ncb)
        elif ncb > 0:
            kw = self.split_compress_window(k[..., : ncb * st, :]) + self.k_intrablock_positions[None, :, None]
            vw = self.split_compress_window(v[..., : ncb * st, :]) + self.v_intrablock_positions[None, :, None]
        else:
            kw = k.new_zeros(b, hkv, 0, self.compress_block_size, d)
            vw = v.new_zeros(b, hkv, 0, self.compress_block_size, d)
        ck, cv = self.k_compress(kw), self.v_compress(vw)

        if return_cache:
            overlap = self.compress_block_size - st
            run_k, run_v = k, v
            if overlap > 0:
                run_k, run_v = F.pad(run_k, (0, 0, overlap, 0)), F.pad(run_v, (0, 0, overlap, 0))
            cache_compressed = ((ck, cv), (run_k[..., ncb * st:, :], run_v[..., ncb * st:, :]))

        # branch 1: compressed attention, with the per-block importance as a by-product
        num_mem = self.num_mem_compress_kv
        mem_k, mem_v = self.compress_mem_kv[0].expand(b, -1, -1, -1), self.compress_mem_kv[1].expand(b, -1, -1, -1)
        ck_full, cv_full = torch.cat((mem_k, ck), dim=-2), torch.cat((mem_v, cv), dim=-2)
        sel_heads = hkv if self.query_heads_share_selected_kv else h
        num_selected = min(self.num_selected_blocks, ncb, ncb // (sel // st))
        # the kernel also averages the logits per selection block where it can, unless their gradient is wanted
        pool = sel // st if self.causal and not self.use_diff_topk and sel % st == 0 else 0
        o_cmp, importance = ops.compressed_attend(q, ck_full, cv_full, num_mem, st, self.causal, sel_heads=sel_heads,
                                                  want_importance=True, impl=impl, pool=pool) if num_selected > 0 else \
            (ops.compressed_attend(q, ck_full, cv_full, num_mem, st, self.causal, want_importance=False, impl=impl), None)

        qr, kr = self.rotary_emb.rotate_queries_with_cached_keys(q, k)
        if return_cache:
            cache_kv = (kr, v)

        # branch 2: block selection, then attention over the selected blocks
        idx = vals = fmask = None
        if num_selected > 0:
            vals, idx = ops.select_blocks(importance if self.use_diff_topk else importance.detach(), sel, st,
                                          num_selected, dtype=q.dtype)
            fmask = vals > 1e-10
            if forced_selection is not None:
                idx, fmask = forced_selection
            # differentiable top-k (NSA:715): the slots are scaled by 1 in the forward, the gradient of that scale
            # reaches the selected probabilities and through them the compressed logits
            slot_scale = vals + (1. - vals).detach() if self.use_diff_topk else None
            o_sel = ops.native_sparse_attend(qr, kr, v, sel, idx, fmask, sel_scale=slot_scale,
                                             include_block_causal=self.causal, impl=impl)
        else:
            o_sel = ops.block_diagonal_attend(qr, kr, v, sel, self.causal, impl=impl)

        # branch 3: sliding window; then the learned gates mix the three and merge heads
        o_swa = ops.sliding_window_attend(qr, kr, v, self.sliding_window_size, self.causal, impl=impl)
        gates = self.to_strategy_combine(x).view(b, n, h, 3).transpose(1, 2)
        merged = ops.gated_combine(o_cmp, o_sel, o_swa, gates)
        out = self.combine_heads(merged)

        if return_intermediates:
            return out, dict(q=q, k=k, v=v, ck=ck, cv=cv, qr=qr, kr=kr, importance=importance, vals=vals, idx=idx,
                             fmask=fmask, o_cmp=o_cmp, o_sel=o_sel, o_swa=o_swa, gates=gates, merged=merged)
        if not return_cache:
            return out
        return out, (cache_kv, cache_compressed)
