"""bf16 parity of the composed path against the CPU oracle.

  * the block selection in bf16, rung by rung: (L0) the ranking kernel on the oracle's own bf16 probabilities,
    (L1) the whole reduction chain from the oracle's bf16 head-averaged logits, (L2) a whole layer, where the agreement
    of the selection is reported and everything after the selection is compared with the oracle's blocks forced;
  * the shapes of the baseline's configurations that the small cases of the other files do not reach: the full layer
    (16384 tokens, 16 / 4 heads) through sampled query rows, and a long-context head group (8 heads per KV head,
    dim_head 128).

Contract: selection values bit-identical wherever the softmax of the two implementations agrees in fp32 (a last-bit
difference of `exp` can move a probability across a bf16 rounding boundary: counted, reported and bounded below);
block indices identical wherever the k+1 largest probabilities of a row are distinct; floating-point tensors within
2e-2 (+ the bf16 spacing of the value).  Every comparison records the error it observed (tests/util.py:OBSERVED)."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import (SUM_REL, Checks, assert_bf16_no_worse_than_reference, assert_close_bf16, observe,
                  selection_agreement)

import native_sparse_attention_pytorch_b200 as nsa
from native_sparse_attention_pytorch_b200 import SparseAttention, ops

pytestmark = pytest.mark.gpu
DEV = 'cuda'


# ---------------------------------------------------------------------------------------------------- L0 / L1 ---

def synthetic_csim(g, ncb, n, seed, hkv=2):
    """bf16 logits [1, hkv*g, n, 1 + ncb] as the compressed branch returns them: one memory column, then the block
    columns; every row sees a random number of leading columns, the rest carry upstream's finite sentinel."""
    csim = (recipe.randn((1, hkv * g, n, 1 + ncb), seed) * 2.0).bfloat16()
    limit = recipe.randint(0, ncb + 1, (n,), seed + 1)
    limit[: min(n, 4)] = torch.tensor([0, 1, ncb, ncb // 2])[: min(n, 4)]
    hidden = torch.arange(ncb)[None, :] >= limit[:, None]
    sentinel = torch.tensor(-torch.finfo(torch.bfloat16).max // 10, dtype=torch.bfloat16)
    csim[..., 1:] = torch.where(hidden, sentinel, csim[..., 1:])
    return csim


LADDER = [
    # heads per KV head, stride, selection block, compressed columns, queries, blocks to pick
    (2, 64, 64, 256, 600, 16),      # stride == block: 256 block columns, no own-block fill
    (4, 16, 64, 1024, 600, 16),     # 4 compressed columns per block: 256 block columns (the full-layer shape)
    (8, 16, 64, 4096, 300, 16),     # 1024 block columns (the long-context shape), 8 heads per KV head
    (2, 64, 64, 1024, 300, 16),     # 1024 block columns without the per-block mean
    (4, 4, 8, 96, 200, 3),          # short rows
]


@pytest.mark.parametrize('case', LADDER)
def test_selection_ladder_bf16(case):
    g, st, sel, ncb, n, nsel = case
    hkv = 2
    csim = synthetic_csim(g, ncb, n, seed=50 + g)
    probs = O.importance_scores(csim, 1, hkv, st, sel, True)               # bf16, upstream's rounding chain
    assert probs.dtype == torch.bfloat16
    ref_vals, ref_idx = O.select_blocks(probs, nsel)
    k = ref_vals.shape[-1]
    top = probs.float().topk(min(k + 1, probs.shape[-1]), dim=-1).values
    boundary_unique = top[..., k - 1] > top[..., k] if probs.shape[-1] > k else torch.ones_like(top[..., 0], dtype=torch.bool)

    # (L0) the ranking kernel on the oracle's own probabilities
    vals0, idx0 = nsa.select_blocks(probs.float().to(DEV), sel, st, nsel, dtype=torch.bfloat16, input_is_prob=True)
    vals0, idx0 = vals0.cpu(), idx0.cpu()
    assert torch.equal(vals0, ref_vals), 'L0: the picked probabilities differ'
    assert torch.equal(vals0 > 1e-10, ref_vals > 1e-10)
    assert torch.equal(probs.gather(-1, idx0), vals0), 'L0: an index does not hold the value reported for it'
    m0, mr = vals0 > 1e-10, ref_vals > 1e-10
    rate0 = selection_agreement(idx0[boundary_unique], m0[boundary_unique], ref_idx[boundary_unique], mr[boundary_unique])
    observe('L0', rows=probs[..., 0].numel(), rows_with_distinct_boundary=boundary_unique.sum().item(), agreement=rate0)
    assert rate0 == 1.0, 'L0: different blocks although the k-th and (k+1)-th probabilities differ'

    # (L1) mean over the columns of a block, own-block fill, sink softmax, rounding, top-k -- from the bf16 head means
    imp = csim[..., 1:].reshape(1, hkv, g, n, ncb).mean(dim=2)
    assert imp.dtype == torch.bfloat16
    vals1, idx1 = nsa.select_blocks(imp.float().to(DEV), sel, st, nsel, dtype=torch.bfloat16)
    vals1, idx1 = vals1.cpu(), idx1.cpu()
    # the same chain evaluated by PyTorch on the GPU: tells a difference of the kernel from a difference between
    # PyTorch's CPU and CUDA softmax
    probs_cuda = O.importance_scores(csim.to(DEV), 1, hkv, st, sel, True)
    cuda_vals, _ = O.select_blocks(probs_cuda, nsel)
    cuda_vals = cuda_vals.cpu()

    def mismatch(a, b):
        bad = a != b
        ulp = (a.float() - b.float()).abs() / torch.clamp(torch.maximum(a.float().abs(), b.float().abs()), min=1e-30)
        return bad.sum().item(), bad.any(dim=-1).sum().item(), (ulp[bad].max().item() if bad.any() else 0.0)

    cnt_cpu, rows_cpu, rel_cpu = mismatch(vals1, ref_vals)
    cnt_cuda, rows_cuda, rel_cuda = mismatch(vals1, cuda_vals)
    cnt_tt, rows_tt, rel_tt = mismatch(cuda_vals, ref_vals)
    rows = vals1[..., 0].numel()
    observe('L1 values', rows=rows, picked=vals1.numel(), kernel_vs_torch_cpu=cnt_cpu, kernel_vs_torch_cuda=cnt_cuda,
            torch_cuda_vs_torch_cpu=cnt_tt, rows_kernel_vs_torch_cpu=rows_cpu, rows_kernel_vs_torch_cuda=rows_cuda,
            max_rel_diff_vs_cpu=rel_cpu, max_rel_diff_vs_cuda=rel_cuda)
    print(f'L1 {case}: {cnt_cpu} of {vals1.numel()} picked probabilities differ from PyTorch-CPU, {cnt_cuda} from '
          f'PyTorch-CUDA (PyTorch CPU vs CUDA: {cnt_tt})')
    # a differing value is one bf16 step away (2^-8 relative at most), and rare
    assert max(rel_cpu, rel_cuda) <= 2.0 ** -7
    assert rows_cpu <= max(2, rows // 100), f'L1: {rows_cpu} of {rows} rows differ from the CPU chain'
    assert torch.equal(vals1 > 1e-10, ref_vals > 1e-10)
    # where the values agree and the boundary is distinct, the blocks are the reference's
    ok = (vals1 == ref_vals).all(dim=-1) & boundary_unique
    m1 = vals1 > 1e-10
    rate1 = selection_agreement(idx1[ok], m1[ok], ref_idx[ok], mr[ok])
    observe('L1 blocks', rows_compared=ok.sum().item(), agreement=rate1,
            agreement_all_rows=selection_agreement(idx1, m1, ref_idx, mr))
    assert ok.float().mean().item() > 0.5
    assert rate1 == 1.0


# ----------------------------------------------------------------------------------------------------- L2 ---

L2_KW = dict(dim=256, dim_head=64, heads=8, kv_heads=2, causal=True, sliding_window_size=128, compress_block_size=32,
             compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=8)


def test_layer_bf16_with_the_oracles_selection_forced():
    """A layer that selects blocks, on the tensor-core kernels (block 64, 4 heads per KV head): the selection is
    compared with the oracle's (agreement reported against the oracle run in fp32 and in bf16); then the oracle's
    fp32 selection is forced on the kernels and every tensor after it is compared: selected branch, merged output,
    the gradients at the boundary of the hot path, the input gradient, and the parameter gradients through their
    error against the fp32 oracle, which must not exceed that of the oracle itself run in bf16 on the same blocks."""
    b, n = 1, 1024
    attn = SparseAttention(**L2_KW, use_triton_kernel=True, kernel_impl='sm100')
    recipe.fill_weights(attn, seed=7)
    attn = attn.to(DEV).bfloat16()
    weights = {k: v.float().cpu() for k, v in attn.state_dict().items()}
    ref = O.OracleSparseAttention(**L2_KW)
    ref.load_state_dict(weights)
    ref16 = O.OracleSparseAttention(**L2_KW)
    ref16.load_state_dict(weights)
    ref16 = ref16.bfloat16()
    x = recipe.randn((b, n, L2_KW['dim']), 11).bfloat16()
    up = recipe.randn((b, n, L2_KW['dim']), 13).bfloat16()
    boundary = ('q', 'k', 'v', 'ck', 'cv', 'gates', 'o_sel')

    # fp32 oracle with its own selection: the truth
    xr = x.float().requires_grad_()
    rout, rmid = ref(xr, return_intermediates=True)
    for key in boundary:
        rmid[key].retain_grad()
    (rout * up.float()).sum().backward()
    forced = (rmid['idx'], rmid['fmask'])

    # the kernels' own selection, and the bf16 oracle's, against it
    with torch.no_grad():
        _, mid_free = attn(x.to(DEV), return_intermediates=True)
        _, mid16_free = ref16(x, return_intermediates=True)
    ops.check_device_status()
    agree_fp32 = selection_agreement(mid_free['idx'], mid_free['fmask'], *forced)
    agree_bf16 = selection_agreement(mid_free['idx'], mid_free['fmask'], mid16_free['idx'], mid16_free['fmask'])
    oracle_self = selection_agreement(mid16_free['idx'], mid16_free['fmask'], *forced)
    observe('L2 selection agreement (share of queries with identical block sets)', kernels_vs_oracle_fp32=agree_fp32,
            kernels_vs_oracle_bf16=agree_bf16, oracle_bf16_vs_oracle_fp32=oracle_self)
    print(f'L2 selection: kernels vs fp32 oracle {agree_fp32:.4f}, vs bf16 oracle {agree_bf16:.4f}; '
          f'bf16 oracle vs fp32 oracle {oracle_self:.4f}')
    assert torch.equal(mid_free['fmask'].sum(-1).cpu(), forced[1].sum(-1)), 'number of visible blocks per query'
    assert agree_fp32 >= oracle_self - 0.05      # no further from the truth than upstream's own bf16 run is

    # everything after the selection, on the same blocks
    xg = x.to(DEV).requires_grad_()
    out, mid = attn(xg, return_intermediates=True, forced_selection=(forced[0].to(DEV), forced[1].to(DEV)))
    for key in boundary:
        mid[key].retain_grad()
    (out * up.to(DEV)).sum().backward()
    ops.check_device_status()
    x16 = x.clone().requires_grad_()
    out16, mid16 = ref16(x16, return_intermediates=True, forced_selection=forced)
    for key in boundary:
        mid16[key].retain_grad()
    (out16 * up).sum().backward()

    # The kernels see bf16 q, k, v, gates where the fp32 oracle sees unrounded ones, so every tensor is held to the
    # bf16 contract against the fp32 oracle or, failing that, to the error of the oracle's own bf16 run (same weights,
    # same blocks).
    check = Checks()
    for key in ('o_cmp', 'o_swa', 'o_sel', 'merged'):
        check(assert_bf16_no_worse_than_reference, mid[key], rmid[key], mid16[key], key)
    check(assert_bf16_no_worse_than_reference, out, rout, out16, 'out')
    for key in boundary:
        check(assert_bf16_no_worse_than_reference, mid[key].grad, rmid[key].grad, mid16[key].grad, 'd ' + key,
              rel_to_max=SUM_REL['dk'] if key in ('k', 'v', 'ck', 'cv') else 0.0)
    check(assert_bf16_no_worse_than_reference, xg.grad, xr.grad, x16.grad, 'd inp')
    ours, theirs = dict(attn.named_parameters()), dict(ref16.named_parameters())

    def param_grad(name, truth):
        e_ours = (ours[name].grad.float().cpu() - truth).abs().max().item()
        e_ref = (theirs[name].grad.float() - truth).abs().max().item()
        spacing = 2.0 ** -8 * truth.abs().max().item()       # both results are stored in bf16
        observe('d ' + name, err_kernels_vs_fp32=e_ours, err_oracle_bf16_vs_fp32=e_ref, max_abs=truth.abs().max().item())
        assert e_ours <= 1.5 * e_ref + spacing, (name, e_ours, e_ref)

    for name, p in ref.named_parameters():
        if p.grad is not None:
            check(param_grad, name, p.grad)
    check.done()


# ----------------------------------------------------------------------------- baseline shapes, sampled rows ---

def test_selected_gradients_at_the_benchmark_grouping():
    """8 query heads per KV head, 16 selected blocks + the own block (the grouping of the kernel benchmark), at a
    length the oracle's gather formulation fits: out, lse, dq, dk, dv element by element."""
    b, hq, hkv, n, d, nsel, blk = 1, 8, 1, 2048, 64, 16, 64
    gen = torch.Generator().manual_seed(5)
    q, up = (torch.randn(b, hq, n, d, generator=gen).bfloat16() for _ in range(2))
    k, v = (torch.randn(b, hkv, n, d, generator=gen).bfloat16() for _ in range(2))
    nfb = n // blk
    scores = torch.randn(b, hkv, n, nfb, generator=gen)
    scores.masked_fill_(torch.arange(nfb)[None, :] >= (torch.arange(n) // blk)[:, None], float('-inf'))
    vals, idx = scores.topk(nsel, dim=-1)
    mask = torch.isfinite(vals)
    idx = idx.masked_fill(~mask, 0)
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref, ref_lse = O.selected_attend(qo, ko, vo, blk, idx, mask, True, return_lse=True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out, lse = nsa.native_sparse_attend(qg, kg, vg, blk, idx.to(DEV), mask.to(DEV), return_lse=True, impl='sm100')
    gd = torch.autograd.grad((out * up.to(DEV)).sum(), (qg, kg, vg))
    ops.check_device_status()
    for got, want, what in zip((out, lse, *gd), (ref, ref_lse, *rd), ('out', 'lse', 'dq', 'dk', 'dv')):
        assert_close_bf16(got, want, what, rel_to_max=SUM_REL.get(what, 0.0))


def test_full_layer_shape_sampled_rows():
    """The full-layer configuration (batch 2, 16384 tokens, dim 1024, 16 / 4 heads, stride 16, block 64, 16 blocks,
    window 512, bf16) through the module.  The oracle cannot hold this shape, so one (batch, KV head) slice is checked
    on a sample of query rows: each branch against the oracle evaluated on the kernels' own inputs for those rows, the
    selection against the oracle's selection from its own logits (agreement reported), the merged rows."""
    kw = dict(dim=1024, dim_head=64, heads=16, kv_heads=4, sliding_window_size=512, compress_block_size=32,
              compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=16, causal=True)
    torch.manual_seed(0)
    attn = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='sm100').to(DEV).bfloat16()
    with torch.no_grad():
        attn.compress_mem_kv.copy_(recipe.randn(attn.compress_mem_kv.shape, 3, 0.5))
    bsz, n, g, st, blk = 2, 16384, 4, 16, 64
    x = recipe.randn((bsz, n, kw['dim']), 21).bfloat16().to(DEV)
    with torch.no_grad():
        _, mid = attn(x, return_intermediates=True)
    ops.check_device_status()
    bi, h = 1, 2
    hs = slice(h * g, (h + 1) * g)
    rows = torch.cat((torch.arange(0, 70), torch.arange(1000, 1030), torch.arange(8190, 8200),
                      torch.arange(n - 40, n)))
    cut = lambda key, heads: mid[key][bi:bi + 1, heads].float().cpu()
    q, qr, gates = cut('q', hs), cut('qr', hs), cut('gates', hs)
    kr, v, ck, cv = (cut(key, slice(h, h + 1)) for key in ('kr', 'v', 'ck', 'cv'))
    mem = attn.compress_mem_kv.detach().float().cpu()[:, h:h + 1]
    rows_dev = rows.to(DEV)
    got = lambda key: mid[key][bi:bi + 1, hs][:, :, rows_dev]

    o_cmp, csim = O.compressed_attend(q, ck, cv, mem[0], mem[1], st, True, rows=rows)
    assert_close_bf16(got('o_cmp'), o_cmp, 'compressed branch')
    idx, fmask = mid['idx'][bi:bi + 1, h:h + 1][:, :, rows_dev].cpu(), mid['fmask'][bi:bi + 1, h:h + 1][:, :, rows_dev].cpu()
    for dtype, label in ((torch.float32, 'fp32'), (torch.bfloat16, 'bf16')):
        c = csim if dtype == torch.float32 else O.compressed_attend(q.bfloat16(), ck.bfloat16(), cv.bfloat16(), mem[0].bfloat16(),
                                                                    mem[1].bfloat16(), st, True, rows=rows)[1]
        probs = O.importance_scores(c, 1, 1, st, blk, True, rows=rows)
        rv, ri = O.select_blocks(probs, 16)
        # identical block sets, and -- probabilities tie often with fresh weights -- picks that are a top-16 of the
        # oracle's probabilities (the same multiset of values) whichever of the tied blocks were taken
        mine = probs.gather(-1, idx).float().sort(dim=-1).values
        observe('selection agreement on the sampled rows, oracle in ' + label,
                share=selection_agreement(idx, fmask, ri, rv > 1e-10),
                share_valid_top16=(mine == rv.float().sort(dim=-1).values).all(dim=-1).float().mean().item())
        assert torch.equal(fmask.sum(-1), (rv > 1e-10).sum(-1)), 'number of visible blocks per query'
    o_sel = _selected_rows(qr, kr, v, blk, idx, fmask, rows)
    assert_close_bf16(got('o_sel'), o_sel, 'selected branch')
    o_swa = O.sliding_attend(qr, kr, v, kw['sliding_window_size'], True, rows=rows)
    assert_close_bf16(got('o_swa'), o_swa, 'sliding branch')
    merged = O.combine(o_cmp, o_sel, o_swa, gates[:, :, rows])
    d = kw['dim_head']
    assert_close_bf16(mid['merged'][bi:bi + 1, rows_dev][..., h * g * d:(h + 1) * g * d], merged, 'merged rows')


def _selected_rows(qr, kr, v, blk, idx_rows, mask_rows, rows):
    """The oracle's selected-block attention for the query positions `rows`, given the selection of those rows only."""
    n = qr.shape[2]
    idx = torch.zeros(*idx_rows.shape[:2], n, idx_rows.shape[-1], dtype=idx_rows.dtype)
    mask = torch.zeros(*mask_rows.shape[:2], n, mask_rows.shape[-1], dtype=torch.bool)
    idx[:, :, rows], mask[:, :, rows] = idx_rows, mask_rows
    return O.selected_attend(qr, kr, v, blk, idx, mask, True, rows=rows)


@pytest.mark.parametrize('case', [(1, 8, 1, 260, 128, 2), (1, 8, 1, 1500, 128, 16)])
def test_long_context_head_group_selected_branch(case):
    """8 query heads per KV head at dim_head 128 (the grouping of the long-context configuration): forward and
    backward of the selected branch against the oracle."""
    b, hq, hkv, n, d, nsel = case
    blk = 64
    nfb = -(-n // blk)
    q, up = (recipe.randn((b, hq, n, d), s).bfloat16() for s in (1, 2))
    k, v = (recipe.randn((b, hkv, n, d), s).bfloat16() for s in (3, 4))
    scores = recipe.randn((b, hkv, n, nfb), 5)
    scores.masked_fill_(torch.arange(nfb)[None, :] >= (torch.arange(n) // blk)[:, None], float('-inf'))
    vals, idx = scores.topk(min(nsel, nfb), dim=-1)
    mask = torch.isfinite(vals)
    idx = idx.masked_fill(~mask, 0)
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref = O.selected_attend(qo, ko, vo, blk, idx, mask, True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.native_sparse_attend(qg, kg, vg, blk, idx.to(DEV), mask.to(DEV), impl='sm100')
    gd = torch.autograd.grad((out * up.to(DEV)).sum(), (qg, kg, vg))
    ops.check_device_status()
    for got, want, what in zip((out, *gd), (ref, *rd), ('out', 'dq', 'dk', 'dv')):
        assert_close_bf16(got, want, what, rel_to_max=SUM_REL.get(what, 0.0))
