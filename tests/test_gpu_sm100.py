"""The tensor-core (tcgen05 / TMA) selected-block kernels, forced with impl='sm100', against the CPU
oracle at small sizes and against the fp32-accumulate generic kernels at a size with many chunks per
KV block.  bf16 tolerance: 2e-2 (+ bf16 spacing of the value)."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import assert_close_bf16

import native_sparse_attention_pytorch_b200 as nsa
from native_sparse_attention_pytorch_b200 import ops

pytestmark = pytest.mark.gpu
DEV = 'cuda'
BLOCK = 64


def make_case(b, hq, hkv, n, d, nsel, seed, strictly_past=True):
    nfb = -(-n // BLOCK)
    q = recipe.randn((b, hq, n, d), seed).bfloat16()
    k = recipe.randn((b, hkv, n, d), seed + 1).bfloat16()
    v = recipe.randn((b, hkv, n, d), seed + 2).bfloat16()
    idx = recipe.randint(0, nfb, (b, hkv, n, nsel), seed + 3)
    mask = recipe.randint(0, 4, (b, hkv, n, nsel), seed + 4) > 0
    if strictly_past:
        mask &= idx < (torch.arange(n) // BLOCK)[None, None, :, None]
    up = recipe.randn((b, hq, n, d), seed + 5).bfloat16()
    return q, k, v, idx, mask, up


def run_gpu(q, k, v, idx, mask, up, impl, causal=True, scale_grad=False):
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    sc = torch.ones(idx.shape, device=DEV, requires_grad=True) if scale_grad else None
    out, lse = nsa.native_sparse_attend(qg, kg, vg, BLOCK, idx.to(DEV), mask.to(DEV), sel_scale=sc,
                                        include_block_causal=causal, return_lse=True, impl=impl)
    ins = (qg, kg, vg) + ((sc,) if scale_grad else ())
    grads = torch.autograd.grad((out * up.to(DEV)).sum(), ins)
    ops.check_device_status()
    return (out, lse, *grads)


CASES = [
    # b, hq, hkv, n, d, nsel
    (2, 8, 2, 300, 64, 3),
    (1, 8, 1, 515, 64, 4),
    (1, 2, 2, 200, 64, 2),
    (1, 16, 1, 260, 128, 2),
    (2, 4, 2, 129, 128, 3),
    (1, 4, 2, 64, 64, 1),
    (1, 2, 1, 1, 64, 1),
]


@pytest.mark.parametrize('case', CASES)
def test_sm100_selected_matches_oracle(case):
    b, hq, hkv, n, d, nsel = case
    q, k, v, idx, mask, up = make_case(b, hq, hkv, n, d, nsel, seed=3)
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    so = torch.ones(idx.shape, requires_grad=True)
    ref, ref_lse = O.selected_attend(qo, ko, vo, BLOCK, idx, mask, True, gates=so, return_lse=True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo, so))
    got = run_gpu(q, k, v, idx, mask, up, 'sm100', scale_grad=True)
    for g, r, w in zip(got, (ref, ref_lse, *rd), ('out', 'lse', 'dq', 'dk', 'dv', 'dscale')):
        # the slot gradient sums 64*G products built from the bf16-stored output; allow 0.5 % of its largest value
        assert_close_bf16(g, r, w, rel_to_max=5e-3 if w == 'dscale' else 0.0)


def test_sm100_future_blocks_duplicates_and_the_partial_last_block():
    # indices may point anywhere (also at the ragged last block, whose missing keys count as zero keys)
    b, hq, hkv, n, d, nsel = 1, 8, 2, 200, 64, 3
    q, k, v, idx, mask, up = make_case(b, hq, hkv, n, d, nsel, seed=11, strictly_past=False)
    idx[..., 1] = idx[..., 0]          # the same block in two slots counts twice
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref = O.selected_attend(qo, ko, vo, BLOCK, idx, mask, True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo))
    out, _, dq, dk, dv = run_gpu(q, k, v, idx, mask, up, 'sm100')
    for g, r, w in zip((out, dq, dk, dv), (ref, *rd), ('out', 'dq', 'dk', 'dv')):
        assert_close_bf16(g, r, w)


@pytest.mark.parametrize('causal', [True, False])
def test_sm100_block_diagonal_fallback(causal):
    b, hq, hkv, n, d = 2, 8, 2, 150, 64
    q, k, v, _, _, up = make_case(b, hq, hkv, n, d, 1, seed=5)
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref = O.block_diagonal_attend(qo, ko, vo, BLOCK, causal)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.block_diagonal_attend(qg, kg, vg, BLOCK, causal, impl='sm100')
    gd = torch.autograd.grad((out * up.to(DEV)).sum(), (qg, kg, vg))
    ops.check_device_status()
    for g, r, w in zip((out, *gd), (ref, *rd), ('out', 'dq', 'dk', 'dv')):
        assert_close_bf16(g, r, w)


def test_sm100_many_chunks_per_block_matches_generic_kernels():
    # 4096 tokens, 16 of up to 63 past blocks per query: the early KV blocks collect thousands of queries
    b, hq, hkv, n, d, nsel = 1, 16, 2, 4096, 64, 16
    g = torch.Generator().manual_seed(0)
    q = torch.randn(b, hq, n, d, generator=g).bfloat16()
    k = torch.randn(b, hkv, n, d, generator=g).bfloat16()
    v = torch.randn(b, hkv, n, d, generator=g).bfloat16()
    up = torch.randn(b, hq, n, d, generator=g).bfloat16()
    nfb = n // BLOCK
    scores = torch.randn(b, hkv, n, nfb, generator=g)
    scores.masked_fill_(torch.arange(nfb)[None, :] >= (torch.arange(n) // BLOCK)[:, None], float('-inf'))
    vals, idx = scores.topk(nsel, dim=-1)
    mask = torch.isfinite(vals)
    idx = idx.masked_fill(~mask, 0)
    fast = run_gpu(q, k, v, idx, mask, up, 'sm100')
    slow = run_gpu(q, k, v, idx, mask, up, 'simt')
    for f, s, w in zip(fast, slow, ('out', 'lse', 'dq', 'dk', 'dv')):
        assert_close_bf16(f, s, w, roundings=2)
    rows = torch.cat((torch.arange(0, 130), torch.arange(2000, 2064), torch.arange(n - 64, n)))
    ref = O.selected_attend(q.float(), k.float(), v.float(), BLOCK, idx, mask, True, rows=rows)
    assert_close_bf16(fast[0][:, :, rows.to(DEV)], ref, 'out rows')


def test_sm100_refuses_shapes_it_does_not_serve():
    q, k, v, idx, mask, up = make_case(1, 4, 2, 100, 32, 2, seed=1)
    with pytest.raises(RuntimeError):
        nsa.native_sparse_attend(q.to(DEV), k.to(DEV), v.to(DEV), BLOCK, idx.to(DEV), mask.to(DEV), impl='sm100')
