"""The tensor-core (tcgen05 / TMA) selected-block kernels, forced with impl='sm100', against the CPU
oracle at small sizes and against the fp32-accumulate generic kernels at a size with many chunks per
KV block.  bf16 tolerance: 2e-2 (+ bf16 spacing of the value)."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import SUM_REL, agreeing_queries, assert_bf16_no_worse_than_reference, assert_close_bf16, observe

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
    (1, 8, 1, 330, 128, 3),        # 8 heads per KV head at dim_head 128: the long-context grouping
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
        assert_close_bf16(g, r, w, rel_to_max=SUM_REL.get(w, 0.0))


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
        assert_close_bf16(g, r, w, rel_to_max=SUM_REL.get(w, 0.0))


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
        assert_close_bf16(g, r, w, rel_to_max=SUM_REL.get(w, 0.0))


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


# ---- the compressed and the sliding branch on the same tensor-core kernels ---------------------------------------

SWA_CASES = [
    # b, hq, hkv, n, d, window
    (2, 8, 2, 300, 64, 100),
    (1, 4, 1, 515, 64, 512),
    (1, 16, 1, 200, 128, 64),
    (1, 2, 2, 130, 64, 0),
    (1, 8, 1, 97, 64, 1000),
]


@pytest.mark.parametrize('case', SWA_CASES)
def test_sm100_sliding_matches_oracle(case):
    b, hq, hkv, n, d, win = case
    q = recipe.randn((b, hq, n, d), 1).bfloat16()
    k = recipe.randn((b, hkv, n, d), 2).bfloat16()
    v = recipe.randn((b, hkv, n, d), 3).bfloat16()
    up = recipe.randn((b, hq, n, d), 4).bfloat16()
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref = O.sliding_attend(qo, ko, vo, win, True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.sliding_window_attend(qg, kg, vg, win, True, impl='sm100')
    gd = torch.autograd.grad((out * up.to(DEV)).sum(), (qg, kg, vg))
    ops.check_device_status()
    for g, r, w in zip((out, *gd), (ref, *rd), ('out', 'dq', 'dk', 'dv')):
        assert_close_bf16(g, r, w, rel_to_max=SUM_REL.get(w, 0.0))


def check_importance(imp, q, ck, cv, mem, st, m, what='importance'):
    """The importance output against the oracle's own bf16 chain (bf16 tensors in: product, scaled logit and head mean
    are each rounded to bf16 as upstream's tensors are).  The tensor cores and the CPU add the 64 or 128 products of a
    logit in different orders, so a logit can land on the neighbouring bf16 value, at each of its two roundings; the
    mean over the heads then differs by at most two bf16 steps of the largest logit that entered it, plus its own
    rounding.  Everything else must be identical: the share of bit-identical entries is recorded."""
    b, hq, n, _ = q.shape
    hkv, ncb = ck.shape[1], ck.shape[2]
    _, csim16 = O.compressed_attend(q, ck, cv, mem[0], mem[1], st, True)
    assert csim16.dtype == torch.bfloat16
    per_head = csim16[..., m:].reshape(b, hkv, hq // hkv, n, ncb)
    ref16 = per_head.mean(dim=2).float()
    imp = imp.float().cpu()
    vis = ref16 > -1e30
    assert torch.equal(vis, imp > -1e30), what + ': visible columns'
    biggest = per_head.float().abs().amax(dim=2)
    allowed = 2 * 2.0 ** -7 * biggest + 2.0 ** -8 * ref16.abs() + 1e-6
    diff = (imp - ref16).abs()
    observe(what, identical_share=(imp == ref16)[vis].float().mean().item(), max_abs_err=diff[vis].max().item(),
            max_abs_ref=ref16[vis].abs().max().item(), worst_over_allowed=(diff[vis] / allowed[vis]).max().item())
    assert (diff[vis] <= allowed[vis]).all(), f'{what}: {(diff[vis] / allowed[vis]).max().item():.2f} x the allowed steps'
    assert torch.equal(imp[~vis], ref16[~vis]), what + ': sentinel of the invisible columns'


CMP_CASES = [
    # b, hq, hkv, n, d, stride, num_mem
    (2, 8, 2, 300, 64, 4, 1),
    (1, 4, 1, 1000, 64, 16, 2),
    (1, 8, 1, 260, 128, 2, 1),
    (1, 2, 2, 70, 64, 1, 1),
    (1, 4, 2, 200, 64, 4, 1),      # two heads per KV head
    (1, 16, 1, 130, 128, 2, 1),    # sixteen
]


@pytest.mark.parametrize('case', CMP_CASES)
def test_sm100_compressed_matches_oracle(case):
    b, hq, hkv, n, d, st, m = case
    ncb = n // st
    q = recipe.randn((b, hq, n, d), 1).bfloat16()
    ck = recipe.randn((b, hkv, ncb, d), 2).bfloat16()
    cv = recipe.randn((b, hkv, ncb, d), 3).bfloat16()
    mem = recipe.randn((2, hkv, m, d), 4).bfloat16()
    up = recipe.randn((b, hq, n, d), 5).bfloat16()
    qo, cko, cvo, memo = (t.float().requires_grad_() for t in (q, ck, cv, mem))
    ref, csim = O.compressed_attend(qo, cko, cvo, memo[0], memo[1], st, True)
    rd = torch.autograd.grad((ref * up.float()).sum(), (qo, cko, cvo, memo))
    qg, ckg, cvg, memg = (t.to(DEV).requires_grad_() for t in (q, ck, cv, mem))
    ckf = torch.cat((memg[0].expand(b, -1, -1, -1), ckg), dim=-2)
    cvf = torch.cat((memg[1].expand(b, -1, -1, -1), cvg), dim=-2)
    out, imp = nsa.compressed_attend(qg, ckf, cvf, m, st, True, impl='sm100')
    gd = torch.autograd.grad((out * up.to(DEV)).sum(), (qg, ckg, cvg, memg))
    ops.check_device_status()
    for g, r, w in zip((out, *gd), (ref, *rd), ('out', 'dq', 'dck', 'dcv', 'dmem')):
        # a compressed key (and above all a memory slot) collects gradient from every later query of every head:
        # allow 0.5 % of the largest value on those sums
        assert_close_bf16(g, r, w, rel_to_max=5e-3 if w in ('dck', 'dcv', 'dmem') else 0.0)
    check_importance(imp, q, ck, cv, mem, st, m)
    # the generic kernels write the same importance values (same rounding chain, other summation order)
    _, imp_simt = nsa.compressed_attend(qg, ckf, cvf, m, st, True, impl='simt')
    check_importance(imp_simt, q, ck, cv, mem, st, m, 'importance of the generic kernels')


POOL_CASES = [
    # b, hq, hkv, n, d, stride, num_mem, cpf, nsel
    (2, 8, 2, 1000, 64, 4, 1, 4, 6),       # selection block 16
    (1, 8, 1, 2077, 128, 16, 1, 4, 16),    # the long-context grouping: 8 heads per KV head, dim_head 128, block 64
    (1, 16, 4, 1500, 64, 16, 1, 4, 16),    # four heads per KV head (32 queries per tile)
    (1, 16, 1, 700, 64, 8, 2, 2, 5),       # sixteen; two memory slots; two columns per block
    (1, 8, 2, 900, 64, 16, 1, 1, 8),       # selection block = stride: no averaging, no own-block exclusion
    (1, 4, 1, 1300, 64, 4, 3, 8, 4),       # three memory slots, eight columns per block
]


@pytest.mark.parametrize('case', POOL_CASES)
def test_compressed_forward_pools_the_importance_per_selection_block(case):
    """With `pool` the compressed forward also does the per-block mean of the selection chain and hands a bf16 tensor
    of one value per selection block to the selection, instead of the fp32 matrix of every block column.  Wherever it
    is defined (the blocks before a query's own) it must hold, bit for bit, the mean the selection kernel would have
    formed from the full matrix, and the selection from it must be the same in every slot, masked ones included."""
    b, hq, hkv, n, d, st, m, cpf, nsel = case
    block = st * cpf
    ncb = (n - 2 * st) // st + 1
    q = recipe.randn((b, hq, n, d), 1).bfloat16().to(DEV)
    ck = recipe.randn((b, hkv, m + ncb, d), 2).bfloat16().to(DEV)
    cv = recipe.randn((b, hkv, m + ncb, d), 3).bfloat16().to(DEV)
    out0, imp = nsa.compressed_attend(q, ck, cv, m, st, True, impl='sm100')
    out1, pooled = nsa.compressed_attend(q, ck, cv, m, st, True, impl='sm100', pool=cpf)
    ops.check_device_status()
    assert imp.dtype == torch.float32 and pooled.dtype == torch.bfloat16
    cols = ncb // cpf
    assert pooled.shape == (b, hkv, n, cols)
    assert torch.equal(out0, out1)
    # the selection kernel's own averaging: the columns of a block added one after the other in fp32, divided, rounded
    x = imp[..., : cols * cpf].reshape(b, hkv, n, cols, cpf)
    acc = torch.zeros_like(x[..., 0])
    for c in range(cpf):
        acc = acc + x[..., c]
    want = (acc / float(cpf)).bfloat16() if cpf > 1 else x[..., 0].bfloat16()
    defined = torch.arange(cols, device=DEV)[None, :] < (torch.arange(n, device=DEV) // block)[:, None]
    assert defined.any()
    assert torch.equal(pooled[..., defined], want[..., defined])
    k = min(nsel, cols)
    vals0, idx0 = nsa.select_blocks(imp, block, st, k, dtype=torch.bfloat16)
    vals1, idx1 = nsa.select_blocks(pooled, block, st, k, dtype=torch.bfloat16)
    assert torch.equal(idx0, idx1) and torch.equal(vals0, vals1)
    assert (vals1 > 1e-10).any()
    observe(f'pooled selection {case}', identical_rows=float(torch.equal(idx0, idx1)),
            selected_share=(vals1 > 1e-10).float().mean().item())


def test_pooled_importance_is_refused_where_it_is_not_served():
    q = recipe.randn((1, 2, 200, 64), 1).bfloat16().to(DEV)         # two heads per KV head: the ring does not fit
    ck = recipe.randn((1, 1, 51, 64), 2).bfloat16().to(DEV)
    out, imp = nsa.compressed_attend(q, ck, ck, 1, 4, True, pool=4)
    assert imp.dtype == torch.float32                                # the operator falls back to the full matrix


@pytest.mark.parametrize('d', [64, 128])
def test_dense_forward_rescales_when_later_keys_dominate(d):
    # Keys grow with their position, so the running maximum of a row jumps by far more than 2^8 from one key block to
    # the next: the query-tile-stationary forward must rescale its accumulator (its lazy path), also for rows whose
    # first blocks hold nothing visible (sliding window) and for both halves of a 128-wide head.
    b, hq, hkv, n, win, st, m = 1, 8, 2, 700, 200, 2, 1
    q = recipe.randn((b, hq, n, d), 1).bfloat16()
    grow = (1.0 + 20.0 * (torch.arange(n) // 64).float() / (n // 64)).view(1, 1, n, 1)
    k = (recipe.randn((b, hkv, n, d), 2) * grow).bfloat16()
    v = recipe.randn((b, hkv, n, d), 3).bfloat16()
    ref = O.sliding_attend(q.float(), k.float(), v.float(), win, True)
    out = nsa.sliding_window_attend(q.to(DEV), k.to(DEV), v.to(DEV), win, True, impl='sm100')
    ops.check_device_status()
    assert_close_bf16(out, ref, 'sliding out')
    ncb = n // st
    growc = (1.0 + 20.0 * (torch.arange(ncb) // 64).float() / (ncb // 64)).view(1, 1, ncb, 1)
    ck = (recipe.randn((b, hkv, ncb, d), 4) * growc).bfloat16()
    cv = recipe.randn((b, hkv, ncb, d), 5).bfloat16()
    mem = recipe.randn((2, hkv, m, d), 6).bfloat16()
    ref, csim = O.compressed_attend(q.float(), ck.float(), cv.float(), mem[0].float(), mem[1].float(), st, True)
    ckf = torch.cat((mem[0].expand(b, -1, -1, -1), ck), dim=-2).to(DEV)
    cvf = torch.cat((mem[1].expand(b, -1, -1, -1), cv), dim=-2).to(DEV)
    out, imp = nsa.compressed_attend(q.to(DEV), ckf, cvf, m, st, True, impl='sm100')
    ops.check_device_status()
    assert_close_bf16(out, ref, 'compressed out')
    check_importance(imp, q, ck, cv, mem, st, m)


def test_sm100_layer_bf16_uses_tensor_core_branches():
    # a whole layer at a shape all three branches serve on tensor cores, against the fp32 oracle
    from native_sparse_attention_pytorch_b200 import SparseAttention
    kw = dict(dim=128, dim_head=64, heads=4, kv_heads=2, causal=True, sliding_window_size=70, compress_block_size=16,
              compress_block_sliding_stride=8, selection_block_size=64, num_selected_blocks=2)
    attn = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='sm100')
    recipe.fill_weights(attn, seed=7)
    attn = attn.to(DEV).bfloat16()
    ref = O.OracleSparseAttention(**kw)
    ref.load_state_dict({k_: v_.float().cpu() for k_, v_ in attn.state_dict().items()})
    x = recipe.randn((2, 300, 128), 11).bfloat16()
    out, mid = attn(x.to(DEV), return_intermediates=True)
    rout, rmid = ref(x.float(), return_intermediates=True)
    ops.check_device_status()
    # the oracle's own bf16 run on the fp32 run's blocks: the yardstick where values are too large for 2e-2
    ref16 = O.OracleSparseAttention(**kw)
    ref16.load_state_dict(ref.state_dict())
    out16, mid16 = ref16.bfloat16()(x, return_intermediates=True, forced_selection=(rmid['idx'], rmid['fmask']))
    assert_bf16_no_worse_than_reference(mid['o_cmp'], rmid['o_cmp'], mid16['o_cmp'], 'compressed branch')
    assert_bf16_no_worse_than_reference(mid['o_swa'], rmid['o_swa'], mid16['o_swa'], 'sliding branch')
    # the selection, then the selected branch and the output on the queries whose selection agrees
    assert torch.equal(mid['fmask'].sum(-1).cpu(), rmid['fmask'].sum(-1)), 'number of visible blocks per query'
    same = agreeing_queries(mid['idx'], mid['fmask'], rmid['idx'], rmid['fmask'])          # [B, Hkv, N]
    observe('selection agreement', share=same.float().mean().item())
    assert same.float().mean().item() > 0.5
    per_head = same.repeat_interleave(kw['heads'] // kw['kv_heads'], dim=1)
    assert_bf16_no_worse_than_reference(mid['o_sel'].cpu()[per_head], rmid['o_sel'][per_head], mid16['o_sel'][per_head],
                                        'selected branch')
    whole = same.all(dim=1)
    assert_bf16_no_worse_than_reference(out.cpu()[whole], rout[whole], out16[whole], 'out')


def test_full_benchmark_size_properties():
    """The kernel-level benchmark shape (batch 4, 8192 tokens, 32 / 4 heads, 16 selected blocks + own block) is far too
    large for the gather formulation of the oracle, so it is checked through what does not depend on size: the output
    of a sample of query rows against the oracle evaluated on those rows only, and three identities of the backward
    -- the rows of P sum to one, so  sum_keys dv = sum_(queries, heads) do ;  the rows of dS sum to zero and
    dq . q and dk . k both total scale * sum(dS * S), so  sum(dq * q) = sum(dk * k)  per KV head."""
    import bench
    w = bench.WORKLOADS[bench.DEFAULT_WORKLOAD]
    q, k, v, idx, mask, do = bench.make_inputs(w, seed=0)
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.native_sparse_attend(qg, kg, vg, w['block'], idx.to(DEV), mask.to(DEV), include_block_causal=True,
                                   impl='sm100')
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), do.to(DEV))
    ops.check_device_status()
    # sampled rows of batch element 1, KV head 2: first blocks, a block boundary, the middle, the end
    g = w['q_heads'] // w['kv_heads']
    rows = torch.tensor([0, 1, 63, 64, 65, 127, 128, 1000, 4095, 4096, 8000, 8190, 8191])
    hs = slice(2 * g, 3 * g)
    qs = q[1:2, hs].float().requires_grad_()
    ref = O.selected_attend(qs, k[1:2, 2:3].float(), v[1:2, 2:3].float(), w['block'], idx[1:2, 2:3],
                            mask[1:2, 2:3], True, rows=rows)
    assert_close_bf16(out[1:2, hs][:, :, rows.to(DEV)], ref, 'sampled output rows')
    (ref * do[1:2, hs][:, :, rows].float()).sum().backward()      # a query's dq depends on its own row only
    assert_close_bf16(dq[1:2, hs][:, :, rows.to(DEV)], qs.grad[:, :, rows], 'dq of the sampled rows')
    b, hkv, n, d = k.shape
    do_sum = do.float().view(b, hkv, g, n, d).sum(dim=(2, 3)).to(DEV)            # [B, Hkv, d]
    dv_sum = dv.float().sum(dim=2)
    assert (dv_sum - do_sum).abs().max().item() <= 2e-3 * do_sum.abs().max().item() + 0.5   # sums of 2.6e5 bf16 terms
    lhs = (dq.float() * qg.float()).view(b, hkv, g, n, d).sum(dim=(2, 3, 4))
    rhs = (dk.float() * kg.float()).sum(dim=(2, 3))
    scale_ref = (dq.float() * qg.float()).view(b, hkv, -1).abs().sum(dim=-1)
    assert ((lhs - rhs).abs() <= 2e-3 * scale_ref).all(), (lhs, rhs)


def test_many_single_chunk_items_keep_the_accumulator_handover_in_order():
    """A layer with fresh weights at the language-model shape: nearly every key block is selected by its own queries
    only, so the backward walks thousands of one-chunk items and hands its dK/dV accumulator over at every chunk.
    (This is the shape on which a flush once started one item early.)  Every run must end with a clean status and
    agree with the generic kernels."""
    from native_sparse_attention_pytorch_b200 import SparseAttention
    kw = dict(dim=512, dim_head=64, heads=8, kv_heads=4, causal=True, sliding_window_size=512, compress_block_size=32,
              compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=16)
    torch.manual_seed(0)
    fast = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='sm100').to(DEV).bfloat16()
    slow = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='simt').to(DEV).bfloat16()
    slow.load_state_dict(fast.state_dict())
    x = recipe.randn((4, 8192, 512), 3).bfloat16().to(DEV)
    up = recipe.randn((4, 8192, 512), 4).bfloat16().to(DEV)
    xs = x.clone().requires_grad_()
    slow(xs).backward(up)
    for _ in range(4):
        xf = x.clone().requires_grad_()
        out = fast(xf)
        out.backward(up)
        ops.check_device_status()
        assert_close_bf16(xf.grad, xs.grad, 'd input', rel_to_max=5e-3, roundings=2)


@pytest.mark.parametrize('case', [(2, 8, 2, 300, 64, 3), (1, 16, 1, 260, 128, 2), (1, 8, 1, 2000, 64, 6)])
def test_backward_with_the_forwards_index_equals_a_rebuilt_one(case, monkeypatch):
    # the backward normally takes the index (which queries attend which key block) the forward built; rebuilding it
    # from the same idx and mask must give the same gradients (dq exactly: its merge is ordered; dk, dv are sums of
    # fp32 atomics whose order may differ from launch to launch)
    b, hq, hkv, n, d, nsel = case
    q, k, v, idx, mask, up = make_case(b, hq, hkv, n, d, nsel, seed=21)
    assert ops.REUSE_INDEX
    kept = run_gpu(q, k, v, idx, mask, up, 'sm100', scale_grad=True)
    monkeypatch.setattr(ops, 'REUSE_INDEX', False)
    rebuilt = run_gpu(q, k, v, idx, mask, up, 'sm100', scale_grad=True)
    assert torch.equal(kept[0], rebuilt[0]) and torch.equal(kept[2], rebuilt[2])
    for a, r, what in zip(kept[3:], rebuilt[3:], ('dk', 'dv', 'dscale')):
        assert (a.float() - r.float()).abs().max().item() <= 1e-5 * max(1.0, r.float().abs().max().item()) + \
            2.0 ** -8 * r.float().abs().max().item() * (a.dtype == torch.bfloat16), what


def test_backward_refuses_an_index_that_was_not_built_for_it():
    # a kept index whose tag does not match (here: cleared) makes the kernels do nothing and report status 2;
    # no address is ever derived from it
    q, k, v, idx, mask, up = make_case(1, 8, 2, 300, 64, 3, seed=5)
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.native_sparse_attend(qg, kg, vg, BLOCK, idx.to(DEV), mask.to(DEV), impl='sm100')
    assert out.grad_fn.index is not None and out.grad_fn.index.numel() > 256
    out.grad_fn.index.zero_()
    torch.autograd.grad((out * up.to(DEV)).sum(), (qg, kg, vg))
    with pytest.raises(RuntimeError, match='index that was not built'):
        ops.check_device_status()


def test_gradients_come_back_in_the_layout_of_strided_inputs():
    # q, k, v as the layer makes them: [b, h, n, d] views of a [b, n, (heads d)] projection output.  Where the backward
    # stores whole rows of dq (tensor-core family, dim_head 64) dq is written directly in bf16 in q's layout, and the
    # inverse rotary writes in the layout of its input: the values equal those of contiguous inputs, and turning the
    # gradient back into [b, n, (h d)] needs no copy.
    from native_sparse_attention_pytorch_b200.rotary import RotaryEmbedding
    b, hq, hkv, n, d, nsel, win = 2, 8, 2, 300, 64, 3, 100
    _, _, _, idx, mask, up = make_case(b, hq, hkv, n, d, nsel, seed=31)
    proj = recipe.randn((b, n, (hq + 2 * hkv) * d), 32).bfloat16().to(DEV)
    split = lambda t: tuple(x.unflatten(-1, (-1, d)).transpose(1, 2) for x in t.split((hq * d, hkv * d, hkv * d), dim=-1))
    idx, mask, up = idx.to(DEV), mask.to(DEV), up.to(DEV)
    rot = RotaryEmbedding(d).to(DEV)

    def grads(strided):
        q, k, v = split(proj)
        if not strided:
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        q, k, v = (t.detach().requires_grad_() if not strided else t.requires_grad_() for t in (q, k, v))
        qr, kr = rot.rotate_queries_or_keys(q), rot.rotate_queries_or_keys(k)
        o1 = nsa.native_sparse_attend(qr, kr, v, BLOCK, idx, mask, impl='sm100')
        o2 = nsa.sliding_window_attend(qr, kr, v, win, True, impl='sm100')
        return torch.autograd.grad(((o1 + o2) * up).sum(), (q, k, v, qr))

    gs, gc = grads(True), grads(False)
    ops.check_device_status()
    for a, r, what in zip(gs, gc, ('dq', 'dk', 'dv', 'dq rotated')):
        assert a.dtype == torch.bfloat16 and a.shape == r.shape
        tol = 0.0 if what.startswith('dq') else 1e-5 + 2.0 ** -8      # dk, dv: fp32 atomics in any order, then one rounding
        assert (a.float() - r.float()).abs().max().item() <= tol * max(1.0, r.float().abs().max().item()), what
    assert gs[0].transpose(1, 2).is_contiguous() and gs[1].transpose(1, 2).is_contiguous()   # [b, n, h, d] in memory
    assert gs[3].is_contiguous() and gc[0].is_contiguous()


def test_sliding_and_compressed_backward_reuse_a_per_shape_index():
    # their index depends on the sizes only: the first backward of a shape builds it, later ones take the kept copy
    b, hq, hkv, n, d, win, st, m = 1, 8, 2, 700, 64, 130, 4, 1
    ops._shape_index.clear()
    q, k, v, up = (recipe.randn((b, h, n, d), s).bfloat16().to(DEV) for h, s in ((hq, 1), (hkv, 2), (hkv, 3), (hq, 4)))
    ck, cv = (recipe.randn((b, hkv, m + n // st, d), s).bfloat16().to(DEV) for s in (5, 6))

    def grads():
        qs, ks, vs, cks, cvs = (t.clone().requires_grad_() for t in (q, k, v, ck, cv))
        o1 = nsa.sliding_window_attend(qs, ks, vs, win, True, impl='sm100')
        o2, _ = nsa.compressed_attend(qs, cks, cvs, m, st, True, impl='sm100')
        return torch.autograd.grad(((o1 + o2) * up).sum(), (qs, ks, vs, cks, cvs))

    first = grads()
    assert len(ops._shape_index) == 2
    second = grads()
    ops.check_device_status()
    assert len(ops._shape_index) == 2
    assert torch.equal(first[0], second[0])                         # dq: ordered merge
    for a, r in zip(first[1:], second[1:]):                         # fp32 atomics in any order, then one rounding
        assert (a.float() - r.float()).abs().max().item() <= (1e-5 + 2.0 ** -8) * max(1.0, r.float().abs().max().item())


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """The library's self-test block waits, with a limit of about a millisecond, on a barrier nobody arrives on: it
    must return by itself, free its tensor memory and report status 1 -- the path every tensor-core kernel takes when
    a hand-over is lost.  Afterwards the same context runs a tensor-core kernel normally."""
    import ctypes as C
    from native_sparse_attention_pytorch_b200 import _lib as L
    lib = L.load()
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    L.check(lib.nsa_selftest_bounded_wait(status.data_ptr(), 2_000_000, stream))
    torch.cuda.synchronize()
    assert status.item() == 1
    assert lib.nsa_selftest_bounded_wait(status.data_ptr(), 0, stream) == -2          # the limit must be positive
    # the status travels through the module's accumulator like a real kernel's would, and surfaces at the next poll
    ws = torch.zeros(256, dtype=torch.uint8, device=DEV)
    ws[:4].view(torch.int32).copy_(status)
    ops.check_device_status()                               # clean so far
    ops._keep_status(ws)
    with pytest.raises(RuntimeError, match='bounded wait'):
        ops.check_device_status()
    ops._keep_status(ws)
    ops.poll_device_status(DEV)                             # starts the copy
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match='bounded wait'):
        ops.poll_device_status(DEV)                         # sees it, one call late, without synchronising
    ops.check_device_status()                               # and the accumulator is clean again
    q, k, v, idx, mask, up = make_case(1, 8, 2, 300, 64, 3, seed=3)
    run_gpu(q, k, v, idx, mask, up, 'sm100')                # tensor memory is free again: a real kernel runs


def test_launch_counter_counts_the_kernels_of_a_step():
    import ctypes as C
    from native_sparse_attention_pytorch_b200 import _lib as L
    lib = L.load()
    q, k, v, idx, mask, up = make_case(1, 8, 2, 300, 64, 3, seed=3)
    before = lib.nsa_launch_count()
    run_gpu(q, k, v, idx, mask, up, 'sm100')
    # forward: index pre-pass (4) + forward + merge; backward on the forward's index: delta + backward + dQ merge
    assert lib.nsa_launch_count() - before == 9


def test_forward_index_is_shared_between_calls_over_the_same_selection():
    """Runs of query heads of one KV head attend the same selected blocks: with an `index_cache` the second call takes
    the first call's index instead of building its own (four launches fewer) and computes the same."""
    from native_sparse_attention_pytorch_b200 import _lib as L
    lib = L.load()
    q, k, v, idx, mask, up = make_case(1, 8, 1, 700, 64, 4, seed=5)
    qa, qb = q[:, :4].to(DEV), q[:, 4:].to(DEV)
    kd, vd, idxd, maskd = k.to(DEV), v.to(DEV), idx.to(DEV), mask.to(DEV)
    alone = nsa.native_sparse_attend(qb, kd, vd, 64, idxd, maskd, impl='sm100')
    cache = {}
    n0 = lib.nsa_launch_count()
    nsa.native_sparse_attend(qa, kd, vd, 64, idxd, maskd, impl='sm100', index_cache=cache)
    n1 = lib.nsa_launch_count()
    shared = nsa.native_sparse_attend(qb, kd, vd, 64, idxd, maskd, impl='sm100', index_cache=cache)
    n2 = lib.nsa_launch_count()
    ops.check_device_status()
    assert len(cache) == 1 and (n1 - n0) - (n2 - n1) == 4
    assert torch.equal(shared, alone)
    # an index of another grouping is refused, not followed (its size differs: caught on the host; an index of the
    # right size built for other sizes fails the tag check on the device)
    q2 = q[:, :2].to(DEV)
    key = next(iter(cache))
    wrong = {(tuple(q2.shape),) + key[1:]: cache[key]}
    with pytest.raises(RuntimeError):
        nsa.native_sparse_attend(q2, kd, vd, 64, idxd, maskd, impl='sm100', index_cache=wrong)
        ops.check_device_status()
    ops.check_device_status()


@pytest.mark.parametrize('case', [(1, 8, 2, 700, 64, 4), (1, 8, 1, 600, 128, 3), (2, 4, 1, 333, 64, 2)])
def test_selected_forward_that_combines_and_stores_in_its_merge(case):
    """nsa_sel_fwd_combine_gather: the selected branch whose last kernel also does the gated combine, the head merge
    and the stores must write, byte for byte, what the selected operator followed by the combine writes -- here into
    two local buffers standing in for two ranks, at a feature offset."""
    b, hq, hkv, n, d, nsel = case
    q, k, v, idx, mask, _ = make_case(b, hq, hkv, n, d, nsel, seed=9)
    qd, kd, vd, idxd, maskd = (t.to(DEV) for t in (q, k, v, idx, mask))
    o_cmp = recipe.randn((b, hq, n, d), 31).bfloat16().to(DEV)
    o_swa = recipe.randn((b, hq, n, d), 32).bfloat16().to(DEV)
    gates = torch.sigmoid(recipe.randn((b, hq, n, 3), 33)).bfloat16().to(DEV)
    feats, off = hq * d + 2 * d, d
    want = [torch.zeros(b, n, feats, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    o_sel = nsa.native_sparse_attend(qd, kd, vd, 64, idxd, maskd, impl='sm100')
    ops.gated_combine_gather(o_cmp, o_sel, o_swa, gates, [w.data_ptr() for w in want], feats, off)
    got = [torch.zeros(b, n, feats, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    assert ops.selected_attend_combine_gather(qd, kd, vd, 64, idxd, maskd, o_cmp, o_swa, gates,
                                              [g.data_ptr() for g in got], feats, off, impl='sm100')
    ops.check_device_status()
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    assert got[0][..., :off].abs().max() == 0 and got[0][..., off + hq * d:].abs().max() == 0
    # shapes the tensor-core family does not serve are declined, nothing is written
    assert not ops.selected_attend_combine_gather(qd.float(), kd.float(), vd.float(), 64, idxd, maskd, o_cmp, o_swa, gates,
                                                  [got[0].data_ptr()], feats, off)


def test_combine_backward_hands_the_row_sums_to_the_branch_backwards(monkeypatch):
    """Every branch backward needs delta = sum_d out * d out per row; the gated combine's backward has it already as
    gate * d gate and hands it over through the gradient tensors, so the three branches skip their own pass: three
    launches fewer per layer step, gradients the same up to the rounding of d out (bf16) that the handed-over sums do
    not carry."""
    from native_sparse_attention_pytorch_b200 import SparseAttention, _lib as L
    kw = dict(dim=256, dim_head=64, heads=8, kv_heads=2, causal=True, sliding_window_size=128, compress_block_size=32,
              compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=4)
    attn = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='sm100')
    recipe.fill_weights(attn, seed=7)
    attn = attn.to(DEV).bfloat16()
    x = recipe.randn((2, 700, 256), 11).bfloat16().to(DEV)
    up = recipe.randn((2, 700, 256), 13).bfloat16().to(DEV)
    lib = L.load()

    def run(hand_over):
        monkeypatch.setattr(ops, 'HAND_OVER_DELTA', hand_over)
        attn.zero_grad(set_to_none=True)
        xs = x.clone().requires_grad_()
        out = attn(xs)
        before = lib.nsa_launch_count()
        out.backward(up)
        ops.check_device_status()
        return lib.nsa_launch_count() - before, xs.grad, attn.to_qkv.weight.grad.clone()

    run(False)                                              # the first backward also builds the per-shape indices
    n_own, dx_own, dw_own = run(False)
    n_handed, dx_handed, dw_handed = run(True)
    assert n_own - n_handed == 3, (n_own, n_handed)
    assert_close_bf16(dx_handed, dx_own, 'd input', roundings=2)
    assert_close_bf16(dw_handed, dw_own, 'd to_qkv.weight', roundings=2, rel_to_max=2e-3)


@pytest.mark.parametrize('cols,k', [(1100, 16), (300, 40), (200, 7)])
def test_selection_from_pooled_input_in_every_kernel_variant(cols, k):
    """The pooled bf16 input through the selection kernels the forward's shapes do not reach: rows of more than 1024
    block columns and more than 32 picks use the shared-memory variant, which must honour `pooled` and the causal limit
    as the register variant does.  Reference: the same values as an fp32 matrix with the columns at and past the own
    block set to the masked value by hand."""
    block = 4
    n = cols * block
    pooled = (recipe.randn((1, 2, n, cols), 3) * 3).bfloat16().to(DEV)
    full = pooled.float().clone()
    own = (torch.arange(n, device=DEV) // block)[:, None] <= torch.arange(cols, device=DEV)[None, :]
    full[..., own] = ops.mask_sentinel(torch.bfloat16)
    vals0, idx0 = nsa.select_blocks(full, block, block, k, dtype=torch.bfloat16)
    vals1, idx1 = nsa.select_blocks(pooled, block, block, k, dtype=torch.bfloat16)
    assert torch.equal(vals0, vals1)
    live = vals1 > 1e-10
    assert live.any() and torch.equal(idx0[live], idx1[live])
    # slots without a visible block: probability 0 in both; their column is the lowest zero column in both
    assert torch.equal(idx0, idx1)
