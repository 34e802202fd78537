"""GPU parity of every operator against the CPU oracle and the stored upstream
vectors.  All calls go through the C ABI (ctypes).  Tolerances: fp32 1e-4
relative, bf16 2e-2 max-abs, integer outputs exact."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import assert_close_bf16, assert_close_f32, load_golden, same_selection

import native_sparse_attention_pytorch_b200 as nsa
from native_sparse_attention_pytorch_b200 import _lib as nsa_lib

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def grads_of(out, upstream, inputs):
    gs = torch.autograd.grad((out * upstream).sum(), inputs, allow_unused=True)
    return gs


def closeness(dtype):
    return assert_close_f32 if dtype == torch.float32 else assert_close_bf16


# ---------------------------------------------------------------- selected ---

@pytest.mark.parametrize('impl', ['simt', 'auto'])
@pytest.mark.parametrize('name', list(recipe.OP_CASES))
def test_selected_matches_upstream_vectors(name, impl):
    c = recipe.OP_CASES[name]
    gold = load_golden(name)
    q, k, v, idx, mask = (t.to(DEV) for t in recipe.op_inputs(name))
    scale = torch.ones(idx.shape, device=DEV)
    q, k, v, scale = (t.requires_grad_() for t in (q, k, v, scale))
    out, lse = nsa.native_sparse_attend(q, k, v, c['block'], idx, mask, sel_scale=scale, return_lse=True, impl=impl)
    up = recipe.randn(out.shape, 29).to(DEV)
    dq, dk, dv, dscale = grads_of(out, up, (q, k, v, scale))
    assert_close_f32(out, gold['out'], 'out')
    assert_close_f32(lse, gold['lse'], 'lse')
    assert_close_f32(dq, gold['dq'], 'dq')
    assert_close_f32(dk, gold['dk'], 'dk')
    assert_close_f32(dv, gold['dv'], 'dv')
    assert_close_f32(dscale, gold['dscale'], 'dscale')


SEL_CASES = [
    # b, hq, hkv, hs, n, d, block, nsel, causal, future_blocks
    (2, 4, 2, 2, 75, 32, 8, 3, True, False),
    (1, 8, 1, 1, 130, 64, 16, 4, True, False),
    (2, 4, 4, 4, 31, 64, 4, 2, False, True),     # README-like: one head per group, non-causal
    (1, 4, 2, 4, 50, 16, 8, 2, True, False),     # per-query-head selection
    (1, 16, 1, 1, 40, 128, 8, 2, True, False),   # 16 heads in a group, widest head
    (2, 2, 2, 2, 37, 24, 5, 2, False, True),     # odd block size, dim not a power of two
]


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('case', SEL_CASES)
def test_selected_matches_oracle(case, dtype):
    b, hq, hkv, hs, n, d, block, nsel, causal, future = case
    nfb = -(-n // block)
    q = recipe.randn((b, hq, n, d), 1).to(dtype)
    k = recipe.randn((b, hkv, n, d), 2).to(dtype)
    v = recipe.randn((b, hkv, n, d), 3).to(dtype)
    idx = recipe.randint(0, nfb, (b, hs, n, nsel), 4)
    mask = recipe.randint(0, 3, (b, hs, n, nsel), 5) > 0
    if causal and not future:
        own = (torch.arange(n) // block)[None, None, :, None]
        mask &= idx < own
    up = recipe.randn((b, hq, n, d), 6).to(dtype)

    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref, ref_lse = O.selected_attend(qo, ko, vo, block, idx, mask, causal, return_lse=True)
    rdq, rdk, rdv = grads_of(ref, up.float(), (qo, ko, vo))

    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out, lse = nsa.native_sparse_attend(qg, kg, vg, block, idx.to(DEV), mask.to(DEV), include_block_causal=causal,
                                        return_lse=True)
    dq, dk, dv = grads_of(out, up.to(DEV), (qg, kg, vg))
    close = closeness(dtype)
    close(out, ref, 'out')
    visible = torch.isfinite(lse.cpu()) & (ref_lse > -1e30)
    close(torch.where(visible, lse.cpu(), 0), torch.where(visible, ref_lse, 0), 'lse')
    close(dq, rdq, 'dq')
    close(dk, rdk, 'dk')
    close(dv, rdv, 'dv')


def test_selected_rows_without_any_visible_key_average_their_slots():
    # non-causal, every slot masked: upstream's finite fill turns the softmax into a plain mean
    b, h, n, d, block = 1, 2, 16, 16, 4
    q, k, v = (recipe.randn((b, h, n, d), s) for s in (1, 2, 3))
    idx = recipe.randint(0, 4, (b, h, n, 2), 4)
    mask = torch.zeros(b, h, n, 2, dtype=torch.bool)
    mask[:, :, ::2, 0] = True
    qo, ko, vo = (t.clone().requires_grad_() for t in (q, k, v))
    ref = O.selected_attend(qo, ko, vo, block, idx, mask, causal=False)
    up = recipe.randn(ref.shape, 9)
    rd = grads_of(ref, up, (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.native_sparse_attend(qg, kg, vg, block, idx.to(DEV), mask.to(DEV), include_block_causal=False)
    gd = grads_of(out, up.to(DEV), (qg, kg, vg))
    assert_close_f32(out, ref, 'out')
    for g, r, w in zip(gd, rd, ('dq', 'dk', 'dv')):
        assert_close_f32(g, r, w)


@pytest.mark.parametrize('causal', [True, False])
def test_block_diagonal_fallback(causal):
    b, hq, hkv, n, d, block = 2, 4, 2, 29, 32, 8
    q = recipe.randn((b, hq, n, d), 1)
    k = recipe.randn((b, hkv, n, d), 2)
    v = recipe.randn((b, hkv, n, d), 3)
    qo, ko, vo = (t.clone().requires_grad_() for t in (q, k, v))
    ref = O.block_diagonal_attend(qo, ko, vo, block, causal)
    up = recipe.randn(ref.shape, 7)
    rd = grads_of(ref, up, (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.block_diagonal_attend(qg, kg, vg, block, causal)
    gd = grads_of(out, up.to(DEV), (qg, kg, vg))
    assert_close_f32(out, ref, 'out')
    for g, r, w in zip(gd, rd, ('dq', 'dk', 'dv')):
        assert_close_f32(g, r, w)


def test_selected_accepts_strided_views_of_a_fused_projection():
    b, n, hq, hkv, d, block = 2, 40, 4, 2, 32, 8
    fused = recipe.randn((b, n, (hq + 2 * hkv) * d), 1).to(DEV)
    q, k, v = fused.split((hq * d, hkv * d, hkv * d), dim=-1)
    q, k, v = (t.view(b, n, -1, d).transpose(1, 2) for t in (q, k, v))
    idx = recipe.randint(0, 5, (b, hkv, n, 2), 2).to(DEV)
    mask = idx < (torch.arange(n, device=DEV) // block)[None, None, :, None]
    out = nsa.native_sparse_attend(q, k, v, block, idx, mask)
    ref = O.selected_attend(q.cpu(), k.cpu(), v.cpu(), block, idx.cpu(), mask.cpu(), True)
    assert_close_f32(out, ref, 'out')


# -------------------------------------------------------------- compressed ---

CMP_CASES = [
    # b, hq, hkv, n, d, stride, num_mem, causal, share
    (2, 4, 2, 61, 32, 4, 1, True, True),
    (1, 8, 1, 100, 64, 2, 2, True, True),
    (2, 4, 4, 31, 64, 2, 1, False, True),
    (1, 4, 2, 50, 16, 4, 1, True, False),
]


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('case', CMP_CASES)
def test_compressed_matches_oracle(case, dtype):
    b, hq, hkv, n, d, st, m, causal, share = case
    ncb = n // st
    q = recipe.randn((b, hq, n, d), 1).to(dtype)
    ck = recipe.randn((b, hkv, ncb, d), 2).to(dtype)
    cv = recipe.randn((b, hkv, ncb, d), 3).to(dtype)
    mem = recipe.randn((2, hkv, m, d), 4).to(dtype)
    up = recipe.randn((b, hq, n, d), 5).to(dtype)

    qo, cko, cvo, memo = (t.float().requires_grad_() for t in (q, ck, cv, mem))
    ref, csim = O.compressed_attend(qo, cko, cvo, memo[0], memo[1], st, causal)
    rdq, rdck, rdcv, rdmem = grads_of(ref, up.float(), (qo, cko, cvo, memo))

    qg, ckg, cvg, memg = (t.to(DEV).requires_grad_() for t in (q, ck, cv, mem))
    ckf = torch.cat((memg[0].expand(b, -1, -1, -1), ckg), dim=-2)
    cvf = torch.cat((memg[1].expand(b, -1, -1, -1), cvg), dim=-2)
    out, imp = nsa.compressed_attend(qg, ckf, cvf, m, st, causal, sel_heads=hkv if share else hq)
    dq, dck, dcv, dmem = grads_of(out, up.to(DEV), (qg, ckg, cvg, memg))
    close = closeness(dtype)
    close(out, ref, 'out')
    close(dq, rdq, 'dq')
    # a compressed key (above all a memory slot) collects gradient from every later query of every head; in bf16
    # allow 0.5 % of the largest value on those sums
    wide = dict(rel_to_max=5e-3) if dtype == torch.bfloat16 else {}
    close(dck, rdck, 'dck', **wide)
    close(dcv, rdcv, 'dcv', **wide)
    close(dmem, rdmem, 'dmem', **wide)
    # importance = head-mean of the block logits, the sentinel where invisible
    ref_imp = csim[..., m:]
    if share:
        ref_imp = ref_imp.reshape(b, hkv, hq // hkv, n, ncb).mean(dim=2)
    vis = ref_imp > -1e30
    assert torch.equal(vis, imp.cpu() > -1e30)
    close(torch.where(vis, imp.cpu(), 0), torch.where(vis, ref_imp, 0), 'importance')
    if dtype == torch.float32:
        assert torch.equal(imp.cpu()[~vis], ref_imp[~vis])      # sentinel values are bit-identical


# --------------------------------------------------------------- selection ---

@pytest.mark.parametrize('st,sel,nsel', [(4, 8, 2), (2, 8, 3), (4, 4, 2), (4, 16, 16), (2, 10, 2)])
@pytest.mark.parametrize('causal', [True, False])
def test_selection_is_bit_exact_given_the_scores(st, sel, nsel, causal):
    b, hq, hkv, n, d = 2, 4, 2, 97, 16
    ncb = n // st
    q = recipe.randn((b, hq, n, d), 1)
    ck = recipe.randn((b, hkv, ncb, d), 2)
    cv = recipe.randn((b, hkv, ncb, d), 3)
    mem = recipe.randn((2, hkv, 1, d), 4)
    _, csim = O.compressed_attend(q, ck, cv, mem[0], mem[1], st, causal)
    probs = O.importance_scores(csim, 1, hkv, st, sel, True)
    ref_vals, ref_idx = O.select_blocks(probs, nsel)

    # (L0) ranking kernel on the oracle's own probabilities: identical indices wherever the value is unique
    vals0, idx0 = nsa.select_blocks(probs.to(DEV), sel, st, nsel, input_is_prob=True)
    assert torch.equal(vals0.cpu(), ref_vals)
    assert same_selection(idx0, vals0 > 1e-10, ref_idx, ref_vals > 1e-10)
    k = ref_vals.shape[-1]
    if probs.shape[-1] > k:   # rows whose k+1 largest values are all different have one valid answer
        top = probs.topk(k + 1, dim=-1).values
        unique = (top[..., :-1] > top[..., 1:]).all(dim=-1)
        assert unique.any()
        assert torch.equal(idx0.cpu()[unique], ref_idx[unique])

    # (L1) the whole chain from head-averaged logits: mean over cpf, own-block fill, sink softmax, top-k
    imp = csim[..., 1:].reshape(b, hkv, hq // hkv, n, ncb).mean(dim=2)
    vals1, idx1 = nsa.select_blocks(imp.to(DEV), sel, st, nsel)
    assert_close_f32(vals1, ref_vals, 'values', tol=1e-6)
    assert same_selection(idx1, vals1 > 1e-10, ref_idx, ref_vals > 1e-10)


def test_selection_breaks_ties_towards_the_lower_index():
    p = torch.tensor([0.1, 0.4, 0.4, 0.0, 0.1, 0.0]).view(1, 1, 1, 6).to(DEV)
    vals, idx = nsa.select_blocks(p, 4, 4, 5, input_is_prob=True)
    assert idx.flatten().tolist() == [1, 2, 0, 4, 3]
    assert vals.flatten().tolist() == pytest.approx([0.4, 0.4, 0.1, 0.1, 0.0])


# ----------------------------------------------------------------- sliding ---

@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('case', [(2, 4, 2, 70, 32, 9, True), (1, 8, 1, 64, 64, 40, True),
                                  (2, 4, 4, 31, 64, 2, False), (1, 2, 1, 20, 16, 100, False)])
def test_sliding_matches_oracle(case, dtype):
    b, hq, hkv, n, d, win, causal = case
    q = recipe.randn((b, hq, n, d), 1).to(dtype)
    k = recipe.randn((b, hkv, n, d), 2).to(dtype)
    v = recipe.randn((b, hkv, n, d), 3).to(dtype)
    up = recipe.randn((b, hq, n, d), 4).to(dtype)
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref = O.sliding_attend(qo, ko, vo, win, causal)
    rd = grads_of(ref, up.float(), (qo, ko, vo))
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = nsa.sliding_window_attend(qg, kg, vg, win, causal)
    gd = grads_of(out, up.to(DEV), (qg, kg, vg))
    close = closeness(dtype)
    close(out, ref, 'out')
    for g, r, w in zip(gd, rd, ('dq', 'dk', 'dv')):
        close(g, r, w)


@pytest.mark.parametrize('dtype,block,n', [(torch.float32, 16, 100), (torch.bfloat16, 64, 300)])
def test_selected_attend_returns_upstreams_sliding_output_too(dtype, block, n):
    """`return_sliding_window_out` (TRI:1949, 1975-1987): a second output, causal attention over the query's own
    position and the `block_size` keys before it, with its own log-sum-exp; gradients flow through both."""
    b, hq, hkv, d, nsel = 1, 8, 2, 64, 3
    q = recipe.randn((b, hq, n, d), 1).to(dtype)
    k = recipe.randn((b, hkv, n, d), 2).to(dtype)
    v = recipe.randn((b, hkv, n, d), 3).to(dtype)
    up = recipe.randn((b, hq, n, d), 4).to(dtype)
    idx = recipe.randint(0, -(-n // block), (b, hkv, n, nsel), 5)
    mask = idx < (torch.arange(n) // block)[None, None, :, None]
    qo, ko, vo = (t.float().requires_grad_() for t in (q, k, v))
    ref_sel = O.selected_attend(qo, ko, vo, block, idx, mask, True)
    ref_swa = O.sliding_attend(qo, ko, vo, block, True)
    rd = grads_of(ref_sel + ref_swa, up.float(), (qo, ko, vo))
    # the sliding branch's log-sum-exp, restated: scaled logits of the visible keys
    g = hq // hkv
    logits = torch.einsum('bhid,bhjd->bhij', qo.detach(), ko.detach().repeat_interleave(g, dim=1)) * d ** -0.5
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    logits = logits.masked_fill(~((j <= i) & (i - j <= block)), float('-inf'))
    ref_lse = logits.logsumexp(dim=-1)
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    (out, swa), (lse, swa_lse) = nsa.native_sparse_attend(qg, kg, vg, block, idx.to(DEV), mask.to(DEV),
                                                            return_lse=True, return_sliding_window_out=True)
    gd = grads_of(out + swa, up.to(DEV), (qg, kg, vg))
    close = closeness(dtype)
    close(out, ref_sel, 'out')
    close(swa, ref_swa, 'sliding out')
    assert torch.allclose(swa_lse.cpu(), ref_lse, atol=1e-4 if dtype == torch.float32 else 2e-2)
    assert lse.shape == swa_lse.shape == (b, hq, n)
    for got, want, w in zip(gd, rd, ('dq', 'dk', 'dv')):
        if dtype == torch.bfloat16 and w != 'dq':     # sums over every later query of four heads, two branches
            assert_close_bf16(got, want, w, rel_to_max=2e-3)
        else:
            close(got, want, w)
    with pytest.raises(ValueError):
        nsa.native_sparse_attend(qg, kg, vg, block, idx.to(DEV), mask.to(DEV), include_block_causal=False,
                                 return_sliding_window_out=True)


# ----------------------------------------------------------------- combine ---

@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_combine_matches_oracle(dtype):
    b, h, n, d = 2, 4, 37, 32
    os_ = [recipe.randn((b, h, n, d), s).to(dtype) for s in (1, 2, 3)]
    gates = torch.sigmoid(recipe.randn((b, n, h * 3), 4)).to(dtype)
    up = recipe.randn((b, n, h * d), 5).to(dtype)
    ro = [t.float().requires_grad_() for t in os_]
    rg = gates.float().requires_grad_()
    ref = O.combine(*ro, rg.view(b, n, h, 3).transpose(1, 2))
    rd = grads_of(ref, up.float(), (*ro, rg))
    go = [t.to(DEV).requires_grad_() for t in os_]
    gg = gates.to(DEV).requires_grad_()
    out = nsa.gated_combine(*go, gg.view(b, n, h, 3).transpose(1, 2))
    gd = grads_of(out, up.to(DEV), (*go, gg))
    close = closeness(dtype)
    close(out, ref, 'out')
    for g, r, w in zip(gd, rd, ('d_cmp', 'd_sel', 'd_swa', 'd_gates')):
        close(g, r, w)


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_combine_gather_writes_every_destination(dtype):
    # the fused combine + all-gather kernel with its destinations on one GPU: two buffers stand for two ranks' outputs
    from native_sparse_attention_pytorch_b200 import ops
    b, h, n, d = 2, 4, 37, 32
    os_ = [recipe.randn((b, h, n, d), s).to(dtype).to(DEV) for s in (1, 2, 3)]
    gates = torch.sigmoid(recipe.randn((b, n, h * 3), 4)).to(dtype).to(DEV).view(b, n, h, 3).transpose(1, 2)
    ref = O.combine(*[t.float().cpu() for t in os_], gates.float().cpu())
    total, offset = 3 * h * d, h * d           # this "rank" owns the middle third of the features
    outs = [torch.full((b, n, total), 7.0, dtype=dtype, device=DEV) for _ in range(2)]
    ops.gated_combine_gather(*os_, gates, [t.data_ptr() for t in outs], total, offset)
    close = closeness(dtype)
    for t in outs:
        close(t[..., offset:offset + h * d], ref, 'own features')
        assert bool((t[..., :offset] == 7).all()) and bool((t[..., offset + h * d:] == 7).all())
    with pytest.raises(nsa_lib.NsaError):
        ops.gated_combine_gather(*os_, gates, [outs[0].data_ptr()], total, total - 8)      # heads do not fit


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_rotary_kernel_matches_oracle(dtype):
    from native_sparse_attention_pytorch_b200.rotary import RotaryEmbedding
    b, h, n, d = 2, 3, 77, 32
    base = recipe.randn((b, n, h * d), 1).to(dtype)                 # heads as a strided view, as after to_qkv
    up = recipe.randn((b, h, n, d), 2).to(dtype)
    for offset in (0, 5):
        xr = base.float().view(b, n, h, d).transpose(1, 2).requires_grad_()
        ref = O.rotary(xr, offset=offset)
        (rg,) = torch.autograd.grad((ref * up.float()).sum(), xr)
        xg = base.to(DEV).view(b, n, h, d).transpose(1, 2).requires_grad_()
        out = RotaryEmbedding(d).to(DEV).rotate_queries_or_keys(xg, offset=offset)
        (gg,) = torch.autograd.grad((out * up.to(DEV)).sum(), xg)
        assert out.is_contiguous() and out.dtype == dtype
        if dtype == torch.float32:
            assert_close_f32(out, ref, 'out', tol=2e-6)              # same fp32 operations; cos/sin tables from the GPU
            assert_close_f32(gg, rg, 'd x')
        else:
            assert_close_bf16(out, ref, 'out')
            assert_close_bf16(gg, rg, 'd x')


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('shape', [(3, 37, 64), (2, 1000, 512), (1, 5, 1000), (4, 9, 2048 // 2), (0, 4, 64)])
def test_rms_norm_kernel_matches_the_formula(dtype, shape):
    """y = x * rsqrt(mean(x^2) + eps) * weight in fp32 on the CPU (the formula of torch.nn.RMSNorm; its default eps is
    the machine epsilon of fp32 for bf16 inputs too), forward and backward, also through a strided view and an fp32 weight."""
    from native_sparse_attention_pytorch_b200.norm import RMSNorm, rms_norm, rms_norm_supported
    b, n, dim = shape
    x = recipe.randn((b, n, 2 * dim), 11).to(dtype)[..., :dim]        # rows 2*dim apart
    wt = (1.0 + 0.3 * recipe.randn((dim,), 12)).to(dtype)
    up = recipe.randn((b, n, dim), 13).to(dtype)
    eps = torch.finfo(torch.float32).eps
    xr, wr = x.float().requires_grad_(), wt.float().requires_grad_()
    ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps) * wr
    rdx, rdw = torch.autograd.grad((ref * up.float()).sum(), (xr, wr))
    for weight_dtype in sorted({dtype, torch.float32}, key=str):
        mod = RMSNorm(dim).to(DEV).to(weight_dtype)
        with torch.no_grad():
            mod.weight.copy_(wt)
        xg = x.to(DEV).requires_grad_()
        assert rms_norm_supported(xg, mod.weight)
        out = mod(xg)
        assert out.dtype == dtype and out.shape == x.shape
        gdx, gdw = torch.autograd.grad((out * up.to(DEV)).sum(), (xg, mod.weight))
        assert gdw.dtype == weight_dtype
        if dtype == torch.float32:
            assert_close_f32(out, ref, 'y')
            assert_close_f32(gdx, rdx, 'dx')
            assert_close_f32(gdw, rdw, 'dweight')
        else:
            assert_close_bf16(out, ref, 'y')
            assert_close_bf16(gdx, rdx, 'dx')
            assert_close_bf16(gdw, rdw, 'dweight')
        assert torch.equal(rms_norm(x.to(DEV), mod.weight.detach()), out.detach())


@pytest.mark.gpu
@pytest.mark.parametrize('shape', [(2, 4, 16384, 16, 64, 16), (1, 1, 65536, 16, 64, 16)])
def test_selection_at_full_size_equals_the_oracle_steps(shape):
    """The selection kernel at the row lengths of the full-layer and the long-context configuration (256 and 1024
    block columns per row), against the oracle's steps evaluated with the same tensor on the GPU.  PyTorch's CUDA
    softmax and the kernel's differ in the last bit here and there, so two blocks whose probabilities are one ulp apart
    may swap: the picks must be a top-k of the oracle's probabilities up to that ulp, in non-increasing order, and
    identical for (nearly) all rows whose k+1 largest values are distinct."""
    b, hs, n, st, sel, nsel = shape
    ncb = n // st
    gen = torch.Generator(DEV).manual_seed(3)
    imp = torch.randn(b, hs, n, ncb, generator=gen, device=DEV)
    invisible = torch.arange(ncb, device=DEV)[None, :] >= (torch.arange(n, device=DEV) // st)[:, None]
    imp = imp.masked_fill(invisible, nsa.ops.mask_sentinel(torch.float32))
    probs = O.importance_scores(imp, 0, hs, st, sel, True)
    ref_vals, ref_idx = O.select_blocks(probs, nsel)
    vals, idx = nsa.select_blocks(imp, sel, st, nsel)
    assert_close_f32(vals, ref_vals, 'values', tol=1e-6)
    assert torch.equal(vals > 1e-10, ref_vals > 1e-10)
    top = probs.topk(nsel + 1, dim=-1).values
    unique = (top[..., :-1] > top[..., 1:]).all(dim=-1)
    assert unique.float().mean().item() > 0.5
    same = (idx == ref_idx).all(dim=-1)
    assert same[unique].float().mean().item() > 0.999
    picked = probs.gather(-1, idx)                      # the oracle's probabilities of the kernel's picks
    ulp = 2e-7 * probs.amax(dim=-1, keepdim=True)
    assert (picked >= top[..., -1:] - ulp).all()        # none of them is below the (k+1)-th largest
    assert (picked[..., :-1] >= picked[..., 1:] - ulp).all()


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('block,stride', [(8, 4), (5, 2), (4, 4), (32, 16)])
def test_compress_windows_match_pad_unfold_add(dtype, block, stride):
    from native_sparse_attention_pytorch_b200 import ops
    b, h, n, d = 2, 3, 77, 32
    ncb = n // stride
    base = recipe.randn((b, n, h * d), 1).to(dtype)                   # heads as a strided view
    pos = recipe.randn((h, block, d), 2).to(dtype)
    up = recipe.randn((b, h, ncb, block, d), 3).to(dtype)
    xr = base.float().view(b, n, h, d).transpose(1, 2).requires_grad_()
    pr = pos.float().requires_grad_()
    ref = O.compress_windows(xr[..., : ncb * stride, :], block, stride) + pr[None, :, None]
    gx, gp = torch.autograd.grad((ref * up.float()).sum(), (xr, pr))
    xg = base.to(DEV).view(b, n, h, d).transpose(1, 2).requires_grad_()
    pg = pos.to(DEV).requires_grad_()
    out = ops.compress_windows(xg, pg, block, stride, ncb)
    dx, dp = torch.autograd.grad((out * up.to(DEV)).sum(), (xg, pg))
    close = closeness(dtype)
    close(out, ref, 'windows')
    close(dx, gx, 'd x')
    assert_close_bf16(dp, gp, 'd positions', rel_to_max=5e-3) if dtype == torch.bfloat16 else close(dp, gp, 'd positions')
