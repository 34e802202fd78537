"""The CPU oracle against the vectors stored from the unmodified upstream
library (tests/golden/make_golden.py).  This is what pins the oracle."""
import os

import numpy as np
import pytest
import torch

import recipe
from oracle import nsa_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


def load(name):
    z = np.load(os.path.join(GOLDEN, name + '.npz'))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def close(a, b, tol=2e-5):
    assert a.shape == b.shape, (a.shape, b.shape)
    err = (a - b).abs().max().item() if a.numel() else 0.0
    ref = b.abs().max().item() if b.numel() else 1.0
    assert err <= tol * max(1.0, ref), f'max abs err {err} (ref max {ref})'


@pytest.mark.parametrize('name', list(recipe.LAYER_CASES))
def test_layer_matches_upstream(name):
    c = recipe.LAYER_CASES[name]
    gold = load('layer_' + name)
    kw = dict(c['kw'])
    attn = O.OracleSparseAttention(**kw)
    recipe.fill_weights(attn, seed=7, rich=c['rich'])
    x = recipe.layer_input(name).requires_grad_()
    out, mid = attn(x, return_intermediates=True)
    for key in ('o_cmp', 'o_sel', 'o_swa', 'gates', 'ck', 'cv'):
        if mid.get(key) is not None and mid[key].requires_grad:
            mid[key].retain_grad()
    (out * recipe.randn(out.shape, 13)).sum().backward()

    close(out, gold['out'])
    close(x.grad, gold['x_grad'], 5e-5)
    if 'idx' in gold:
        assert torch.equal(mid['idx'], gold['idx'])          # selection is bit-exact
        close(mid['vals'], gold['vals'], 1e-6)
        close(mid['probs'], gold['probs'], 1e-6)
    else:
        assert mid['idx'] is None
    close(mid['o_sel'], gold['o_sel'])
    close(mid['gates'].grad, gold['gates_grad'].reshape(mid['gates'].permute(0, 2, 1, 3).shape).permute(0, 2, 1, 3)
          if gold['gates_grad'].shape != mid['gates'].shape else gold['gates_grad'], 5e-5)
    for key in ('csim', 'o_cmp', 'o_swa', 'qr', 'kr'):
        if key in gold:
            close(mid[key], gold[key])
    for key in ('o_cmp', 'o_sel', 'o_swa', 'ck', 'cv'):
        if key + '_grad' in gold:
            close(mid[key].grad, gold[key + '_grad'], 5e-5)
    for pname, p in attn.named_parameters():
        g = gold.get('pgrad.' + pname)
        if g is None:
            assert p.grad is None or p.grad.abs().sum() == 0, pname
            continue
        got = torch.tensor([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()], dtype=torch.float64)
        assert torch.allclose(got, g, rtol=2e-4, atol=1e-6), (pname, got, g)


@pytest.mark.parametrize('name', list(recipe.OP_CASES))
def test_selected_attend_matches_upstream_kernel_check(name):
    c = recipe.OP_CASES[name]
    gold = load(name)
    q, k, v, idx, mask = recipe.op_inputs(name)
    scale = torch.ones(idx.shape)
    q, k, v, scale = (t.clone().requires_grad_() for t in (q, k, v, scale))
    out, lse = O.selected_attend(q, k, v, c['block'], idx, mask, causal=True, gates=scale, return_lse=True)
    (out * recipe.randn(out.shape, 29)).sum().backward()
    close(out, gold['out'])
    close(lse, gold['lse'])
    close(q.grad, gold['dq'], 5e-5)
    close(k.grad, gold['dk'], 5e-5)
    close(v.grad, gold['dv'], 5e-5)
    close(scale.grad, gold['dscale'], 5e-5)


def test_rows_subset_is_consistent():
    q, k, v, idx, mask = recipe.op_inputs('op_ragged')
    full = O.selected_attend(q, k, v, 16, idx, mask, causal=True)
    rows = torch.tensor([0, 5, 16, 31, 106])
    part = O.selected_attend(q, k, v, 16, idx, mask, causal=True, rows=rows)
    close(part, full[:, :, rows], 1e-6)


def test_language_model_harness_matches_upstream_transformer():
    """The benchmark's language-model harness (bench.build_lm), built around the oracle's layer, against the stored
    results of upstream's Transformer on the same seeded weights and token ids: loss, logits, gradient norms."""
    import bench
    gold = load('lm_toy')
    model, _ = bench.build_lm(recipe.LM_CASE, 'cpu', dtype=torch.float32,
                              attn_cls=lambda **kw: O.OracleSparseAttention(**kw))
    recipe.lm_fill_weights(model, seed=9)
    ids = recipe.lm_ids()
    loss = model(ids)
    loss.backward()
    assert abs(loss.item() - gold['loss'].item()) <= 1e-5 * abs(gold['loss'].item())
    with torch.no_grad():
        close(model.logits(ids[:, :-1]), gold['logits'], 2e-5)
    seen = 0
    for pname, p in model.named_parameters():
        g = gold.get('pgrad.' + pname)
        if g is None:
            assert p.grad is None or p.grad.abs().sum().item() == 0, pname
            continue
        got = torch.tensor([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()], dtype=torch.float64)
        assert torch.allclose(got, g, rtol=1e-3, atol=1e-7), (pname, got, g)
        seen += 1
    assert seen == sum(1 for k in gold if k.startswith('pgrad.'))
