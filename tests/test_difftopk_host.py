"""The host-side part of the differentiable top-k (upstream NSA:715): the gradient of the selected probabilities with
respect to the importance matrix, and of the importance with respect to q and the compressed keys, are plain PyTorch
in `ops`; here they are checked on the CPU against autograd through the oracle's own formulation."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from native_sparse_attention_pytorch_b200 import ops


@pytest.mark.parametrize('st,blk,g', [(4, 8, 2), (8, 8, 1), (2, 8, 4)])
def test_selection_gradient_reaches_q_and_compressed_keys(st, blk, g):
    b, hkv, n, d, nsel, m = 2, 2, 70, 16, 3, 1
    ncb = n // st
    q = recipe.randn((b, hkv * g, n, d), 1).requires_grad_()
    ck = recipe.randn((b, hkv, ncb, d), 2).requires_grad_()
    cv = recipe.randn((b, hkv, ncb, d), 3)
    mem = recipe.randn((2, hkv, m, d), 4)
    _, csim = O.compressed_attend(q, ck, cv, mem[0], mem[1], st, True)
    vals, idx = O.select_blocks(O.importance_scores(csim, m, hkv, st, blk), nsel)
    w = recipe.randn(tuple(vals.shape), 5)
    gq, gck = torch.autograd.grad((vals * w).sum(), (q, ck))

    imp = csim[..., m:].reshape(b, hkv, g, n, ncb).mean(dim=2).detach().requires_grad_()
    carried = ops._SelectValuesGrad.apply(imp, vals.detach(), idx, blk, st)
    assert torch.equal(carried, vals)
    (dimp,) = torch.autograd.grad((carried * w).sum(), imp)
    dq, dck = torch.zeros_like(q), torch.zeros(b, hkv, m + ncb, d)
    ck_full = torch.cat((mem[0].expand(b, -1, -1, -1), ck.detach()), dim=2)
    ops._importance_backward(dimp, q.detach(), ck_full, dq, dck, m, st, True, hkv, d ** -0.5)
    assert (dq - gq).abs().max() <= 1e-6 * max(1.0, gq.abs().max())
    assert (dck[:, :, m:] - gck).abs().max() <= 1e-6 * max(1.0, gck.abs().max())
    assert dck[:, :, :m].abs().max() == 0          # memory slots are not part of the importance
