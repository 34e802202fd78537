"""The per-pass forms of the head-sharded hot path on ONE GPU: with `sharding.LocalOutput` (the output tensor as the
only destination) every form that `sharded_attend_core` offers for the fused gather -- stores on a side stream, runs of
query heads, the selected branch's merge kernel doing the combine -- runs without other ranks and must reproduce
`attend_core` byte for byte.  (The same forms across two GPUs: tests/test_gpu_multi.py.)"""
import pytest
import torch

import recipe

pytestmark = pytest.mark.gpu
DEV = 'cuda'


@pytest.mark.parametrize('d,g', [(64, 4), (128, 8)])
def test_every_form_equals_the_plain_hot_path(d, g):
    from native_sparse_attention_pytorch_b200 import ops, sharding
    from native_sparse_attention_pytorch_b200.rotary import RotaryEmbedding
    b, hkv, n = 1, 2, 900
    st, blk, nsel, win, mem = 16, 64, 4, 128, 1
    ncb = (n - 2 * st) // st + 1
    bf = lambda shape, seed: recipe.randn(shape, seed).bfloat16().to(DEV)
    q, k, v = bf((b, hkv * g, n, d), 21), bf((b, hkv, n, d), 22), bf((b, hkv, n, d), 23)
    ck, cv = bf((b, hkv, mem + ncb, d), 24), bf((b, hkv, mem + ncb, d), 25)
    gates = torch.sigmoid(recipe.randn((b, hkv * g, n, 3), 26)).bfloat16().to(DEV)
    qr, kr = RotaryEmbedding(d).rotate_queries_with_cached_keys(q, k)
    cfg = dict(num_mem=mem, stride=st, block=blk, num_selected=nsel, window=win, causal=True)
    full = sharding.attend_core(q, qr, kr, v, ck, cv, gates, **cfg)
    out = sharding.LocalOutput(b, n, hkv * g * d, torch.bfloat16, torch.device(DEV))
    forms = [dict(), dict(overlap=True), dict(overlap=True, head_splits=2), dict(overlap=True, head_splits=(g // 2, g // 4, g // 4)),
             dict(fuse_merge=True), dict(fuse_merge=True, head_splits=2), dict(fuse_merge=True, heads_per_pass=2)]
    for form in forms:
        out.buffer.zero_()
        got = sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=out, **form, **cfg)
        ops.check_device_status()
        assert torch.equal(got, full), form
    # without a destination object the merged tensor comes back directly
    assert torch.equal(sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, **cfg), full)
    with pytest.raises(ValueError):
        sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=out, head_splits=3, **cfg)
