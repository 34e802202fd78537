"""The multi-rank path on CPU: two (and four) gloo ranks split the (batch, KV head) units, run the operator on
their share -- the CPU oracle stands in for the CUDA operator here -- and all-gather the output."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import recipe
from oracle import nsa_oracle as O
from native_sparse_attention_pytorch_b200 import sharding


def test_unit_ranges_cover_everything_once():
    for units in (1, 3, 8, 16):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                a, b = sharding.unit_range(units, world, r)
                got += list(range(a, b))
            assert got == list(range(units))


def test_plan_prefers_batch_then_heads():
    assert sharding.plan(8, 4, 8) == ('batch', 8)
    assert sharding.plan(1, 8, 8) == ('heads', 8)
    assert sharding.plan(2, 4, 8) == ('heads', 4)
    assert sharding.local_slices(2, 4, 8, 5) == (slice(1, 2), slice(1, 2))
    with pytest.raises(ValueError):
        sharding.plan(3, 4, 8)


def oracle_attend(q, k, v, block, idx, mask, include_block_causal=True):
    return O.selected_attend(q, k, v, block, idx, mask, include_block_causal)


def worker(rank, world, port, batch, hkv, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        g, n, d, block, nsel = 2, 70, 16, 8, 2
        q = recipe.randn((batch, hkv * g, n, d), 1)
        k = recipe.randn((batch, hkv, n, d), 2)
        v = recipe.randn((batch, hkv, n, d), 3)
        idx = recipe.randint(0, -(-n // block), (batch, hkv, n, nsel), 4)
        mask = idx < (torch.arange(n) // block)[None, None, :, None]
        out = sharding.sharded_selected_attend(q, k, v, block, idx, mask, attend_fn=oracle_attend)
        full = oracle_attend(q, k, v, block, idx, mask)
        ret[rank] = float((out - full).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world,batch,hkv', [(2, 2, 2), (2, 1, 4), (4, 2, 2)])
def test_sharded_attend_equals_unsharded(world, batch, hkv):
    port = 29500 + (os.getpid() % 2000) + world * 7 + batch
    ret = mp.Manager().dict()
    mp.spawn(worker, args=(world, port, batch, hkv, ret), nprocs=world, join=True)
    assert len(ret) == world and all(e < 1e-6 for e in ret.values()), dict(ret)
