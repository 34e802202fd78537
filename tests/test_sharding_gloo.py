"""The multi-rank path on CPU: two (and four) gloo ranks split the (batch, KV head) units, run the operator on
their share -- the CPU oracle stands in for the CUDA operator here -- and all-gather the output."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import recipe
from util import free_port
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
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(worker, args=(world, port, batch, hkv, ret), nprocs=world, join=True)
    assert len(ret) == world and all(e < 1e-6 for e in ret.values()), dict(ret)


# ---- the whole hot path, KV-head groups split over the ranks, output all-gathered --------------------------------

NUM_MEM, STRIDE, BLOCK, NSEL, WINDOW = 1, 4, 8, 2, 6


def _oracle_fns():
    def compressed(q, ck, cv, num_mem, stride, causal, sel_heads=None, want_importance=True):
        hkv = ck.shape[1]
        zero = ck.new_zeros(hkv, 0, ck.shape[-1])
        out, csim = O.compressed_attend(q, ck, cv, zero, zero, stride, causal) if num_mem == 0 else \
            _compressed_with_mem(q, ck, cv, num_mem, stride, causal)
        return out, (csim, hkv)

    def _compressed_with_mem(q, ck, cv, num_mem, stride, causal):
        # the operator takes the memory slots in front of ck / cv; the oracle takes them apart (batch 1 per call)
        outs, sims = [], []
        for b in range(q.shape[0]):
            o, s = O.compressed_attend(q[b:b + 1], ck[b:b + 1, :, num_mem:], cv[b:b + 1, :, num_mem:],
                                       ck[b, :, :num_mem], cv[b, :, :num_mem], stride, causal)
            outs.append(o)
            sims.append(s)
        return torch.cat(outs), torch.cat(sims)

    def select(importance, block, stride, nsel, dtype=None):
        csim, hkv = importance
        return O.select_blocks(O.importance_scores(csim, NUM_MEM, hkv, stride, block), nsel)

    def selected(q, k, v, block, idx, mask, include_block_causal=True):
        return O.selected_attend(q, k, v, block, idx, mask, include_block_causal)

    return dict(compressed=compressed, select=select, selected=selected, sliding=O.sliding_attend, combine=O.combine)


def core_worker(rank, world, port, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        b, hkv, g, n, d = 1, 4, 2, 50, 16
        ncb = n // STRIDE
        q = recipe.randn((b, hkv * g, n, d), 11)
        k = recipe.randn((b, hkv, n, d), 12)
        v = recipe.randn((b, hkv, n, d), 13)
        qr, kr = O.rotary(q), O.rotary(k)
        ck = recipe.randn((b, hkv, NUM_MEM + ncb, d), 14)
        cv = recipe.randn((b, hkv, NUM_MEM + ncb, d), 15)
        gates = torch.sigmoid(recipe.randn((b, hkv * g, n, 3), 16))
        cfg = dict(num_mem=NUM_MEM, stride=STRIDE, block=BLOCK, num_selected=NSEL, window=WINDOW, causal=True,
                   attend_fns=_oracle_fns())
        out = sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, **cfg)
        full = sharding.attend_core(q, qr, kr, v, ck, cv, gates, **cfg)
        ret[rank] = (tuple(out.shape), float((out - full).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4])
def test_head_sharded_hot_path_equals_unsharded(world):
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(core_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for shape, err in ret.values():
        assert shape == (1, 50, 4 * 2 * 16) and err < 1e-6, dict(ret)


def test_kv_head_range():
    assert [sharding.kv_head_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        sharding.kv_head_range(8, 3, 0)


def grad_worker(rank, world, port, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        torch.manual_seed(3)
        layers = torch.nn.ModuleList([torch.nn.Linear(6, 6) for _ in range(3)])
        unused = torch.nn.Linear(6, 6)                    # never reached by the backward: summed by finish()
        x = recipe.randn((4, 6), 10 + rank)

        def backward():
            for p in list(layers.parameters()) + list(unused.parameters()):
                p.grad = None
            h = x
            for layer in layers:
                h = torch.tanh(layer(h))
            h.square().sum().backward()

        backward()
        want = []
        for p in layers.parameters():                     # the flat form: one all-reduce per gradient after the backward
            g = p.grad.clone()
            dist.all_reduce(g)
            want.append(g)
        reducer = sharding.BucketedGradientSum([list(layer.parameters()) for layer in reversed(layers)] +
                                               [list(unused.parameters())])
        for _ in range(2):                                # twice: the counters are reset by start()
            reducer.start()
            backward()
            reducer.finish()
            got = [p.grad for p in layers.parameters()]
            ok = all(torch.equal(a, b) for a, b in zip(got, want))
        ret[rank] = ok and all(p.grad is None for p in unused.parameters())
    finally:
        dist.destroy_process_group()


def test_bucketed_gradient_sum_equals_the_flat_all_reduce():
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(grad_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}
