"""The head-sharded hot path on two GPUs: the fused combine + gather (stores into the peers' symmetric memory) and the
NCCL all-gather give the same output as one GPU holding all heads.  Runs as two child processes; skipped on a box
with fewer than two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import recipe
from util import free_port


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    try:
        from native_sparse_attention_pytorch_b200 import ops, sharding
        from native_sparse_attention_pytorch_b200.rotary import RotaryEmbedding
        b, hkv, g, n, d = 1, 4, 4, 700, 64
        st, blk, nsel, win, mem = 16, 64, 4, 128, 1
        ncb = n // st
        bf = lambda shape, seed: recipe.randn(shape, seed).bfloat16().to(dev)
        q, k, v = bf((b, hkv * g, n, d), 21), bf((b, hkv, n, d), 22), bf((b, hkv, n, d), 23)
        ck, cv = bf((b, hkv, mem + ncb, d), 24), bf((b, hkv, mem + ncb, d), 25)
        gates = torch.sigmoid(recipe.randn((b, hkv * g, n, 3), 26)).bfloat16().to(dev)
        qr, kr = RotaryEmbedding(d).to(dev).rotate_queries_with_cached_keys(q, k)
        cfg = dict(num_mem=mem, stride=st, block=blk, num_selected=nsel, window=win, causal=True)
        full = sharding.attend_core(q, qr, kr, v, ck, cv, gates, **cfg)
        via_nccl = sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, **cfg)
        peer = sharding.PeerOutput(b, n, hkv * g * d, torch.bfloat16, dev)
        fused = sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=peer, **cfg).clone()
        fused2 = sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=peer, **cfg).clone()  # buffer reuse
        # the stores on a side stream, and the query heads of every KV head in two, four and uneven runs
        over = [sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=peer, overlap=True,
                                             head_splits=sp, **cfg).clone() for sp in (1, 2, 4, (2, 1, 1))]
        # the combine and the stores done by the selected branch's last kernel
        over += [sharding.sharded_attend_core(q, qr, kr, v, ck, cv, gates, peer_output=peer, fuse_merge=True,
                                              head_splits=sp, **cfg).clone() for sp in (1, 2)]
        ops.check_device_status()
        torch.cuda.synchronize()
        ret[rank] = (bool(torch.equal(via_nccl, full)), bool(torch.equal(fused, full)), bool(torch.equal(fused2, full)),
                     all(bool(torch.equal(o, full)) for o in over))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_fused_gather_equals_nccl_gather_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, True, True, True), 1: (True, True, True, True)}, dict(ret)
