"""nsa_sel_fwd_static: the selected-block forward for callers that cannot allocate device memory
when they call (they pass inputs and outputs only; the work buffer is a fixed area inside the
library).  Called through the C ABI and compared with nsa_sel_fwd on the same inputs, twice in a
row with different inputs, because the shared area keeps whatever the previous call left in it.
This file sorts last on purpose, so a run that stops at the first failure has already executed
every other test."""
import ctypes as C

import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import assert_close_bf16

from native_sparse_attention_pytorch_b200 import _lib as L

pytestmark = pytest.mark.gpu
DEV = 'cuda'
BLOCK = 64


def problem(seed, b=1, hq=8, hkv=2, n=700, d=64, nsel=4):
    nfb = -(-n // BLOCK)
    q = recipe.randn((b, hq, n, d), seed).bfloat16().to(DEV)
    k = recipe.randn((b, hkv, n, d), seed + 1).bfloat16().to(DEV)
    v = recipe.randn((b, hkv, n, d), seed + 2).bfloat16().to(DEV)
    idx = recipe.randint(0, nfb, (b, hkv, n, nsel), seed + 3).to(DEV)
    mask = (idx < (torch.arange(n, device=DEV) // BLOCK)[None, None, :, None]).view(torch.uint8)
    return q, k, v, idx, mask


def args_for(q, k, v, idx, mask, out, lse, ws=None):
    b, hq, n, d = q.shape
    a = L.SelFwdArgs(q=L.t4(q), k=L.t4(k), v=L.t4(v), out=L.t4(out), idx=idx.data_ptr(), mask=mask.data_ptr(),
                     lse=lse.data_ptr(), batch=b, q_heads=hq, kv_heads=k.shape[1], sel_heads=idx.shape[1], seq=n,
                     dim_head=d, block=BLOCK, nsel=idx.shape[-1], diag=L.DIAG_CAUSAL, dtype=L.NSA_BF16,
                     impl=L.IMPL_SM100, scale=d ** -0.5, workspace=None, workspace_bytes=0)
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def run_both(lib, seed, **kw):
    q, k, v, idx, mask = problem(seed, **kw)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ref_out, new_out = torch.empty_like(q), torch.full_like(q, float('nan'))
    ref_lse = torch.empty(q.shape[:3], dtype=torch.float32, device=DEV)
    new_lse = torch.full_like(ref_lse, float('nan'))
    a = args_for(q, k, v, idx, mask, ref_out, ref_lse)
    need = lib.nsa_sel_workspace_bytes(C.byref(a), 0)
    assert 0 < need <= lib.nsa_sel_static_scratch_bytes()
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    L.check(lib.nsa_sel_fwd(C.byref(args_for(q, k, v, idx, mask, ref_out, ref_lse, ws)), stream))
    status = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    torch.cuda.synchronize()
    free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    L.check(lib.nsa_sel_fwd_static(C.byref(args_for(q, k, v, idx, mask, new_out, new_lse)), stream))
    L.check(lib.nsa_sel_static_status(status.data_ptr(), stream))
    torch.cuda.synchronize()
    # the call took no device memory: neither from the driver nor from PyTorch's pool
    assert torch.cuda.mem_get_info()[0] >= free_before and torch.cuda.memory_allocated() == held_before
    assert status.item() == 0, 'a kernel of the static forward gave up on a wait'
    assert_close_bf16(new_out, ref_out, 'out', roundings=2)
    assert_close_bf16(new_lse, ref_lse, 'lse')
    return q, k, v, idx, mask, new_out


def test_static_scratch_forward_matches_the_regular_entry_point_twice_in_a_row():
    lib = L.load()
    run_both(lib, seed=41)                                 # the first call on the device also looks the area up
    run_both(lib, seed=97, n=333, hq=4, hkv=1, nsel=2)     # a different, smaller problem over the same area
    # dim_head 128, and the result against the CPU oracle as well
    q, k, v, idx, mask, out = run_both(lib, seed=7, n=400, hq=8, hkv=1, d=128, nsel=3)
    ref = O.selected_attend(q.float().cpu(), k.float().cpu(), v.float().cpu(), BLOCK, idx.cpu(), mask.bool().cpu(), True)
    assert_close_bf16(out, ref, 'out vs oracle')


def test_static_scratch_forward_rejects_what_does_not_fit():
    lib = L.load()
    q, k, v, idx, mask = problem(5, b=1, hq=32, hkv=4, n=4096, nsel=16)   # needs far more than the built-in area
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=DEV)
    rc = lib.nsa_sel_fwd_static(C.byref(args_for(q, k, v, idx, mask, out, lse)), None)
    assert rc == -5 and b'scratch' in lib.nsa_last_error()
    small = problem(6, d=32)                                               # a shape only the generic kernels serve
    out = torch.empty_like(small[0])
    lse = torch.empty(small[0].shape[:3], dtype=torch.float32, device=DEV)
    assert lib.nsa_sel_fwd_static(C.byref(args_for(*small, out, lse)), None) == -6
