"""Host-side checks that need no GPU: the library loads, exports every entry
point the header declares, agrees with the binding on struct layouts, and
rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest
import torch

from native_sparse_attention_pytorch_b200 import _lib as L
from native_sparse_attention_pytorch_b200 import SparseAttention, native_sparse_attend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entry_points():
    text = open(os.path.join(ROOT, 'include', 'nsa_b200.h')).read()
    return sorted(set(re.findall(r'\b(nsa_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_are_exported():
    lib = L.load()
    names = declared_entry_points()
    assert set(names) == set(L.ENTRY_POINTS), (names, L.ENTRY_POINTS)
    for n in names:
        assert getattr(lib, n) is not None


def test_struct_layouts_agree():
    lib = L.load()
    for which, st in enumerate(L._STRUCTS):
        assert lib.nsa_struct_size(which) == C.sizeof(st), st.__name__
    assert lib.nsa_struct_size(99) == -1
    assert lib.nsa_abi_version() >= 1


def test_null_and_shape_errors_are_reported_without_a_device():
    lib = L.load()
    assert lib.nsa_sel_fwd(None, None) == -1
    a = L.SelFwdArgs(batch=1, q_heads=3, kv_heads=2, sel_heads=2, seq=8, dim_head=64, block=4, nsel=0, diag=1,
                     dtype=L.NSA_F32, impl=L.IMPL_SIMT, scale=0.125)
    assert lib.nsa_sel_fwd(C.byref(a), None) == -2          # 3 query heads over 2 kv heads
    assert b'q_heads' in lib.nsa_last_error()
    a.q_heads = 4
    a.dim_head = 60
    assert lib.nsa_sel_fwd(C.byref(a), None) == -2          # dim_head not a multiple of 8
    a.dim_head = 64
    a.dtype = 7
    assert lib.nsa_sel_fwd(C.byref(a), None) == -3
    a.dtype = L.NSA_BF16
    assert lib.nsa_sel_fwd(C.byref(a), None) == -1          # q pointer is NULL
    s = L.SelectArgs(importance=None, idx=None, vals=None, rows=1, seq=1, ncb=4, cpf=2, k=3, block=4, dtype=0)
    assert lib.nsa_select(C.byref(s), None) == -2           # k > ncb / cpf


def test_no_cpu_fallback():
    attn = SparseAttention(dim=64, dim_head=16, heads=4, sliding_window_size=2, compress_block_size=4,
                           compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2,
                           use_triton_kernel=True)
    with pytest.raises(RuntimeError):
        attn(torch.randn(1, 8, 64))
    q = torch.randn(1, 2, 8, 16)
    idx = torch.zeros(1, 2, 8, 1, dtype=torch.long)
    with pytest.raises(RuntimeError):
        native_sparse_attend(q, q, q, 4, idx, idx.bool())
    eager = SparseAttention(dim=64, dim_head=16, heads=4, sliding_window_size=2, compress_block_size=4,
                            compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2)
    with pytest.raises(RuntimeError):
        eager(torch.randn(1, 8, 64))


def test_state_dict_names_match_upstream():
    attn = SparseAttention(dim=64, dim_head=16, heads=4, kv_heads=2, sliding_window_size=2, compress_block_size=4,
                           compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2)
    assert sorted(attn.state_dict()) == [
        'combine_heads.weight', 'compress_mem_kv', 'k_compress.1.bias', 'k_compress.1.weight', 'k_compress.3.bias',
        'k_compress.3.weight', 'k_intrablock_positions', 'norm.weight', 'to_qkv.weight',
        'to_strategy_combine.0.bias', 'to_strategy_combine.0.weight', 'v_compress.1.bias', 'v_compress.1.weight',
        'v_compress.3.bias', 'v_compress.3.weight', 'v_intrablock_positions']


def test_rotary_and_gather_entry_points_validate_their_arguments():
    lib = L.load()
    assert lib.nsa_rotary(None, None) == -1
    r = L.RotaryArgs(batch=1, heads=2, seq=8, dim_head=60, dtype=L.NSA_BF16, inverse=0)
    assert lib.nsa_rotary(C.byref(r), None) == -2            # dim_head not a multiple of 16 bytes
    r.dim_head = 64
    assert lib.nsa_rotary(C.byref(r), None) == -1            # pointers are NULL
    r.dtype = 9
    assert lib.nsa_rotary(C.byref(r), None) == -3
    r.dtype, r.seq = L.NSA_F32, 0
    assert lib.nsa_rotary(C.byref(r), None) == 0             # nothing to do

    assert lib.nsa_combine_fwd_gather(None, None) == -1
    fwd = L.CombineFwdArgs(batch=1, q_heads=2, seq=4, dim_head=64, dtype=L.NSA_BF16)
    g = L.CombineGatherArgs(fwd=fwd, num_outs=0, total_features=256, feature_offset=0)
    assert lib.nsa_combine_fwd_gather(C.byref(g), None) == -1    # branch outputs are NULL: reported first
    assert L.MAX_GATHER == 8


def test_norm_entry_points_validate_their_arguments():
    lib = L.load()
    assert lib.nsa_rmsnorm_fwd(None, None) == -1 and lib.nsa_rmsnorm_bwd(None, None) == -1
    a = L.RmsNormFwdArgs(rows=4, x_stride=60, dim=60, dtype=L.NSA_BF16, eps=1e-6)
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == -2        # dim not a multiple of 16 bytes
    a.dim, a.x_stride = 4096, 4096
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == -2        # more pieces than a warp keeps in registers
    a.dim, a.x_stride = 512, 256
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == -2        # overlapping rows
    a.x_stride = 512
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == -1        # pointers are NULL
    a.dtype = 7
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == -3
    a.dtype, a.rows = L.NSA_F32, 0
    assert lib.nsa_rmsnorm_fwd(C.byref(a), None) == 0         # nothing to do
    b = L.RmsNormBwdArgs(fwd=a)
    assert lib.nsa_rmsnorm_bwd(C.byref(b), None) == -1        # the weight gradient is written even for no rows


def test_norm_module_is_state_dict_compatible_and_runs_on_cpu():
    from native_sparse_attention_pytorch_b200.norm import RMSNorm, rms_norm
    m, ref = RMSNorm(24), torch.nn.RMSNorm(24)
    assert list(m.state_dict()) == list(ref.state_dict()) and m.eps is None
    x = torch.randn(3, 5, 24)
    assert torch.equal(m(x), ref(x)) and torch.equal(rms_norm(x, m.weight), ref(x))


def test_decode_and_diff_topk_are_part_of_the_module_interface():
    import inspect
    sig = inspect.signature(SparseAttention.forward)
    assert list(sig.parameters)[:7] == ['self', 'inp', 'cache', 'disable_triton_kernel', 'sliding_window_flex_mask',
                                        'fine_selection_flex_mask', 'return_cache']
    assert hasattr(SparseAttention, 'forward_inference')
    attn = SparseAttention(dim=64, dim_head=16, heads=4, sliding_window_size=2, compress_block_size=4,
                           compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2,
                           causal=True, use_diff_topk=True, use_triton_kernel=True)
    assert attn.use_diff_topk
    with pytest.raises(RuntimeError):                         # still no CPU path, also with a cache
        attn(torch.randn(1, 1, 64), cache=((torch.zeros(1, 4, 0, 16),) * 2, ((torch.zeros(1, 4, 0, 16),) * 2,) * 2))
