"""ctypes binding of libnsa_b200.so (declarations in include/nsa_b200.h).

The library is the only implementation this package has: loading fails with a
clear error when it has not been built, and every operator raises when its
tensors are not on a CUDA device.  There is no eager or CPU fallback."""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libnsa_b200.so')

NSA_F32, NSA_BF16 = 0, 1
NSA_ERR_UNSUPPORTED = -6
DIAG_NONE, DIAG_CAUSAL, DIAG_FULL = 0, 1, 2
IMPL_AUTO, IMPL_SIMT, IMPL_SM100 = 0, 1, 2
IMPL_BY_NAME = {'auto': IMPL_AUTO, 'simt': IMPL_SIMT, 'sm100': IMPL_SM100}

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class Tensor4(C.Structure):
    _fields_ = [('ptr', vp), ('stride_b', i64), ('stride_h', i64), ('stride_n', i64)]


class SelFwdArgs(C.Structure):
    _fields_ = [('q', Tensor4), ('k', Tensor4), ('v', Tensor4), ('out', Tensor4),
                ('idx', vp), ('mask', vp), ('lse', vp),
                ('batch', i32), ('q_heads', i32), ('kv_heads', i32), ('sel_heads', i32), ('seq', i32), ('dim_head', i32),
                ('block', i32), ('nsel', i32), ('diag', i32), ('dtype', i32), ('impl', i32), ('scale', f32),
                ('workspace', vp), ('workspace_bytes', i64), ('index', vp), ('index_bytes', i64)]


class SelBwdArgs(C.Structure):
    _fields_ = [('fwd', SelFwdArgs), ('dout', Tensor4), ('dq', vp), ('dk', vp), ('dv', vp), ('slot_grads', vp),
                ('index', vp), ('index_bytes', i64), ('dq_out', Tensor4), ('delta', vp)]


class CmpFwdArgs(C.Structure):
    _fields_ = [('q', Tensor4), ('ck', Tensor4), ('cv', Tensor4), ('out', Tensor4), ('lse', vp), ('importance', vp),
                ('batch', i32), ('q_heads', i32), ('kv_heads', i32), ('sel_heads', i32), ('seq', i32), ('dim_head', i32),
                ('num_mem', i32), ('ncb', i32), ('stride', i32), ('causal', i32), ('dtype', i32), ('impl', i32),
                ('scale', f32), ('sentinel', f32), ('workspace', vp), ('workspace_bytes', i64), ('pooled', vp),
                ('pool', i32)]


class CmpBwdArgs(C.Structure):
    _fields_ = [('fwd', CmpFwdArgs), ('dout', Tensor4), ('dq', vp), ('dck', vp), ('dcv', vp), ('dq_out', Tensor4),
                ('index', vp), ('index_bytes', i64), ('delta', vp)]


class SelectArgs(C.Structure):
    _fields_ = [('importance', vp), ('idx', vp), ('vals', vp), ('rows', i32), ('seq', i32), ('ncb', i32), ('cpf', i32),
                ('k', i32), ('block', i32), ('exclude_own', i32), ('input_is_prob', i32), ('dtype', i32),
                ('pooled', vp), ('causal_limit', i32)]


class SwaFwdArgs(C.Structure):
    _fields_ = [('q', Tensor4), ('k', Tensor4), ('v', Tensor4), ('out', Tensor4), ('lse', vp),
                ('batch', i32), ('q_heads', i32), ('kv_heads', i32), ('seq', i32), ('dim_head', i32),
                ('window', i32), ('causal', i32), ('dtype', i32), ('impl', i32), ('scale', f32),
                ('workspace', vp), ('workspace_bytes', i64)]


class SwaBwdArgs(C.Structure):
    _fields_ = [('fwd', SwaFwdArgs), ('dout', Tensor4), ('dq', vp), ('dk', vp), ('dv', vp), ('dq_out', Tensor4),
                ('index', vp), ('index_bytes', i64), ('delta', vp)]


class CombineFwdArgs(C.Structure):
    _fields_ = [('o_cmp', Tensor4), ('o_sel', Tensor4), ('o_swa', Tensor4), ('gates', Tensor4), ('out', vp),
                ('batch', i32), ('q_heads', i32), ('seq', i32), ('dim_head', i32), ('dtype', i32)]


class CombineBwdArgs(C.Structure):
    _fields_ = [('fwd', CombineFwdArgs), ('dout', vp), ('d_cmp', vp), ('d_sel', vp), ('d_swa', vp), ('d_gates', vp),
                ('delta', vp)]


MAX_GATHER = 8


class CombineGatherArgs(C.Structure):
    _fields_ = [('fwd', CombineFwdArgs), ('outs', vp * MAX_GATHER), ('num_outs', i32), ('multicast', i32),
                ('total_features', i64), ('feature_offset', i64)]


class RotaryArgs(C.Structure):
    _fields_ = [('x', Tensor4), ('out', vp), ('cos_table', vp), ('sin_table', vp), ('batch', i32), ('heads', i32),
                ('seq', i32), ('dim_head', i32), ('dtype', i32), ('inverse', i32),
                ('out_stride_b', i64), ('out_stride_h', i64), ('out_stride_n', i64)]


class WindowsFwdArgs(C.Structure):
    _fields_ = [('x', Tensor4), ('pos', vp), ('out', vp), ('batch', i32), ('heads', i32), ('seq', i32),
                ('dim_head', i32), ('block', i32), ('stride', i32), ('ncb', i32), ('dtype', i32)]


class WindowsBwdArgs(C.Structure):
    _fields_ = [('fwd', WindowsFwdArgs), ('dout', vp), ('dx', vp), ('dpos', vp),
                ('dx_stride_b', i64), ('dx_stride_h', i64), ('dx_stride_n', i64)]


class RmsNormFwdArgs(C.Structure):
    _fields_ = [('x', vp), ('weight', vp), ('y', vp), ('rstd', vp), ('rows', i64), ('x_stride', i64), ('dim', i32),
                ('dtype', i32), ('weight_f32', i32), ('reserved', i32), ('eps', C.c_float), ('reserved2', C.c_float)]


class RmsNormBwdArgs(C.Structure):
    _fields_ = [('fwd', RmsNormFwdArgs), ('dy', vp), ('dx', vp), ('dweight', vp)]


class DecodeArgs(C.Structure):
    _fields_ = [('q', vp), ('qr', vp), ('keys', Tensor4), ('vals', Tensor4), ('ck', Tensor4), ('cv', Tensor4),
                ('mem_k', vp), ('mem_v', vp), ('gates', vp), ('out', vp), ('batch', i32), ('q_heads', i32),
                ('kv_heads', i32), ('dim_head', i32), ('cache_len', i32), ('ncb', i32), ('num_mem', i32),
                ('stride', i32), ('block', i32), ('nsel', i32), ('window', i32), ('dtype', i32), ('scale', f32),
                ('reserved', i32)]


_STRUCTS = [Tensor4, SelFwdArgs, SelBwdArgs, CmpFwdArgs, CmpBwdArgs, SelectArgs, SwaFwdArgs, SwaBwdArgs,
            CombineFwdArgs, CombineBwdArgs, CombineGatherArgs, RotaryArgs, WindowsFwdArgs, WindowsBwdArgs,
            RmsNormFwdArgs, RmsNormBwdArgs, DecodeArgs]

ENTRY_POINTS = ['nsa_sel_fwd', 'nsa_sel_bwd', 'nsa_sel_workspace_bytes', 'nsa_sel_index_bytes', 'nsa_cmp_index_bytes', 'nsa_swa_index_bytes', 'nsa_sel_bwd_stores_dq', 'nsa_cmp_bwd_stores_dq', 'nsa_swa_bwd_stores_dq',
                'nsa_sel_fwd_static', 'nsa_sel_static_status', 'nsa_launch_count', 'nsa_selftest_bounded_wait', 'nsa_decode_step',
                'nsa_sel_static_scratch_bytes', 'nsa_cmp_workspace_bytes', 'nsa_swa_workspace_bytes', 'nsa_cmp_fwd', 'nsa_cmp_fwd_pools', 'nsa_cmp_bwd', 'nsa_select',
                'nsa_swa_fwd', 'nsa_swa_bwd', 'nsa_combine_fwd', 'nsa_combine_bwd', 'nsa_combine_fwd_gather', 'nsa_sel_fwd_combine_gather', 'nsa_rotary', 'nsa_windows_fwd', 'nsa_windows_bwd', 'nsa_rmsnorm_fwd', 'nsa_rmsnorm_bwd', 'nsa_last_error',
                'nsa_abi_version', 'nsa_struct_size']

_lib = None


class NsaError(RuntimeError):
    pass


def load():
    """Load the shared library once; raise if it is missing or its struct
    layouts disagree with this binding."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NsaError(f'{LIB_PATH} is missing: build it with `python -m native_sparse_attention_pytorch_b200.build` '
                       '(this package has no fallback implementation)')
    lib = C.CDLL(LIB_PATH)
    lib.nsa_last_error.restype = C.c_char_p
    lib.nsa_sel_workspace_bytes.restype = i64
    lib.nsa_sel_index_bytes.restype = i64
    lib.nsa_cmp_index_bytes.restype = i64
    lib.nsa_swa_index_bytes.restype = i64
    lib.nsa_sel_static_scratch_bytes.restype = i64
    lib.nsa_launch_count.restype = i64
    lib.nsa_sel_static_status.argtypes = [vp, vp]
    lib.nsa_selftest_bounded_wait.argtypes = [vp, i64, vp]
    lib.nsa_cmp_workspace_bytes.restype = i64
    lib.nsa_swa_workspace_bytes.restype = i64
    for which, st in enumerate(_STRUCTS):
        if lib.nsa_struct_size(which) != C.sizeof(st):
            raise NsaError(f'struct layout mismatch for {st.__name__}: library {lib.nsa_struct_size(which)} '
                           f'bytes, binding {C.sizeof(st)} bytes')
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        msg = load().nsa_last_error().decode()
        raise NsaError(f'libnsa_b200 returned {rc}: {msg}')


def dtype_code(t):
    if t.dtype == torch.float32:
        return NSA_F32
    if t.dtype == torch.bfloat16:
        return NSA_BF16
    raise NsaError(f'unsupported dtype {t.dtype}: the kernels take float32 or bfloat16')


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NsaError('the NSA kernels run on CUDA tensors only; there is no CPU implementation in this package')


def rowwise(t):
    """Return t itself if its last axis is contiguous and rows are 16-byte aligned, else a contiguous copy."""
    per16 = 16 // t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % per16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def t4(t):
    return Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_of(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
