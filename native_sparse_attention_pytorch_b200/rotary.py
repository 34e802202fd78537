"""Rotary position embedding used in front of the selected and sliding
branches (upstream call sites NSA:238, NSA:643).  Convention: inverse
frequency theta^(-2m/d) on the adjacent feature pair (2m, 2m+1), angles in
fp32, result in the input dtype.  On CUDA tensors the rotation is one kernel
of the library (`nsa_rotary`) over tables of cos / sin built here; CPU tensors
(host-side tests) take the same formula in plain PyTorch."""
import ctypes as C

import torch
from torch import nn
from torch.autograd import Function


_INV_FREQ = {}


def _tables(dim, theta, n, offset, device):
    """cos / sin of the angles [n, dim/2], always in fp32: the inverse frequencies are rebuilt here instead of being
    kept as a module buffer, which `module.bfloat16()` would round to 8 bits and so turn positions past a few hundred
    into wrong angles."""
    key = (dim, theta, str(device))
    inv_freq = _INV_FREQ.get(key)
    if inv_freq is None:   # computed on the host (as upstream's package does at construction), kept per device
        inv_freq = _INV_FREQ[key] = (theta ** (-torch.arange(0, dim, 2).float() / dim)).to(device)
    pos = torch.arange(n, device=device, dtype=torch.float32) + offset
    ang = pos[:, None] * inv_freq[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


class _Rotate(Function):
    """out = rotation of every feature pair of x [B, H, N, d] by the angles of the tables [N, d/2]."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        from .ops import dim_order
        ctx.save_for_backward(cos, sin)
        ctx.order = dim_order(x)
        return _launch(x, cos, sin, inverse=False)

    @staticmethod
    def backward(ctx, grad):
        # the gradient is written in the memory layout of the forward's input (heads as a strided view of the
        # projection output), so that the gradient of that view is a view again instead of a copy
        cos, sin = ctx.saved_tensors
        return _launch(grad, cos, sin, inverse=True, order=ctx.order), None, None


def _launch(x, cos, sin, inverse, order=None):
    from . import _lib as L
    from .ops import empty_in_order
    lib = L.load()
    v = 16 // x.element_size()
    if x.stride(-1) != 1 or x.data_ptr() % 16 or any(s % v for s in x.stride()[:-1]):
        x = x.contiguous()
    b, h, n, d = x.shape
    out = empty_in_order((b, h, n, d), order or (0, 1, 2, 3), x.dtype, x.device)
    args = L.RotaryArgs(x=L.t4(x), out=L.ptr(out), cos_table=L.ptr(cos), sin_table=L.ptr(sin), batch=b, heads=h,
                        seq=n, dim_head=d, dtype=L.dtype_code(x), inverse=1 if inverse else 0,
                        out_stride_b=out.stride(0), out_stride_h=out.stride(1), out_stride_n=out.stride(2))
    with torch.cuda.device(x.device):
        L.check(lib.nsa_rotary(C.byref(args), L.stream_of(x)))
    return out


class RotaryEmbedding(nn.Module):
    def __init__(self, dim, theta=10000.0):
        super().__init__()
        self.dim, self.theta = dim, theta

    def rotate_queries_or_keys(self, t, offset=0):
        n = t.shape[-2]
        cos, sin = _tables(self.dim, self.theta, n, offset, t.device)
        if t.is_cuda and t.dim() == 4 and t.dtype in (torch.float32, torch.bfloat16) and \
                t.shape[-1] % (16 // t.element_size()) == 0:
            return _Rotate.apply(t, cos, sin)
        cos, sin = cos.repeat_interleave(2, dim=-1), sin.repeat_interleave(2, dim=-1)
        x = t.float()
        even, odd = x[..., 0::2], x[..., 1::2]
        rotated = torch.stack((-odd, even), dim=-1).flatten(-2)
        return (x * cos + rotated * sin).to(t.dtype)

    def rotate_queries_with_cached_keys(self, q, k):
        nq, nk = q.shape[-2], k.shape[-2]
        return self.rotate_queries_or_keys(q, offset=nk - nq), self.rotate_queries_or_keys(k)
