"""RMS normalisation of the layer input (upstream: the `nn.RMSNorm` built at NSA:230 and applied at NSA:369 / NSA:579;
the language-model harness uses the same module in front of the feed-forward and the logits, transformer.py:134, 210).

`RMSNorm` keeps `nn.RMSNorm`'s constructor, parameter name and default epsilon (when none is given: the machine
epsilon of fp32, the type PyTorch computes the norm of fp32 and bf16 inputs in), so state dicts interchange.  On
CUDA tensors of a supported shape the forward and the backward are one kernel each of the library
(`nsa_rmsnorm_fwd`, `nsa_rmsnorm_bwd`); other inputs (CPU tensors of host-side tests, dims the kernel does not
serve, a module without weight) take `torch.nn.functional.rms_norm`."""
import ctypes as C

import torch
import torch.nn.functional as F
from torch import nn
from torch.autograd import Function

MAX_PIECES = 256          # sixteen-byte pieces per row the kernel keeps in registers


def rms_norm_supported(x, weight):
    if weight is None or not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16) or x.dim() < 1:
        return False
    v = 16 // x.element_size()
    dim = x.shape[-1]
    return dim % v == 0 and dim // v <= MAX_PIECES and weight.shape == (dim,) and \
        weight.dtype in (x.dtype, torch.float32) and weight.device == x.device


def _rows_view(t):
    """[rows, dim] view of t with contiguous rows on 16-byte boundaries, copying only when t cannot give one."""
    dim = t.shape[-1]
    v = 16 // t.element_size()
    t2 = t.reshape(-1, dim)
    if t2.stride(-1) != 1 or t2.data_ptr() % 16 or (t2.shape[0] > 1 and (t2.stride(0) % v or t2.stride(0) < dim)):
        t2 = t2.contiguous()
    return t2


def _fwd_args(L, x2, weight, y, rstd, eps):
    return L.RmsNormFwdArgs(x=L.ptr(x2), weight=L.ptr(weight), y=L.ptr(y) if y is not None else None,
                            rstd=L.ptr(rstd), rows=x2.shape[0], x_stride=x2.stride(0) if x2.shape[0] > 1 else x2.shape[1],
                            dim=x2.shape[1], dtype=L.dtype_code(x2),
                            weight_f32=1 if weight.dtype == torch.float32 and x2.dtype != torch.float32 else 0,
                            reserved=0, eps=eps, reserved2=0.0)


class _RmsNorm(Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        from . import _lib as L
        lib = L.load()
        x2 = _rows_view(x)
        w = weight.contiguous()
        y = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        args = _fwd_args(L, x2, w, y, rstd, eps)
        with torch.cuda.device(x.device):
            L.check(lib.nsa_rmsnorm_fwd(C.byref(args), L.stream_of(x)))
        ctx.save_for_backward(x2, w, rstd)
        ctx.eps, ctx.shape = eps, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, grad):
        from . import _lib as L
        lib = L.load()
        x2, w, rstd = ctx.saved_tensors
        dy = grad.reshape(x2.shape)
        if not dy.is_contiguous() or dy.data_ptr() % 16:
            dy = dy.contiguous()
        dx = torch.empty(x2.shape, dtype=x2.dtype, device=x2.device)
        dweight = torch.empty(x2.shape[1], dtype=torch.float32, device=x2.device)
        args = L.RmsNormBwdArgs(fwd=_fwd_args(L, x2, w, None, rstd, ctx.eps), dy=L.ptr(dy), dx=L.ptr(dx),
                                dweight=L.ptr(dweight))
        with torch.cuda.device(x2.device):
            L.check(lib.nsa_rmsnorm_bwd(C.byref(args), L.stream_of(x2)))
        return dx.view(ctx.shape), dweight.to(w.dtype), None


def rms_norm(x, weight, eps=None):
    """x * rsqrt(mean(x^2, -1) + eps) * weight over the last axis; eps defaults to the machine epsilon of fp32."""
    if rms_norm_supported(x, weight) and x.numel() > 0:
        return _RmsNorm.apply(x, weight, torch.finfo(torch.float32).eps if eps is None else float(eps))
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


class RMSNorm(nn.RMSNorm):
    def forward(self, x):
        if len(self.normalized_shape) == 1 and rms_norm_supported(x, self.weight) and x.numel() > 0:
            return rms_norm(x, self.weight, self.eps)
        return super().forward(x)
