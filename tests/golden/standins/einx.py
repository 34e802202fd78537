"""Stand-in for the `einx` package, used only when importing the upstream
library in the fixture-generation script.  Only the five broadcast helpers the
upstream module path calls are provided; each is the plain elementwise torch
op broadcast to the pattern's output axes."""
import torch


def _parse(pattern):
    lhs, rhs = pattern.split('->') if '->' in pattern else (pattern, None)
    ins = [p.split() for p in lhs.split(',')]
    out = rhs.split() if rhs is not None else max(ins, key=len)
    return ins, out


def _expand(t, axes, out):
    if not torch.is_tensor(t):
        return t
    # place every input axis at its position among the output axes
    idx = [slice(None) if a in axes else None for a in out]
    perm = [axes.index(a) for a in out if a in axes]
    return t.permute(*perm)[tuple(idx)]


def _binary(op):
    def fn(pattern, a, b):
        ins, out = _parse(pattern)
        return op(_expand(a, ins[0], out), _expand(b, ins[1], out))
    return fn


add = _binary(torch.add)
multiply = _binary(torch.mul)
less = _binary(torch.lt)
equal = _binary(torch.eq)


def where(pattern, cond, a, b):
    ins, out = _parse(pattern)
    a = _expand(a, ins[1], out)
    cond = _expand(cond, ins[0], out)
    if torch.is_tensor(b):
        b = _expand(b, ins[2], out)
    return torch.where(cond, a, b)
