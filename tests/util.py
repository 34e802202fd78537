"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')

# tolerances of the parity contract
F32_REL = 1e-4      # fp32: max |a-b| <= F32_REL * max(1, max |b|)
BF16_ABS = 2e-2     # bf16: |a-b| <= BF16_ABS + 2^-8 |b| elementwise; the second term is half the spacing of
                    # bf16 numbers at |b| (a stored bf16 value cannot be closer), it is below 2e-2 for |b| < 5


# dk and dv (and the slot gradients) sum thousands of bf16-rounded terms per element, over every query and head that
# attends the key; their bound gets a stated share of the tensor's largest value on top of BF16_ABS
SUM_REL = {'dk': 2e-3, 'dv': 2e-3, 'dscale': 5e-3}


# Every comparison leaves the error it observed here; conftest.py writes the table to the file named by the
# environment variable NSA_PARITY_REPORT at the end of the session (and pytest -rA shows nothing of it otherwise).
OBSERVED = {}


def _current_test():
    return os.environ.get('PYTEST_CURRENT_TEST', '?').split(' ')[0]


def observe(what, **numbers):
    """Record named numbers (errors, agreement rates) of the running test."""
    OBSERVED.setdefault(_current_test(), {}).setdefault(what or 'value', {}).update(
        {k: (float(v) if v is not None else None) for k, v in numbers.items()})


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + '.npz'))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def assert_close_f32(got, ref, what='', tol=F32_REL):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if ref.numel() == 0:
        return
    err = (got - ref).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    observe(what, max_abs_err=err, bound=bound, max_abs_ref=ref.abs().max().item())
    assert err <= bound, f'{what}: max abs err {err:.3e} > {bound:.3e}'


def assert_close_bf16(got, ref, what='', tol=BF16_ABS, roundings=1, rel_to_max=0.0):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if ref.numel() == 0:
        return
    # `roundings`: how many of the two tensors were themselves rounded to bf16 (each adds half a spacing)
    # `rel_to_max`: extra allowance as a fraction of max |ref|, for sums whose size grows with the problem
    excess = ((got - ref).abs() - roundings * ref.abs() * 2.0 ** -8).max().item() - rel_to_max * ref.abs().max().item()
    observe(what, max_abs_err=(got - ref).abs().max().item(), beyond_spacing=excess, tol=tol,
            max_abs_ref=ref.abs().max().item(), rel_to_max=rel_to_max)
    assert excess <= tol, f'{what}: max abs err beyond bf16 spacing {excess:.3e} > {tol:.1e}'


def selection_agreement(idx_a, mask_a, idx_b, mask_b):
    """Fraction of queries (rows of the last axis) whose masks and sets of visible block indices are identical."""
    ia, ib, ma, mb = idx_a.cpu(), idx_b.cpu(), mask_a.cpu().bool(), mask_b.cpu().bool()
    if ia.numel() == 0:
        return 1.0
    big = int(max(ia.max().item(), ib.max().item())) + 1
    a = torch.where(ma, ia, torch.full_like(ia, big)).sort(dim=-1).values
    b = torch.where(mb, ib, torch.full_like(ib, big)).sort(dim=-1).values
    same = (a == b).all(dim=-1) & (ma.sum(dim=-1) == mb.sum(dim=-1))
    return same.float().mean().item()


def assert_bf16_no_worse_than_reference(got, truth, ref16, what='', tol=BF16_ABS, factor=1.5, rel_to_max=0.0):
    """The bf16 contract against the fp32 truth, or -- for tensors whose inputs were themselves rounded on the way
    (a whole layer: the branches see bf16 q, k, v where the fp32 run sees unrounded ones) -- an error against the
    truth of at most `factor` times the error of the reference's own bf16 run (`ref16`, same weights, same selected
    blocks) plus one bf16 spacing.  Both errors are recorded."""
    got, truth, ref16 = (t.detach().float().cpu() for t in (got, truth, ref16))
    assert got.shape == truth.shape == ref16.shape, (what, got.shape, truth.shape, ref16.shape)
    if truth.numel() == 0:
        return
    top = truth.abs().max().item()
    e_ours = (got - truth).abs().max().item()
    e_ref = (ref16 - truth).abs().max().item()
    beyond = ((got - truth).abs() - truth.abs() * 2.0 ** -8).max().item() - rel_to_max * top
    observe(what, max_abs_err=e_ours, reference_bf16_max_abs_err=e_ref, beyond_spacing=beyond, tol=tol, max_abs_ref=top)
    assert beyond <= tol or e_ours <= factor * e_ref + 2.0 ** -8 * top, \
        f'{what}: max abs err {e_ours:.3e} (beyond bf16 spacing {beyond:.3e} > {tol:.1e}) and above {factor} x the ' \
        f'reference bf16 run\'s own error {e_ref:.3e}'


def agreeing_queries(idx_a, mask_a, idx_b, mask_b):
    """[..., N] bool: the two selections name the same set of visible blocks for the query."""
    ia, ib, ma, mb = idx_a.cpu(), idx_b.cpu(), mask_a.cpu().bool(), mask_b.cpu().bool()
    big = int(max(ia.max().item(), ib.max().item())) + 1
    a = torch.where(ma, ia, torch.full_like(ia, big)).sort(dim=-1).values
    b = torch.where(mb, ib, torch.full_like(ib, big)).sort(dim=-1).values
    return (a == b).all(dim=-1)


def same_selection(idx_a, mask_a, idx_b, mask_b):
    """Selections agree when the masks are identical and, per query, the sets
    of visible block indices are identical (order inside equal values and the
    indices of invisible slots carry no meaning)."""
    if not torch.equal(mask_a.cpu(), mask_b.cpu()):
        return False
    big = idx_a.max().item() + idx_b.max().item() + 1 if idx_a.numel() else 0
    a = torch.where(mask_a.cpu(), idx_a.cpu(), torch.full_like(idx_a.cpu(), big)).sort(dim=-1).values
    b = torch.where(mask_b.cpu(), idx_b.cpu(), torch.full_like(idx_b.cpu(), big)).sort(dim=-1).values
    return torch.equal(a, b)


class Checks:
    """Runs several comparisons to the end and fails once, with every message, so that one run shows all errors."""

    def __init__(self):
        self.failures = []

    def __call__(self, fn, *args, **kw):
        try:
            fn(*args, **kw)
        except AssertionError as e:
            self.failures.append(str(e))

    def done(self):
        assert not self.failures, '; '.join(self.failures)


def free_port():
    """A TCP port nobody listens on right now, for the rendezvous of a test's child processes (a port derived from the
    process id can collide with a socket an earlier run left in TIME_WAIT)."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]
