"""Stand-in for `local_attention.LocalAttention`, used only when importing the
upstream library in the fixture-generation script.  Exact-window attention
written densely: a causal query i sees keys j with 0 <= i - j <= window_size,
a non-causal one sees |i - j| <= window_size."""
import torch
from torch import nn


class LocalAttention(nn.Module):
    def __init__(self, dim, window_size, causal=False, exact_windowsize=True,
                 autopad=True, use_rotary_pos_emb=False, **kwargs):
        super().__init__()
        assert exact_windowsize and not use_rotary_pos_emb
        self.scale = dim ** -0.5
        self.window_size = window_size
        self.causal = causal

    def forward(self, q, k, v):
        n = q.shape[-2]
        pos = torch.arange(n, device=q.device)
        dist = pos[:, None] - pos[None, :]
        visible = dist <= self.window_size
        visible &= dist >= (0 if self.causal else -self.window_size)
        sim = torch.einsum('...id,...jd->...ij', q, k) * self.scale
        sim = sim.masked_fill(~visible, -torch.finfo(sim.dtype).max)
        return torch.einsum('...ij,...jd->...id', sim.softmax(dim=-1), v)
