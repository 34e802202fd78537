"""Stand-in for `rotary_embedding_torch.RotaryEmbedding`, used only when
importing the upstream library in the fixture-generation script.  Standard
rotary embedding: inverse frequencies 10000^(-2m/d), the angle applied to the
adjacent feature pair (2m, 2m+1), angles in fp32, result in the input dtype."""
import torch
from torch import nn


class RotaryEmbedding(nn.Module):
    def __init__(self, dim, theta=10000.0, **kwargs):
        super().__init__()
        inv_freq = theta ** (-torch.arange(0, dim, 2).float() / dim)
        self.register_buffer('inv_freq', inv_freq, persistent=False)

    def _rotate(self, t, positions):
        ang = positions.float()[:, None] * self.inv_freq[None, :].to(t.device)
        cos = ang.cos().repeat_interleave(2, dim=-1)
        sin = ang.sin().repeat_interleave(2, dim=-1)
        x = t.float()
        x1, x2 = x[..., 0::2], x[..., 1::2]
        rot = torch.stack((-x2, x1), dim=-1).flatten(-2)
        return (x * cos + rot * sin).to(t.dtype)

    def rotate_queries_or_keys(self, t, offset=0):
        n = t.shape[-2]
        return self._rotate(t, torch.arange(n, device=t.device) + offset)

    def rotate_queries_with_cached_keys(self, q, k):
        nq, nk = q.shape[-2], k.shape[-2]
        q = self.rotate_queries_or_keys(q, offset=nk - nq)
        k = self.rotate_queries_or_keys(k)
        return q, k
