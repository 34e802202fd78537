"""Rotary position embedding used in front of the selected and sliding
branches (upstream call sites NSA:238, NSA:643).  Convention: inverse
frequency theta^(-2m/d) on the adjacent feature pair (2m, 2m+1), angles in
fp32, result in the input dtype.  Plain PyTorch: it produces inputs of the
hot path and is not part of it."""
import torch
from torch import nn


class RotaryEmbedding(nn.Module):
    def __init__(self, dim, theta=10000.0):
        super().__init__()
        self.register_buffer('inv_freq', theta ** (-torch.arange(0, dim, 2).float() / dim), persistent=False)

    def rotate_queries_or_keys(self, t, offset=0):
        n = t.shape[-2]
        pos = torch.arange(n, device=t.device, dtype=torch.float32) + offset
        ang = pos[:, None] * self.inv_freq.to(t.device)[None, :]
        cos = ang.cos().repeat_interleave(2, dim=-1)
        sin = ang.sin().repeat_interleave(2, dim=-1)
        x = t.float()
        even, odd = x[..., 0::2], x[..., 1::2]
        rotated = torch.stack((-odd, even), dim=-1).flatten(-2)
        return (x * cos + rotated * sin).to(t.dtype)

    def rotate_queries_with_cached_keys(self, q, k):
        nq, nk = q.shape[-2], k.shape[-2]
        return self.rotate_queries_or_keys(q, offset=nk - nq), self.rotate_queries_or_keys(k)
