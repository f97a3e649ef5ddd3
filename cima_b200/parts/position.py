"""Position encodings of a mixer's queries and keys.

``rope``: half-split rotary over the first ``rotary_dim`` dimensions of a head with
inv_freq[i] = theta^(-2i / rotary_dim) (src/kernels.cu:397-414; the reference computes the power in
float32 on the device, here the table is made once in float64 and rounded to float32; the angle,
sine and cosine are float32 on the device).  ``none``: nothing rotates.
A position part offers ``inv_freq`` (float32 [rotary_dim / 2]) and ``rotary_dim``; the attention
mixer hands both to the kernel that rotates and appends.
"""
from __future__ import annotations

import torch

from .registry import register_position


class Rope:
    def __init__(self, spec, rt):
        if spec.rotary_dim % 2 or not (0 <= spec.rotary_dim <= spec.head_dim):
            raise ValueError(f"rope: rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / max(spec.rotary_dim, 1))
        self.inv_freq = inv.to(torch.float32).to(rt.device).contiguous()


class NoPosition:
    def __init__(self, spec, rt):
        self.spec = spec
        self.rotary_dim = 0
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=rt.device)


register_position("rope", Rope)
register_position("none", NoPosition)
