"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, computed in float32 from the float32 residual stream
(src/kernels.cu:37-50).  ``size`` and ``eps`` come from the spec."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from .registry import register_norm


class RMSNorm:
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.weight = None

    def plan(self, name: str) -> Dict[str, TensorSpec]:
        return {name: TensorSpec((self.spec.size,), init="ones_normal")}

    def load(self, tensors: Dict[str, torch.Tensor], name: str) -> None:
        self.weight = self.rt.vector(tensors[name])

    def nbytes(self) -> int:
        return self.weight.numel() * 4

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(*x.shape)
        self.rt.kernels.rmsnorm(x, self.weight, self.spec.eps, out)
        return out


register_norm("rmsnorm", RMSNorm)
