"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, computed in float32 from the float32 residual stream
(src/kernels.cu:37-50).  ``size`` and ``eps`` come from the spec."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from .registry import register_norm


class RowsInfo:
    """What the kernel that last wrote the residual rows left behind, handed from part to part:
    ``ssq`` - partial sums of squares of the rows [rows, parts] (a skinny product can fold the next norm in),
    with ``xw`` = bf16(rows * weight of ``xw_norm``) when the writer knew which norm follows;
    ``norm`` / ``h`` - the rows already normalised with that norm (the residual add and the norm ran as one)."""

    def __init__(self, ssq=None, norm=None, h=None, xw=None, xw_norm=None):
        self.ssq, self.norm, self.h = ssq, norm, h
        self.xw, self.xw_norm = xw, xw_norm       # rows times the weight of ``xw_norm``, bf16 (goes with ssq)


class NormedInput:
    """RMSNorm(x) not yet computed.  A product that can fold the norm in (few rows, bf16) takes ``xw``
    (bf16(x * weight)) and ``ssq`` (partial sums of squares of x's rows), both left by the kernel that
    wrote the rows; everything else calls ``tensor()`` and gets the normalised activations."""

    def __init__(self, norm: "RMSNorm", x: torch.Tensor, ssq, xw=None):
        self.norm, self.x, self.ssq, self.xw = norm, x, ssq, xw
        self._h = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self) -> torch.Tensor:
        if self._h is None:
            self._h = self.norm(self.x)
        return self._h


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

    def state(self, name: str) -> Dict[str, torch.Tensor]:
        return {name: self.weight}

    graph_safe = True

    def lazy(self, x: torch.Tensor, ssq=None, xw=None) -> NormedInput:
        return NormedInput(self, x, ssq, xw)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(*x.shape)
        self.rt.kernels.rmsnorm(x, self.weight, self.spec.eps, out)
        return out


register_norm("rmsnorm", RMSNorm)
