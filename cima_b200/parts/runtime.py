"""What every part is given when it is built: the kernels, the precision and the device."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch


@dataclass
class Runtime:
    kernels: Any                 # cima_b200.kernels.Kernels (tests may pass a stand-in with the same methods)
    dtype: torch.dtype           # dtype of activations and of the cache: bfloat16 or float32
    device: Any

    @property
    def full_precision(self) -> bool:
        return self.dtype is torch.float32

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and biases live as float32 vectors in both precisions (bf16 -> f32 is exact)."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix on the device: float32 on the 32-bit path; otherwise in the dtype it was kept in
        (bfloat16 or float32), a float16 one as bfloat16."""
        if self.full_precision:
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        if t.dtype is torch.float16:
            return t.to(device=self.device, dtype=torch.bfloat16).contiguous()
        return t.to(device=self.device).contiguous()

    def matrix_rows(self, pieces) -> torch.Tensor:
        """Several matrices of one width stacked by rows into one device matrix (q | k | v, gate | up), each piece
        uploaded into its place: the host never holds the stacked copy.  Pieces kept in different dtypes meet in
        float32, as does everything on the 32-bit path."""
        pieces = list(pieces)
        kept = {torch.bfloat16 if (p.dtype is torch.float16 and not self.full_precision) else p.dtype for p in pieces}
        dtype = torch.float32 if (self.full_precision or len(kept) > 1) else kept.pop()
        rows = sum(p.shape[0] for p in pieces)
        out = torch.empty((rows, pieces[0].shape[1]), dtype=dtype, device=self.device)
        r = 0
        for p in pieces:
            if p.shape[1] != out.shape[1]:
                raise ValueError(f"matrices of widths {p.shape[1]} and {out.shape[1]} cannot be stacked by rows")
            out[r:r + p.shape[0]].copy_(p)
            r += p.shape[0]
        return out
