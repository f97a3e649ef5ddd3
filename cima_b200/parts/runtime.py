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
