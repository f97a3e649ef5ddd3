"""Gated feed-forward: x += (act(h Wg^T) * (h Wu^T)) Wd^T in float32, act by the spec's ``activation``: SiLU
g / (1 + exp(-g)) as the reference has it (src/kernels.cu:81-84; src/models/transformer.rs:1219-1229 and
:1273-1291), or one of the other entries of ``kernels.ACTIVATIONS`` (tanh or erf GELU, ReLU), which every kernel
that applies the activation takes as a parameter.  Rows are independent, so a long step is cut into row chunks
that bound the [rows, 2I] scratch."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from .linear import GatedLinearPair, Linear
from .registry import register_feed_forward

_SCRATCH_ELEMS = 1 << 29          # elements of the [rows, 2I] gate|up scratch per chunk


class GatedMLP:
    def __init__(self, spec, layer: int, rt):
        from ..kernels import ACTIVATIONS
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"gated_mlp: activation '{spec.activation}' is not one of {sorted(ACTIVATIONS)}")
        if spec.bias:
            raise ValueError("gated_mlp: biases are not implemented")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.gate_up = None
        self.down = None

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        return {f"{prefix}{names['gate']}.weight": TensorSpec((s.intermediate, s.hidden)),
                f"{prefix}{names['up']}.weight": TensorSpec((s.intermediate, s.hidden)),
                f"{prefix}{names['down']}.weight": TensorSpec((s.hidden, s.intermediate))}

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str, names: Dict[str, str]) -> None:
        self.gate_up = GatedLinearPair(tensors[f"{prefix}{names['gate']}.weight"],
                                       tensors[f"{prefix}{names['up']}.weight"], self.rt, self.spec.activation)
        self.down = Linear(tensors[f"{prefix}{names['down']}.weight"], None, self.rt)

    def nbytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        w, I = self.gate_up.lin.weight, self.spec.intermediate
        return {f"{prefix}{names['gate']}.weight": w[:I], f"{prefix}{names['up']}.weight": w[I:],
                f"{prefix}{names['down']}.weight": self.down.weight}

    def scratch_row(self) -> int:
        return 2 * self.spec.intermediate

    graph_safe = True

    takes_pending_norm = True
    takes_next_norm = True

    def forward(self, h, x: torch.Tensor, batch, next_norm=None):
        rows = h.shape[0]
        chunk = max(64, _SCRATCH_ELEMS // (2 * self.spec.intermediate))
        chunk -= chunk % 256 if chunk >= 256 else 0          # whole row tiles for the tensor-core product
        if rows <= chunk:
            return self.down.accumulate(self.gate_up.activated(h), x, next_norm)
        if hasattr(h, "tensor"):
            h = h.tensor()
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            self.down.accumulate(self.gate_up.activated(h[r0:r1]), x[r0:r1])
        return None


register_feed_forward("gated_mlp", GatedMLP)
