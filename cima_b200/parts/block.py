"""Arrangement of a layer's parts.  ``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/transformer.rs:1024-1319).  The block builds its parts from the spec through the
registries; it does not know which kinds they are, nor which model it is in.

Interface of the parts it holds:
  norm(x) -> h, norm.lazy(x, ssq)   mixer.forward(h, x, batch, cache, site)   (adds into x)
  feed_forward.forward(h, x, batch) (adds into x)
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights.loader import TensorSpec
from .registry import build_feed_forward, build_mixer, build_norm, register_block


class PreNormBlock:
    def __init__(self, spec, layer: int, rt):
        self.spec, self.layer, self.rt = spec, layer, rt
        self.mixer_norm = build_norm(spec.mixer_norm, rt)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        self.ffn_norm = build_norm(spec.ffn_norm, rt)
        self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt)

    def plan(self) -> Dict[str, TensorSpec]:
        s = self.spec
        p: Dict[str, TensorSpec] = {}
        p.update(self.mixer_norm.plan(f"{s.prefix}{s.names['mixer_norm']}.weight"))
        p.update(self.mixer.plan(s.prefix, s.names))
        p.update(self.ffn_norm.plan(f"{s.prefix}{s.names['ffn_norm']}.weight"))
        p.update(self.feed_forward.plan(s.prefix, s.names))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.mixer_norm.load(tensors, f"{s.prefix}{s.names['mixer_norm']}.weight")
        self.mixer.load(tensors, s.prefix, s.names)
        self.ffn_norm.load(tensors, f"{s.prefix}{s.names['ffn_norm']}.weight")
        self.feed_forward.load(tensors, s.prefix, s.names)

    def cache_requests(self, site: int) -> List[object]:
        return list(self.mixer.cache_requests(site))

    def nbytes(self) -> int:
        return self.mixer_norm.nbytes() + self.mixer.nbytes() + self.ffn_norm.nbytes() + self.feed_forward.nbytes()

    def forward(self, x: torch.Tensor, batch, cache, site: int, ssq=None):
        """``ssq``: partial sums of squares of x's rows if the kernel that last wrote x left them (else
        None); the same for the rows as this block leaves them is returned.  A part that declares
        ``takes_pending_norm`` gets the norm as a ``NormedInput`` and may fold it into its first product;
        any other part gets the normalised tensor.  A part that returns nothing invalidates the sums."""
        ssq = self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x, ssq), x, batch, cache, site)
        return self.feed_forward.forward(self._normed(self.ffn_norm, self.feed_forward, x, ssq), x, batch)

    @staticmethod
    def _normed(norm, part, x, ssq):
        if getattr(part, "takes_pending_norm", False) and hasattr(norm, "lazy"):
            return norm.lazy(x, ssq)
        return norm(x)


register_block("prenorm", PreNormBlock)
