"""Arrangement of a layer's parts.  ``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/transformer.rs:1024-1319).  The block builds its parts from the spec through the
registries; it does not know which kinds they are, nor which model it is in.

Interface of the parts it holds:
  norm(x) -> h, norm.lazy(x, ssq)   mixer.forward(h, x, batch, cache, site[, next_norm=])   (adds into x)
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

    def state(self) -> Dict[str, torch.Tensor]:
        """The layer's tensors by name as they are kept on the device (the inverse of ``load``).  A part offers
        ``state`` with the arguments of its ``plan``; one that does not cannot be written out."""
        s = self.spec
        out: Dict[str, torch.Tensor] = {}
        for part, args in ((self.mixer_norm, (f"{s.prefix}{s.names['mixer_norm']}.weight",)), (self.mixer, (s.prefix, s.names)),
                           (self.ffn_norm, (f"{s.prefix}{s.names['ffn_norm']}.weight",)), (self.feed_forward, (s.prefix, s.names))):
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def scratch_row(self) -> int:
        """Values of the widest activation row that a step holds inside this layer (sizes the memory forecast)."""
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in (self.mixer, self.feed_forward))

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this layer may be recorded as a CUDA graph: every part says so itself
        (``graph_safe = True``: it reads nothing of the batch on the host and keeps its buffers' addresses); a part
        that says nothing is taken as unfit, and the stepper then decodes step by step."""
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward))

    def nbytes(self) -> int:
        return self.mixer_norm.nbytes() + self.mixer.nbytes() + self.ffn_norm.nbytes() + self.feed_forward.nbytes()

    def forward(self, x: torch.Tensor, batch, cache, site: int, info=None, next_norm=None):
        """``info`` (a ``RowsInfo`` or None): what the kernel that last wrote x left behind; the same for the
        rows as this block leaves them is returned.  ``next_norm``: the norm that reads x after this block.
        A part that declares ``takes_pending_norm`` gets its norm as a ``NormedInput`` and may fold it into
        its first product; one that declares ``takes_next_norm`` is told which norm follows it and may produce
        it with its last product.  Any other part gets the normalised tensor, and what it returns is
        ignored."""
        info = self._run(self.mixer, self.mixer_norm, info, self.ffn_norm, x, (batch, cache, site))
        return self._run(self.feed_forward, self.ffn_norm, info, next_norm, x, (batch,))

    @staticmethod
    def _run(part, norm, info, next_norm, x, args):
        if info is not None and getattr(info, "norm", None) is norm and info.h is not None:
            h = info.h                                             # the rows came normalised already
        elif getattr(part, "takes_pending_norm", False) and hasattr(norm, "lazy"):
            ssq = getattr(info, "ssq", None) if info is not None else None
            xw = info.xw if (info is not None and getattr(info, "xw_norm", None) is norm) else None
            h = norm.lazy(x, ssq, xw)
        else:
            h = norm(x)
        if getattr(part, "takes_next_norm", False):
            return part.forward(h, x, *args, next_norm=next_norm)
        part.forward(h, x, *args)
        return None


register_block("prenorm", PreNormBlock)
