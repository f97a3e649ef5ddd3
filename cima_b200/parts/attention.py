"""Grouped-query causal attention over the paged cache, with optional window.

forward: qkv = h Wqkv^T + b  ->  rotate q, k and append k, v to the layer's pages  ->
attention (prefill: over the step's own keys; decode: over the cache)  ->  x += att Wo^T.
Formulas and order as the reference's layer loop, steps 2-7 (src/models/transformer.rs:1039-1264):
bias before rotation, rotation before caching, scale = spec.scale, head h reads kv head
h / (heads / kv_heads), no output bias unless the spec says so.

Every size (heads, kv heads, head_dim, window, scale, bias flags) is a field of the spec.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import build_position, register_mixer


class Attention:
    def __init__(self, spec, layer: int, rt):
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 16, at most 256")
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} heads are not a multiple of {spec.n_kv_heads} kv heads")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.position = build_position(spec.position, rt)
        self.qd = spec.n_heads * spec.head_dim
        self.kvd = spec.n_kv_heads * spec.head_dim
        self.qkv = None
        self.out = None

    # ------------------------------------------------------------------ weights
    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        p: Dict[str, TensorSpec] = {}
        for key, rows in (("q", self.qd), ("k", self.kvd), ("v", self.kvd)):
            p[f"{prefix}{names[key]}.weight"] = TensorSpec((rows, s.hidden))
            if s.qkv_bias:
                p[f"{prefix}{names[key]}.bias"] = TensorSpec((rows,))
        p[f"{prefix}{names['o']}.weight"] = TensorSpec((s.hidden, self.qd))
        if s.out_bias:
            p[f"{prefix}{names['o']}.bias"] = TensorSpec((s.hidden,))
        return p

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str, names: Dict[str, str]) -> None:
        s = self.spec
        bias = None
        if s.qkv_bias:
            bias = torch.cat([tensors[f"{prefix}{names[k]}.bias"].float() for k in ("q", "k", "v")])
        self.qkv = Linear([tensors[f"{prefix}{names[k]}.weight"] for k in ("q", "k", "v")], bias, self.rt)
        ob = tensors[f"{prefix}{names['o']}.bias"] if s.out_bias else None
        self.out = Linear(tensors[f"{prefix}{names['o']}.weight"], ob, self.rt)

    def nbytes(self) -> int:
        return self.qkv.nbytes() + self.out.nbytes()

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        """The tensors of ``plan`` back out of the stacked matrices, as they are kept on the device."""
        out: Dict[str, torch.Tensor] = {}
        r = 0
        for key, rows in (("q", self.qd), ("k", self.kvd), ("v", self.kvd)):
            out[f"{prefix}{names[key]}.weight"] = self.qkv.weight[r:r + rows]
            if self.qkv.bias is not None:
                out[f"{prefix}{names[key]}.bias"] = self.qkv.bias[r:r + rows]
            r += rows
        out[f"{prefix}{names['o']}.weight"] = self.out.weight
        if self.out.bias is not None:
            out[f"{prefix}{names['o']}.bias"] = self.out.bias
        return out

    def scratch_row(self) -> int:
        """Values of the widest activation row a step of this part holds (its q | k | v row)."""
        return self.qd + 2 * self.kvd

    graph_safe = True              # a decode step reads nothing of the batch on the host

    @property
    def short_context(self) -> int:
        """Positions up to which this mixer's decode kernel takes another road than for long contexts (none if 0):
        the stepper records decode steps for such contexts apart (``StepBatch.max_len`` is their bound)."""
        from ..kernels import short_context
        return short_context(self.spec.head_dim)

    # ------------------------------------------------------------------ cache
    def cache_requests(self, site: int) -> List[object]:
        if self.spec.cache_from is not None:
            return []
        return [KVRequest(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window)]

    # ------------------------------------------------------------------ step
    takes_pending_norm = True      # h may be a NormedInput: the q/k/v product folds the norm in when it can
    takes_next_norm = True         # forward(..., next_norm=): the norm that will read x next, for its last product

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        s, K_ = self.spec, self.rt.kernels
        kv = cache.layer_kv(site)
        writes = s.cache_from is None
        rows = h.shape[0]
        if (not batch.prefill and writes and self.qkv._skinny(rows) and kv.storage.dtype is torch.bfloat16
                and self.position.rotary_dim == s.head_dim and hasattr(K_, "qkv_rope")):
            # decoding: projection, rotation and the append to the cache as one kernel
            qkv = self.rt.empty(rows, self.qd + 2 * self.kvd)
            if self.qkv._folds(h, rows):
                K_.qkv_rope(h.xw, self.qkv.weight, self.qkv.bias, qkv, self.position.inv_freq, batch.row_pos,
                            batch.row_seq, batch.seq_slot, kv, s.n_heads, s.n_kv_heads, s.head_dim,
                            norm=(h.ssq, h.norm.spec.eps))
            else:
                K_.qkv_rope(h.tensor() if hasattr(h, "tensor") else h, self.qkv.weight, self.qkv.bias, qkv,
                            self.position.inv_freq, batch.row_pos, batch.row_seq, batch.seq_slot, kv, s.n_heads,
                            s.n_kv_heads, s.head_dim)
        else:
            qkv = self.qkv.store(h)
            K_.rope_append(qkv, self.position.inv_freq, self.position.rotary_dim, batch.row_pos, batch.row_seq,
                           batch.seq_slot, batch.seq_len, kv if writes else None, s.n_heads, s.n_kv_heads, s.head_dim)
        att = self.rt.empty(h.shape[0], self.qd)
        from_cache = (not batch.prefill) or not writes
        K_.attention(qkv, kv, batch, att, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, from_cache,
                     after_append=True)
        return self.out.accumulate(att, x, next_norm)


register_mixer("attention", Attention)
