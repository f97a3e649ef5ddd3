"""Descriptions of a model as data: one spec per part, one per block, one per model.

An architecture's typed configuration (``qwen2.py``) turns its ``config.json``
keys into these specs; the parts (``cima_b200/parts``) are built from them and
know nothing else about the model they sit in.  Every size and constant is a
field here; none stands in the parts' code.

``kind`` selects the implementation from the part registries
(``cima_b200/parts/registry.py``); ``params`` carries what a kind needs beyond
the common fields, so that a kind defined outside the package needs no change
to these classes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str                    # "rmsnorm"
    size: int
    eps: float
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class PositionSpec:
    kind: str                    # "rope" | "none"
    head_dim: int
    rotary_dim: int              # how many leading dims of a head rotate (<= head_dim, even)
    theta: float
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class MixerSpec:
    """Only ``kind`` and ``hidden`` are every mixer's; the fields after them describe an attention and keep their
    defaults for a mixer that has no heads (a recurrence, a convolution), which puts its own sizes in ``params``."""
    kind: str                    # "attention"
    hidden: int
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    window: int = 0              # 0 = every earlier key; w > 0 = the last w keys
    scale: float = 0.0           # factor of q.k before the softmax
    position: Optional[PositionSpec] = None
    # Site (index into ModelSpec.schedule) whose keys and values this layer reads instead of
    # writing its own; None = own cache.
    cache_from: Optional[int] = None
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                    # "gated_mlp"
    hidden: int
    intermediate: int
    activation: str              # "silu"
    bias: bool = False
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    kind: str                    # "prenorm": x += mixer(norm(x)); x += ffn(norm(x))
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    ffn_norm: NormSpec
    prefix: str                  # tensor-name prefix of the layer, e.g. "model.layers.3."
    # tensor-name stems under the prefix, owned by the architecture's naming
    names: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    hidden: int
    max_position: int
    layers: List[BlockSpec]
    # The order in which layers run: indices into ``layers``.  A layer may be named
    # twice; default is each layer once, in order.
    schedule: List[int]
    final_norm: NormSpec
    tie_head: bool
    embed_name: str
    final_norm_name: str
    head_name: str
    embed_scale: float = 1.0
    # A checkpoint of an untied model that stores no head tensor: the table serves as the head
    # (the reference decides so, src/models/transformer.rs:810, and warns, :839-841).
    head_may_be_absent: bool = False
    # Prefixes of the tensor names above that a checkpoint may leave out (a bare backbone stores
    # "layers.0..." for "model.layers.0..."; the reference tries both, src/models/transformer.rs:472-488).
    optional_prefixes: Tuple[str, ...] = ()

    def describe(self) -> str:
        kinds = [f"{self.layers[i].mixer.kind}"
                 f"{'(w=%d)' % self.layers[i].mixer.window if self.layers[i].mixer.window else ''}"
                 f"+{self.layers[i].feed_forward.kind}" for i in self.schedule]
        return (f"{self.architecture}: vocab {self.vocab}, hidden {self.hidden}, "
                f"{len(self.layers)} layers, schedule {kinds}")
