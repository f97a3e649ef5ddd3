"""Registries of part kinds: a spec's ``kind`` names the class that is built from it.

A kind is added with one ``register_*`` call, from inside or outside this package; the blocks and
the model look parts up here and nowhere else, so a new mixer, feed-forward, norm, position
encoding or block arrangement needs no change to existing files.
"""
from __future__ import annotations

from typing import Callable, Dict

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def _register(family: str, kind: str, factory: Callable) -> None:
    _REGISTRIES[family][kind] = factory


def _build(family: str, kind: str, *args, **kwargs):
    table = _REGISTRIES[family]
    if kind not in table:
        raise KeyError(f"no {family} of kind '{kind}' is registered (known: {sorted(table)})")
    return table[kind](*args, **kwargs)


def register_mixer(kind: str, factory: Callable) -> None: _register("mixer", kind, factory)
def register_feed_forward(kind: str, factory: Callable) -> None: _register("feed_forward", kind, factory)
def register_norm(kind: str, factory: Callable) -> None: _register("norm", kind, factory)
def register_position(kind: str, factory: Callable) -> None: _register("position", kind, factory)
def register_block(kind: str, factory: Callable) -> None: _register("block", kind, factory)


def build_mixer(spec, layer: int, rt): return _build("mixer", spec.kind, spec, layer, rt)
def build_feed_forward(spec, layer: int, rt): return _build("feed_forward", spec.kind, spec, layer, rt)
def build_norm(spec, rt): return _build("norm", spec.kind, spec, rt)
def build_position(spec, rt): return _build("position", spec.kind, spec, rt)
def build_block(spec, layer: int, rt): return _build("block", spec.kind, spec, layer, rt)


def registered(family: str):
    return sorted(_REGISTRIES[family])
