"""One registry from an architecture's name to what builds its model.

The name is ``architectures[0]`` of config.json (``model_type`` as a second
key).  The reference plays this role with an allowlist of model types and a
closed enum of resident graphs (src/models/transformer.rs:113-153,
src/models/mod.rs:215-275); here it is an open table, so that another
architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .specs import ModelSpec


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str                                   # e.g. "Qwen2ForCausalLM"
    model_type: str                             # e.g. "qwen2"
    parse: Callable[[Dict[str, Any]], Any]      # config.json dict -> typed configuration
    spec: Callable[[Any], ModelSpec]            # typed configuration -> ModelSpec


_BY_NAME: Dict[str, ArchitectureEntry] = {}
_BY_TYPE: Dict[str, ArchitectureEntry] = {}


class UnknownArchitecture(ValueError):
    pass


def register_architecture(entry: ArchitectureEntry) -> None:
    _BY_NAME[entry.name] = entry
    _BY_TYPE[entry.model_type] = entry


def registered_architectures():
    return sorted(_BY_NAME)


def lookup_architecture(raw_config: Dict[str, Any]) -> ArchitectureEntry:
    """The entry for a config.json dict; unknown names fail with the list of known ones."""
    archs = raw_config.get("architectures")
    if isinstance(archs, list):
        for a in archs:
            if a in _BY_NAME:
                return _BY_NAME[a]
    mt = raw_config.get("model_type")
    if mt in _BY_TYPE and not archs:
        return _BY_TYPE[mt]
    raise UnknownArchitecture(
        f"config.json names architectures={archs!r}, model_type={mt!r}; "
        f"registered architectures: {registered_architectures()}")


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except OSError as e:
        raise ValueError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ValueError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise ValueError(f"{path} does not hold a JSON object")
    return raw
