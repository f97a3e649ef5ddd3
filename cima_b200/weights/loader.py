"""Weights by tensor name: a plan of what the model wants, checked against what a folder holds.

The parts of a model declare their tensors (name, shape) in a plan; the loader
reads exactly those from safetensors and raises ONE error that lists every
missing tensor, every unexpected one and every wrong shape.  The reference
reports a missing tensor with the names it tried (src/models/transformer.rs:
490-502) and a shape mismatch with both shapes (:563-572), one at a time; a
missing q/k/v bias is silently "no bias" there (:852-858) and is an error here.

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit (or
64-bit) floating point stays 32-bit, integer tensors become int32.  float16
leaves the loader as it is stored and is settled by the model's precision
(``Runtime.matrix``): bfloat16 on the bfloat16 path, float32 (exactly) on the
32-bit path, which would lose three bits by way of bfloat16.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

from .safetensors_io import open_model_files


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str = "normal"        # random-weights mode: "normal" N(0, std) | "ones_normal" 1 + N(0, std)
    std: float = 0.02


class WeightError(ValueError):
    """Missing, unexpected and misshapen tensors of a checkpoint, all in one message."""

    def __init__(self, folder: str, missing, unexpected, wrong_shape, total: int):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"{folder}: the checkpoint ({total} tensors) does not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: found {list(f)}, expected {list(e)}" for n, f, e in self.wrong_shape))
        super().__init__("\n".join(lines))


def stored_to_kept(t: torch.Tensor) -> torch.Tensor:
    """The dtype rule of the loader (see module docstring)."""
    if t.dtype in (torch.bfloat16, torch.float32, torch.float16):
        return t
    if t.dtype is torch.float64:
        return t.to(torch.float32)
    return t.to(torch.int32)


def tensor_names(folder: str) -> List[str]:
    """Names of all tensors that the folder's safetensors files hold (headers only)."""
    where = open_model_files(folder)
    try:
        return sorted(where)
    finally:
        for sf in {id(f): f for f, _ in where.values()}.values():
            sf.close()


def load_tensors(folder: str, plan: Dict[str, TensorSpec], ignore: Iterable[str] = (),
                 optional_prefixes: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Tensors of ``plan`` from ``folder`` (CPU), keyed by the plan's names.  ``ignore`` holds glob
    patterns of names that may be present without being used (a tied model that also stores its head,
    say).  ``optional_prefixes``: prefixes of plan names that a checkpoint may leave out, as the
    reference looks a tensor up under several prefixes (src/models/transformer.rs:472-488): with
    "model.", a file that stores ``layers.0.mlp.up_proj.weight`` serves ``model.layers.0.mlp.up_proj.weight``."""
    where = open_model_files(folder)
    try:
        ignore, optional_prefixes = list(ignore), list(optional_prefixes)
        stored_as: Dict[str, str] = {}
        for n in plan:
            for cand in [n] + [n[len(p):] for p in optional_prefixes if n.startswith(p)]:
                if cand in where:
                    stored_as[n] = cand
                    break
        used = set(stored_as.values())
        missing: List[str] = [n for n in plan if n not in stored_as]
        unexpected = [n for n in where if n not in used and not any(fnmatch.fnmatch(n, p) for p in ignore)]
        wrong = []
        for n, spec in plan.items():
            if n in stored_as:
                found = where[stored_as[n]][0].tensors[stored_as[n]]["shape"]
                if tuple(found) != tuple(spec.shape):
                    wrong.append((stored_as[n], found, spec.shape))
        if missing or unexpected or wrong:
            raise WeightError(folder, sorted(missing), sorted(unexpected), sorted(wrong), len(where))
        return {n: stored_to_kept(where[stored_as[n]][0].read(stored_as[n])) for n in plan}
    finally:
        for sf in {id(f): f for f, _ in where.values()}.values():
            sf.close()
