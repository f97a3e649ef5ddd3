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
import weakref
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


class TensorSource:
    """Tensors by name, fetched one at a time when a part asks for them (``source[name]``), so that loading holds
    one tensor on the host, not one checkpoint.  Counts the bytes of the tensors it handed out that are still alive
    (``live_bytes``) and their highest mark (``peak_bytes``)."""

    def __init__(self):
        self.live_bytes = 0
        self.peak_bytes = 0
        self.fetched: List[str] = []

    def _hand_out(self, name: str, t: torch.Tensor) -> torch.Tensor:
        n = t.numel() * t.element_size()
        self.live_bytes += n
        self.peak_bytes = max(self.peak_bytes, self.live_bytes)
        self.fetched.append(name)
        weakref.finalize(t, self._released, n)
        return t

    def _released(self, n: int) -> None:
        self.live_bytes -= n

    def __contains__(self, name: str) -> bool:
        return name in self.names()

    def names(self) -> List[str]:
        raise NotImplementedError

    def __getitem__(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class CheckpointTensors(TensorSource):
    """The tensors of ``plan`` in a model folder.  Opening checks the whole plan against the files' headers and
    raises ONE ``WeightError``; after that ``source[name]`` reads that tensor from the mapping (the reference uploads
    from its mapping tensor by tensor too, src/formats.rs:1405-1454, src/models/transformer.rs:864-917).
    ``ignore``: glob patterns of names that may be present without being used (a tied model that also stores its
    head, say).  ``optional_prefixes``: prefixes of plan names that a checkpoint may leave out, as the reference
    looks a tensor up under several prefixes (src/models/transformer.rs:472-488): with "model.", a file that stores
    ``layers.0.mlp.up_proj.weight`` serves ``model.layers.0.mlp.up_proj.weight``."""

    def __init__(self, folder: str, plan: Dict[str, TensorSpec], ignore: Iterable[str] = (),
                 optional_prefixes: Iterable[str] = ()):
        super().__init__()
        self.folder = folder
        self._where = open_model_files(folder)
        try:
            where = self._where
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
            self._stored_as = stored_as
        except BaseException:
            self.close()
            raise

    def names(self) -> List[str]:
        return list(self._stored_as)

    def __getitem__(self, name: str) -> torch.Tensor:
        stored = self._stored_as[name]
        return self._hand_out(name, stored_to_kept(self._where[stored][0].read(stored)))

    def close(self) -> None:
        for sf in {id(f): f for f, _ in self._where.values()}.values():
            sf.close()
        self._where = {}


class RandomTensors(TensorSource):
    """The random-weights mode without a folder: ``source[name]`` draws that tensor of ``plan`` from the generator
    seeded by (seed, name), on ``device``.  Drawn on the CPU the values are those that ``write_random_model`` stores;
    drawn on a CUDA device they come from that device's generator (other values, much faster for a large shape).
    The reference's stand-in checkpoint is in memory too and goes through the same build as a file
    (``MockWeights``, src/selftest.rs:23-159)."""

    def __init__(self, plan: Dict[str, TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.plan, self.seed, self.dtype, self.device = plan, int(seed), dtype, device

    def names(self) -> List[str]:
        return list(self.plan)

    def __getitem__(self, name: str) -> torch.Tensor:
        from .random_init import random_tensor
        return self._hand_out(name, random_tensor(self.plan[name], self.seed, name, self.dtype, self.device))


def load_tensors(folder: str, plan: Dict[str, TensorSpec], ignore: Iterable[str] = (),
                 optional_prefixes: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """All tensors of ``plan`` from ``folder`` at once (CPU), keyed by the plan's names: ``CheckpointTensors`` read
    out into a dict, for callers that want the whole checkpoint in memory (tests, tools)."""
    with CheckpointTensors(folder, plan, ignore, optional_prefixes) as src:
        return {n: src[n] for n in plan}
