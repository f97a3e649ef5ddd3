"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

Every tensor of the model's plan is drawn from its own generator, seeded by
(seed, tensor name), so a tensor's values depend on nothing else: N(0, 0.02) for
matrices and biases, 1 + N(0, 0.02) for norm weights, stored as bfloat16.  The
reference's stand-in for a checkpoint is ``MockWeights`` (src/selftest.rs:38-83,
:123-158): xorshift values under the real tensor names, in memory only.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


_SLAB = 1 << 24     # elements drawn at a time: bounds the float32 scratch of a large tensor to 64 MiB


def random_tensor(spec: TensorSpec, seed: int, name: str, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    """The tensor ``name`` drawn from the generator seeded by (seed, name), in slabs of ``_SLAB`` values in float32
    that are rounded into ``dtype`` as they come.  On the CPU a slab (a multiple of 16 values) continues the
    generator's sequence exactly where the last one ended, so the values do not depend on the slab size."""
    if spec.init not in ("normal", "ones_normal"):
        raise ValueError(f"unknown init '{spec.init}' for tensor '{name}'")
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    out = torch.empty(spec.shape, dtype=dtype, device=device)
    flat = out.view(-1)
    n = flat.numel()
    scratch = torch.empty(min(n, _SLAB), dtype=torch.float32, device=device)
    for lo in range(0, n, _SLAB):
        part = scratch[:min(_SLAB, n - lo)]
        part.normal_(0.0, spec.std, generator=g)
        if spec.init == "ones_normal":
            part += 1.0
        flat[lo:lo + part.numel()].copy_(part)
    return out


def random_tensors(plan: Dict[str, TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    return {n: random_tensor(s, seed, n, dtype, device) for n, s in plan.items()}


def write_random_model(folder: str, config_dict: dict, plan: Dict[str, TensorSpec], seed: int,
                       dtype=torch.bfloat16) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_dict, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(plan, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
