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


def random_tensor(spec: TensorSpec, seed: int, name: str, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    # large tensors are drawn in slabs to bound the float32 scratch
    t.normal_(0.0, spec.std, generator=g)
    if spec.init == "ones_normal":
        t += 1.0
    elif spec.init != "normal":
        raise ValueError(f"unknown init '{spec.init}' for tensor '{name}'")
    return t.to(dtype)


def random_tensors(plan: Dict[str, TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    return {n: random_tensor(s, seed, n, dtype, device) for n, s in plan.items()}


def write_random_model(folder: str, config_dict: dict, plan: Dict[str, TensorSpec], seed: int,
                       dtype=torch.bfloat16) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_dict, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(plan, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
