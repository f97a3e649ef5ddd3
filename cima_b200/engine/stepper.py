"""The stepper the generation loop drives for a real model: the model's step function, then the
device sampler on the wanted logits; tokens cross to the host once per step."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..sampling.options import GenOptions
from ..sampling.sampler import DeviceSampler
from .batch import StepEntry


class ModelStepper:
    def __init__(self, model, max_batch: int = 64):
        self.model = model
        self.sampler = DeviceSampler(model)
        cache = model.cache
        self.max_batch = max(1, min(max_batch, cache.n_slots))
        self.max_position = min(model.spec.max_position, cache.max_tokens)
        self.cache_tokens = cache.max_tokens
        self.page_size = cache.page_size
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def open(self, count: int) -> List[int]:
        return self.model.cache.open(count)

    def close(self, slots: Sequence[int]) -> None:
        self.model.cache.close(slots)

    def prefill(self, slots, prompts, options) -> List[int]:
        self.sampler.begin(slots, prompts, options)
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        return self._choose(self.model.step(entries), slots, options, sum(len(p) for p in prompts))

    def decode(self, slots, last_tokens, options) -> List[int]:
        entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, last_tokens)]
        return self._choose(self.model.step(entries), slots, options, len(slots))

    def _choose(self, logits: torch.Tensor, slots, options: Sequence[GenOptions], tokens_in: int) -> List[int]:
        dev = logits.device
        n = len(slots)
        all_greedy = all(o.greedy for o in options)
        tokens = torch.empty(n, dtype=torch.int32, device=dev)
        if all_greedy:
            self.sampler.sample(logits, None, None, tokens, True)
        else:
            row_slot = torch.from_numpy(np.asarray(slots, dtype=np.int32)).to(dev)
            self.sampler.sample(logits, row_slot, DeviceSampler.params(options, dev), tokens, False)
        self.h2d_bytes += 4 * (3 * tokens_in + 3 * n + 1 + n)
        self.d2h_bytes += 4 * n
        return tokens.tolist()
