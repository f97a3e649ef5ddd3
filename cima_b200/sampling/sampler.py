"""The sampler's per-sequence state in the cache's state area, and the call of the device chain.

State per slot: the xorshift64* state, the ring of the last 64 tokens of the sequence's history
(prompt included, as the reference's ``history`` starts as a copy of the prompt,
src/models/mod.rs:1128) and the count of tokens pushed.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..cache.kv import StateRequest
from .options import GenOptions

RING = 64
_MASK = (1 << 64) - 1


def sampler_state() -> List[StateRequest]:
    return [StateRequest("sampler.rng", (1,), torch.int64),
            StateRequest("sampler.ring", (RING,), torch.int32),
            StateRequest("sampler.count", (1,), torch.int32)]


class DeviceSampler:
    def __init__(self, model, max_rows: int = 0):
        """``max_rows``: the most rows one call will bring (the largest batch); the scratch is sized for it at the
        first call, so that a captured decode step and later, larger batches share one buffer."""
        self.model = model
        self.max_rows = max(0, int(max_rows))
        self._retired = []
        self.kernels = model.rt.kernels
        st = model.cache.state
        self.rng, self.ring, self.count = st["sampler.rng"], st["sampler.ring"], st["sampler.count"]
        self._work = None

    def begin(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], options: Sequence[GenOptions]) -> None:
        """Seed the slots' generators and fill their rings with the prompts' tails."""
        n = len(slots)
        rng = np.zeros((n, 1), dtype=np.int64)
        ring = np.zeros((n, RING), dtype=np.int32)
        count = np.zeros((n, 1), dtype=np.int32)
        for i, (p, o) in enumerate(zip(prompts, options)):
            state = max(int(o.seed), 1) & _MASK
            rng[i, 0] = np.array(state, dtype=np.uint64).astype(np.int64)
            tail = list(p)[-RING:]
            # the ring is indexed by (tokens pushed so far) % 64
            total = len(p)
            for j, t in enumerate(tail):
                ring[i, (total - len(tail) + j) % RING] = t
            count[i, 0] = total
        dev = self.rng.device
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=dev)
        self.rng.index_copy_(0, idx, torch.from_numpy(rng).to(dev))
        self.ring.index_copy_(0, idx, torch.from_numpy(ring).to(dev))
        self.count.index_copy_(0, idx, torch.from_numpy(count).to(dev))

    @staticmethod
    def params(options: Sequence[GenOptions], device) -> torch.Tensor:
        p = np.array([[o.temperature, float(o.top_k), o.top_p, o.repeat_penalty] for o in options], dtype=np.float32)
        return torch.from_numpy(p).to(device)

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, params: torch.Tensor,
               tokens: torch.Tensor, all_greedy: bool) -> None:
        """tokens[i] = the choice for row i of ``logits``; the choice is pushed to the slot's history."""
        n, V = logits.shape
        if all_greedy:
            self.kernels.sample(logits, row_slot, params, self.rng, self.ring, self.count, None, tokens, True)
            return
        if self._work is None or self._work.shape[0] < n or self._work.shape[1] != V:
            if self._work is not None:
                self._retired.append(self._work)      # a captured step may still write there: kept, not freed
            self._work = torch.empty((max(n, self.max_rows, 1), V), dtype=torch.float32, device=logits.device)
        self.kernels.sample(logits, row_slot, params, self.rng, self.ring, self.count, self._work, tokens, all_greedy)
