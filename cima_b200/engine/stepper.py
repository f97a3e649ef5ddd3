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
    def __init__(self, model, max_batch: int = 64, use_graphs: bool = True):
        self.model = model
        self.use_graphs = use_graphs and torch.device(model.rt.device).type == "cuda"
        self._graphs = {}
        self._armed = None            # (graph, slots) whose device-side inputs are those of the next step
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
        self._armed = None
        self.model.cache.close(slots)

    def prefill(self, slots, prompts, options) -> List[int]:
        self._armed = None
        self.sampler.begin(slots, prompts, options)
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        return self._choose(self.model.step(entries), slots, options, sum(len(p) for p in prompts))

    def decode(self, slots, last_tokens, options) -> List[int]:
        if not self.use_graphs:
            entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, last_tokens)]
            return self._choose(self.model.step(entries), slots, options, len(slots))
        graph = self._arm(slots, last_tokens, options)
        self.reserve_ahead(slots, 1)
        chosen = graph.run()
        out = chosen.tolist()                        # the step's result crosses to the host here
        self._advance_lengths(slots, 1)
        self.d2h_bytes += 4 * len(slots)
        return out

    # ------------------------------------------------------------------ graph plumbing
    def _arm(self, slots, last_tokens, options):
        """The graph for this batch size with its inputs set: uploaded when the set of sequences
        changed, otherwise already there (the last step fed its tokens forward on the device)."""
        cache = self.model.cache
        all_greedy = all(o.greedy for o in options)
        key = (len(slots), all_greedy)
        graph = self._graphs.get(key)
        if graph is None:
            from .graph import DecodeGraph
            graph = self._graphs[key] = DecodeGraph(self.model, self.sampler, len(slots), all_greedy)
        if self._armed != (key, tuple(slots)):
            params = np.array([[o.temperature, float(o.top_k), o.top_p, o.repeat_penalty] for o in options], dtype=np.float32)
            graph.load(slots, last_tokens, [cache.length(s) for s in slots], params)
            self.h2d_bytes += 4 * (6 * len(slots) + 1) + params.nbytes
            self._armed = (key, tuple(slots))
        elif last_tokens is not None:
            graph.feed(last_tokens)
            self.h2d_bytes += 4 * len(slots)
        return graph

    def reserve_ahead(self, slots, steps: int) -> None:
        cache = self.model.cache
        for s in slots:
            cache.reserve(s, cache.length(s) + steps)
        cache.flush()

    def _advance_lengths(self, slots, steps: int) -> None:
        cache = self.model.cache
        for s in slots:
            cache.commit(s, cache.length(s) + steps)

    def decode_on_device(self, slots, last_tokens, options, steps: int) -> torch.Tensor:
        """``steps`` decode steps without a host round trip between them (tokens are fed forward on
        the device); returns the last step's chosen tokens (device).  Used to time the device alone."""
        graph = self._arm(slots, last_tokens, options)
        self.reserve_ahead(slots, steps)
        for _ in range(steps):
            chosen = graph.run()
        self._advance_lengths(slots, steps)
        return chosen

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
