"""Whether a model with its cache fits the device, asked before anything is allocated.

The reference forecasts the same three shares (weights, keys and values, scratch) against the free memory
and refuses to load what would not fit (src/models/transformer.rs:318-405, ``VramForecast``).  Here the
figures come from the model's own plan of tensors and from what its mixers ask of the cache, so another
architecture is covered without a change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Sequence

import torch

from ..cache import KVRequest, StateRequest


STEP_ROWS = 16384        # the most rows that run as one step; a step that brings more is run in parts (``Model.step``)


class DoesNotFit(RuntimeError):
    """The weights, the cache and the step's scratch together exceed the device's free memory."""


@dataclass(frozen=True)
class Forecast:
    weights: int          # bytes of the tensors of the plan as they are kept on the device
    cache: int            # bytes of the pages of all groups of layers (and of the per-sequence state)
    scratch: int          # bytes a step of the largest prompt needs for its activations and logits

    @property
    def total(self) -> int:
        return self.weights + self.cache + self.scratch

    def describe(self) -> str:
        g = 1024.0 ** 3
        return (f"weights {self.weights / g:.2f} GiB + cache {self.cache / g:.2f} GiB + scratch {self.scratch / g:.2f} GiB "
                f"= {self.total / g:.2f} GiB")


def forecast(plan: Dict[str, object], requests: Sequence[Sequence[object]], dtype: torch.dtype, max_tokens: int,
             hidden: int, vocab: int, widest: int, page_size: int = 64, shares: Sequence[int] = (),
             extra_state: Sequence[StateRequest] = (), max_seqs: int = 0) -> Forecast:
    """``plan``: name -> TensorSpec (matrices are kept in ``dtype``, vectors in float32).  ``requests[i]``: what
    the mixer at site i asks of the cache.  ``widest``: the widest activation row of a layer (its gated
    intermediate, twice, or its q/k/v row)."""
    elt = 4 if dtype is torch.float32 else 2
    weights = 0
    for spec in plan.values():
        n = 1
        for d in spec.shape:
            n *= int(d)
        weights += n * (elt if len(spec.shape) >= 2 else 4)
    n_pages = -(-max_tokens // page_size)
    n_slots = max(1, min(n_pages, max_seqs if max_seqs else 4096))
    groups: Dict[KVRequest, int] = {}
    state = 0
    for site, reqs in enumerate(requests):
        for r in reqs:
            if isinstance(r, KVRequest):
                if site not in shares:
                    groups[r] = groups.get(r, 0) + 1
            elif isinstance(r, StateRequest):
                state += n_slots * _numel(r.shape) * torch.empty((), dtype=r.dtype).element_size()
    for r in extra_state:
        state += n_slots * _numel(r.shape) * torch.empty((), dtype=r.dtype).element_size()
    cache = state
    for r, sites in groups.items():
        cache += sites * n_pages * 2 * r.n_kv_heads * page_size * r.head_dim * elt
    # a step of the longest prompt: the float32 residual, the widest activation and its input, logits of a batch;
    # and the recorded prompt steps that are kept, each with the activations of its rows
    from .graph import MAX_PROMPT_GRAPHS, recorded_prompt_rows
    row = hidden * 4 + (widest + 2 * hidden) * elt
    rows = min(max_tokens, STEP_ROWS)
    scratch = rows * row + min(n_slots, 256) * vocab * 4 * 2
    scratch += MAX_PROMPT_GRAPHS * min(max_tokens, recorded_prompt_rows(weights, len(requests), elt)) * row
    return Forecast(weights, cache, scratch)


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def check_fit(fc: Forecast, device) -> None:
    """Raise ``DoesNotFit`` when the forecast exceeds the device's free memory (CUDA devices only)."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return
    free, total = torch.cuda.mem_get_info(dev)
    if fc.total > free:
        g = 1024.0 ** 3
        raise DoesNotFit(f"the model does not fit {dev}: {fc.describe()}, but {free / g:.2f} of {total / g:.2f} GiB are free "
                         f"(a smaller --max-seq / max_tokens shrinks the cache)")
