"""The generation loop: requests in, tokens out, as many batches one after another as it takes.

The loop is host logic only.  It talks to a *stepper* (``ModelStepper`` for a real model; tests use a
scripted one) through four calls: ``open``, ``prefill``, ``decode``, ``close``.  Its decisions follow the
reference's loop for one sequence (src/models/mod.rs:972-1405), applied to every sequence of a batch:

* a prompt that leaves fewer than 16 positions is cut to its first token plus its newest tail
  (:987-1010);
* budget = min(max_tokens, positions - prompt length) (:1145-1147);
* a sampled stop token ends the sequence with reason "stop" and is neither emitted nor counted,
  unless ``ignore_eos`` (:1262-1269); an exhausted budget ends it with reason "length";
* sequences that end leave the batch, the others go on; when all have ended the batch's slots are
  given back and the next batch starts.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Protocol, Sequence, Union

from ..sampling.options import GenOptions

RESERVED_FOR_ANSWER = 16


@dataclass
class GenResult:
    tokens: List[int]
    finish_reason: str                # "stop" | "length"
    prompt_tokens: int
    truncated: bool = False


@dataclass
class GenStats:
    """Counts and times of one ``generate`` call (the reference's GenStats, src/models/transformer.rs:1791-1806)."""
    prompt_tokens: int = 0
    gen_tokens: int = 0
    batches: int = 0
    reused_tokens: int = 0            # prompt tokens that were not run: their keys were still in the cache
    prefill_s: float = 0.0
    decode_s: float = 0.0
    decode_steps: int = 0

    @property
    def decode_tok_per_s(self) -> float:
        return self.gen_tokens / self.decode_s if self.decode_s > 0 else 0.0


class Stepper(Protocol):
    """What the loop needs of a stepper.  One that keeps finished sequences for later prompts also has
    ``retain_limit`` (> 0), ``adopt(prompts) -> [(slot | None, tokens in common)]``, ``make_room(needs, slots)``,
    ``retain(slots, histories)`` and takes ``prefill(..., reused=[...])`` (see ``ModelStepper``); the loop uses them
    only when ``retain_limit`` is positive."""
    max_batch: int                    # most sequences in one batch
    max_position: int                 # most positions a sequence may hold
    cache_tokens: int                 # positions the cache holds in all
    page_size: int

    def open(self, count: int) -> List[int]: ...
    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], options: Sequence[GenOptions]) -> List[int]: ...
    def decode(self, slots: Sequence[int], last_tokens: Sequence[int], options: Sequence[GenOptions]) -> List[int]: ...
    def close(self, slots: Sequence[int]) -> None: ...


def fit_prompt(prompt: Sequence[int], max_position: int):
    """(tokens, truncated): the prompt, cut if it would leave fewer than 16 positions."""
    prompt = list(prompt)
    if not prompt:
        raise ValueError("a prompt needs at least one token")
    if len(prompt) + RESERVED_FOR_ANSWER > max_position:
        keep = max(max_position - RESERVED_FOR_ANSWER, 2)
        if keep < len(prompt):
            return [prompt[0]] + prompt[len(prompt) - (keep - 1):], True
    return prompt, False


def plan_batches(needs: Sequence[int], max_batch: int, cache_tokens: int, page_size: int) -> List[List[int]]:
    """Requests (by index, in order) packed into batches: at most ``max_batch`` each, and the
    positions each may come to hold (``needs``), rounded up to pages, within the cache."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, need in enumerate(needs):
        pages = -(-need // page_size) * page_size
        if pages > cache_tokens:
            raise ValueError(f"request {i} may hold {need} positions; the cache holds {cache_tokens}")
        if cur and (len(cur) >= max_batch or used + pages > cache_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += pages
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    def __init__(self, stepper: Stepper, eos_ids: Sequence[int] = ()):
        self.stepper = stepper
        self.eos_ids = tuple(eos_ids)
        self.stats = GenStats()
        self._on_token = None

    def generate(self, prompts: Sequence[Sequence[int]],
                 options: Union[GenOptions, Sequence[GenOptions], None] = None,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenResult]:
        """``on_token(i, token)`` is called for every token of request ``i`` as soon as the step that made it is
        read, in the order of the requests within a step (the reference hands each token's text to its
        ``on_token`` as it is generated, src/models/mod.rs:977, :1307); a stop token is not reported."""
        st = self.stepper
        self._on_token = on_token
        n = len(prompts)
        if options is None:
            options = GenOptions()
        opts: List[GenOptions] = [options] * n if isinstance(options, GenOptions) else list(options)
        if len(opts) != n:
            raise ValueError(f"{len(opts)} option sets for {n} prompts")
        fitted = [fit_prompt(p, st.max_position) for p in prompts]
        budgets = [min(o.max_tokens, st.max_position - len(p)) for (p, _), o in zip(fitted, opts)]
        results: List[Optional[GenResult]] = [None] * n
        self.stats = GenStats()
        # a request with no budget produces nothing and needs no step
        todo = []
        for i in range(n):
            if budgets[i] <= 0:
                results[i] = GenResult([], "length", len(fitted[i][0]), fitted[i][1])
            else:
                todo.append(i)
        needs = [len(fitted[i][0]) + budgets[i] for i in todo]
        for batch in plan_batches(needs, st.max_batch, st.cache_tokens, st.page_size):
            self._run_batch([todo[j] for j in batch], fitted, budgets, opts, results)
        return results  # type: ignore[return-value]

    def _run_batch(self, ids, fitted, budgets, opts, results) -> None:
        st = self.stepper
        prompts = [fitted[i][0] for i in ids]
        # a stepper that keeps finished sequences offers them to prompts that begin alike
        keeps = getattr(st, "retain_limit", 0) > 0
        taken = st.adopt(prompts) if keeps else [(None, 0)] * len(ids)
        reused = [n for _, n in taken]
        slots: List[int] = [s for s, _ in taken if s is not None]
        done = False
        try:
            if keeps:
                st.make_room([len(p) + budgets[i] for p, i in zip(prompts, ids)], [s for s, _ in taken])
            fresh = iter(st.open(sum(1 for s, _ in taken if s is None)))
            slots = [s if s is not None else next(fresh) for s, _ in taken]
            self.stats.batches += 1
            stops = [set(self.eos_ids) | set(opts[i].stop) for i in ids]
            out: List[List[int]] = [[] for _ in ids]
            t0 = time.perf_counter()
            if any(reused):
                tokens = st.prefill(slots, prompts, [opts[i] for i in ids], reused=reused)
            else:
                tokens = st.prefill(slots, prompts, [opts[i] for i in ids])
            self.stats.prefill_s += time.perf_counter() - t0
            self.stats.prompt_tokens += sum(len(p) for p in prompts)
            self.stats.reused_tokens += sum(reused)
            live = list(range(len(ids)))
            while True:
                nxt = []
                for j, t in zip(live, tokens):
                    i = ids[j]
                    if t in stops[j] and not opts[i].ignore_eos:
                        results[i] = GenResult(out[j], "stop", len(prompts[j]), fitted[i][1])
                        continue
                    out[j].append(int(t))
                    if self._on_token is not None:
                        self._on_token(i, int(t))
                    if len(out[j]) >= budgets[i]:
                        results[i] = GenResult(out[j], "length", len(prompts[j]), fitted[i][1])
                        continue
                    nxt.append(j)
                live = nxt
                if not live:
                    break
                t0 = time.perf_counter()
                tokens = st.decode([slots[j] for j in live], [out[j][-1] for j in live], [opts[ids[j]] for j in live])
                self.stats.decode_s += time.perf_counter() - t0
                self.stats.decode_steps += 1
            self.stats.gen_tokens += sum(len(o) for o in out)
            if keeps:
                st.retain(slots, [list(p) + o for p, o in zip(prompts, out)])
                done = True
        finally:
            if not done:
                st.close(slots)
