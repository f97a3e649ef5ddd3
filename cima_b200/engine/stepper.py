"""The stepper the generation loop drives for a real model: the model's step function, then the
device sampler on the wanted logits; tokens cross to the host once per step."""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import CacheFull
from ..cache.kv import CapacityError
from ..sampling.options import GenOptions
from ..sampling.sampler import DeviceSampler
from .batch import StepEntry
from .graph import MAX_PROMPT_GRAPHS


MIN_REUSE = 16     # a finished sequence is taken up again only for at least this many tokens in common


class ModelStepper:
    def __init__(self, model, max_batch: int = 64, use_graphs: bool = True, pipeline: bool = True, retain: int = 0):
        self.model = model
        # Run-ahead queues a step that a sequence may turn out not to need.  Keys and values written so are simply
        # beyond the sequence's end; state of fixed size that a mixer keeps per sequence would have taken one token
        # too many, so a model with such state decodes without run-ahead.
        self.pipeline = pipeline and not model.cache.has_mixer_state
        # Finished sequences whose keys and values stay in the cache (slot -> the tokens they stand for), newest
        # last, at most ``retain`` of them: a later prompt that begins with the same tokens goes on from there and
        # runs only what is new.  The reference keeps its one sequence so (session_ids and the incremental prefill,
        # src/models/mod.rs:1022-1058).
        self.retain_limit = max(0, int(retain))
        self._retained: "OrderedDict[int, List[int]]" = OrderedDict()
        self._flight = None           # the decode step that is queued but not yet read
        self._inflight = {}           # slot -> steps queued beyond the committed length
        self._pinned = [None, None]
        self._pin_next = 0
        # a part that reads the batch on the host, or says nothing about it, cannot be recorded: step by step then
        self.use_graphs = (use_graphs and torch.device(model.rt.device).type == "cuda"
                           and getattr(model, "graph_safe", False))
        self._graphs = {}
        self.short_context = int(getattr(model, "short_context", 0) or 0)
        self._prompt_graphs = OrderedDict()      # (sequences, rows of the bucket) -> PromptGraph, the newest last
        from .graph import recorded_prompt_rows
        self.prompt_rows = (recorded_prompt_rows(model.weight_bytes(), len(model.spec.schedule), (4 if model.rt.dtype is torch.float32 else 2))
                            if self.use_graphs else 0)
        self._armed = None            # (graph, slots) whose device-side inputs are those of the next step
        cache = model.cache
        self.max_batch = max(1, min(max_batch, cache.n_slots))
        self.sampler = DeviceSampler(model, max_rows=self.max_batch)
        self.max_position = min(model.spec.max_position, cache.max_tokens)
        self.cache_tokens = cache.max_tokens
        self.page_size = cache.page_size
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def open(self, count: int) -> List[int]:
        cache = self.model.cache
        while cache.slots.free < count and self._retained:
            self._evict_oldest()
        return cache.open(count)

    def close(self, slots: Sequence[int]) -> None:
        self._drain()
        self._armed = None
        self.model.cache.close(slots)

    # ------------------------------------------------------------------ finished sequences kept for later prompts
    def _evict_oldest(self) -> None:
        slot, _ = self._retained.popitem(last=False)
        self.model.cache.close([slot])

    def adopt(self, prompts: Sequence[Sequence[int]]) -> List[Tuple[Optional[int], int]]:
        """For each prompt (slot, n): a kept sequence whose first n tokens are the prompt's (n >= MIN_REUSE, n <
        len(prompt) so that one token is left to run, and the cache can go back to n), taken out of the kept set;
        (None, 0) where there is none.  Longest match first come, first served."""
        cache = self.model.cache
        out: List[Tuple[Optional[int], int]] = []
        for p in prompts:
            best, best_n = None, 0
            for slot, held in self._retained.items():
                cap = min(len(held), len(p) - 1)
                n = 0
                while n < cap and held[n] == p[n]:
                    n += 1
                if n >= MIN_REUSE and n > best_n and cache.can_rewind(slot, n):
                    best, best_n = slot, n
            if best is not None:
                del self._retained[best]
            out.append((best, best_n))
        return out

    def make_room(self, needs: Sequence[int], slots: Sequence[Optional[int]]) -> None:
        """Give kept sequences up, oldest first, until the batch fits the cache: sequence i may come to hold
        ``needs[i]`` positions and goes on in ``slots[i]`` (None: a slot yet to be opened)."""
        cache = self.model.cache
        page = cache.page_size
        want = 0
        for need, slot in zip(needs, slots):
            pages = -(-need // page) * page
            want += pages if slot is None else max(0, pages - cache.held_tokens(slot))
        while self._retained and cache.free_tokens() < want:
            self._evict_oldest()

    def retain(self, slots: Sequence[int], histories: Sequence[Sequence[int]]) -> None:
        """Instead of ``close``: keep these finished sequences (``histories``: prompt and answer) for later prompts,
        the newest ``retain_limit`` of them; the rest is closed."""
        self._drain()
        self._armed = None
        cache = self.model.cache
        for slot, h in zip(slots, histories):
            n = cache.length(slot)                  # positions whose keys are in the cache: the last token was never fed
            self._retained[slot] = list(h[:n])
        while len(self._retained) > self.retain_limit:
            self._evict_oldest()

    def drop_retained(self) -> None:
        while self._retained:
            self._evict_oldest()

    def prefill(self, slots, prompts, options, reused: Optional[Sequence[int]] = None) -> List[int]:
        """The prompts' step.  ``reused[i]`` > 0: slot i already holds that many of prompt i's tokens (``adopt``)."""
        self._drain()
        self._armed = None
        self.sampler.begin(slots, prompts, options)
        reused = list(reused) if reused is not None else [0] * len(slots)
        cache = self.model.cache
        for s, n in zip(slots, reused):
            if n:
                cache.rewind(s, n)
        if not any(reused):
            first = self._short_prompts(slots, prompts, options)
            if first is not None:
                return first
        out: List[Optional[int]] = [None] * len(slots)
        # sequences that start run as one prompt step (attention over the step's own keys), those that go on as
        # another (rows that read the cache)
        for group in ([i for i, n in enumerate(reused) if not n], [i for i, n in enumerate(reused) if n]):
            if not group:
                continue
            entries = [StepEntry(slots[i], prompts[i][reused[i]:], [len(prompts[i]) - reused[i] - 1]) for i in group]
            toks = self._choose(self.model.step(entries), [slots[i] for i in group], [options[i] for i in group],
                                sum(len(e.tokens) for e in entries))
            for i, t in zip(group, toks):
                out[i] = t
        return out  # type: ignore[return-value]

    def _short_prompts(self, slots, prompts, options) -> Optional[List[int]]:
        """The first tokens of a few short prompts through a recorded step (``PromptGraph``), or None where that
        does not apply: graphs off, prompts beyond the largest bucket or more rows than a recorded step takes, no
        room for the bucket's rows, a mixer that keeps state of its own per sequence (the padding's rows would pass
        through it), or a group of layers that keeps a window's keys in a ring of pages (the padding's keys would
        land on ring entries that real positions still need)."""
        from .graph import PROMPT_BUCKETS, PromptGraph
        cache = self.model.cache
        longest = max(len(p) for p in prompts)
        if not self.use_graphs or min(len(p) for p in prompts) == 0 or longest > self.prompt_rows or cache.has_mixer_state:
            return None
        if any(g.ring_pages for g in cache.groups):
            return None
        rows = next(r for r in PROMPT_BUCKETS if r >= longest)
        if rows * len(slots) > self.prompt_rows or rows > self.max_position or any(cache.length(s) for s in slots):
            return None
        vocab = self.model.spec.vocab
        if min(min(p) for p in prompts) < 0 or max(max(p) for p in prompts) >= vocab:
            raise ValueError(f"token ids must lie in [0, {vocab})")
        try:
            cache.must_fit([(s, rows) for s in slots])
        except (CacheFull, CapacityError):
            return None
        for s in slots:
            cache.reserve(s, rows)
        cache.flush()
        key = (len(slots), rows)
        g = self._prompt_graphs.get(key)
        if g is None:
            g = self._prompt_graphs[key] = PromptGraph(self.model, len(slots), rows)
            while len(self._prompt_graphs) > MAX_PROMPT_GRAPHS:          # each holds its step's activations
                self._prompt_graphs.popitem(last=False)
        self._prompt_graphs.move_to_end(key)
        logits = g.run(slots, prompts)
        for s, p in zip(slots, prompts):
            cache.commit(s, len(p))
        return self._choose(logits, slots, options, sum(len(p) for p in prompts))

    def decode(self, slots, last_tokens, options) -> List[int]:
        if not self.use_graphs:
            entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, last_tokens)]
            return self._choose(self.model.step(entries), slots, options, len(slots))
        if not self.pipeline:
            graph = self._arm(slots, last_tokens, options)
            self.reserve_ahead(slots, 1)
            chosen = graph.run()
            view = self._pinned_view(len(slots))
            view.copy_(chosen, non_blocking=True)    # the step's result crosses to the host here, into pinned memory
            torch.cuda.current_stream().synchronize()
            out = view.tolist()
            self._advance_lengths(slots, 1)
            self.d2h_bytes += 4 * len(slots)
            return out
        return self._decode_pipelined(tuple(slots), list(last_tokens), options)

    # ------------------------------------------------------------------ run-ahead
    # With ``pipeline`` the step after the one being read is already queued on the GPU (its input tokens
    # were fed forward on the device), so the host's work between two steps (reading tokens, stop checks,
    # bookkeeping) overlaps the GPU's.  The reference overlaps its 8-byte token fetch with the next step the
    # same way (src/models/mod.rs:1262-1308, src/cuda.rs:2011-2021).  A step that ran ahead for a sequence
    # that then stops has only written keys and values beyond that sequence's end.  The caller must feed
    # back the tokens it was given (the generation loop does); one that feeds other tokens uses
    # ``pipeline=False``.
    def _launch(self, graph, slots):
        """Queue one step of ``graph`` and the copy of its tokens to pinned memory; None if a sequence has
        no room for the position the step would write."""
        cache = self.model.cache
        try:
            for s in slots:
                cache.reserve(s, cache.length(s) + self._inflight.get(s, 0) + 1)
        except (CacheFull, CapacityError):
            return None
        cache.flush()
        chosen = graph.run()
        view = self._pinned_view(len(slots))
        view.copy_(chosen, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        for s in slots:
            self._inflight[s] = self._inflight.get(s, 0) + 1
        self.d2h_bytes += 4 * len(slots)
        return {"slots": slots, "graph": graph, "tokens": view, "event": ev, "fed": None}

    def _pinned_view(self, n: int) -> torch.Tensor:
        """One of two pinned buffers in turn (a step in flight keeps its own until it is read)."""
        i = self._pin_next
        self._pin_next ^= 1
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            self._pinned[i] = torch.empty(max(64, n), dtype=torch.int32).pin_memory()
        return self._pinned[i][:n]

    def _read(self, flight, commit_slots) -> List[int]:
        flight["event"].synchronize()
        toks = flight["tokens"].tolist()
        cache = self.model.cache
        for s in flight["slots"]:
            self._inflight[s] -= 1
        for s in commit_slots:
            cache.commit(s, cache.length(s) + 1)
        return toks

    def _drain(self) -> None:
        if self._flight is not None:
            # the dropped step has run: the graph's positions and lengths on the device are one past the cache's
            # committed lengths, so the next step loads them anew
            self._read(self._flight, ())
            self._flight = None
            self._armed = None
        self._inflight.clear()

    def _context_bound(self, slots, ahead: int) -> int:
        """The bound of the graph that may run the next ``ahead`` steps of these sequences: the short-context bound
        while every sequence stays within it, else 0 (no bound)."""
        cache = self.model.cache
        short = self.short_context
        longest = max(cache.length(s) + self._inflight.get(s, 0) for s in slots) + ahead
        return short if longest <= short else 0

    def _decode_pipelined(self, slots, last_tokens, options) -> List[int]:
        fl = self._flight
        if fl is not None and fl["fed"] is not None and set(slots) <= set(fl["slots"]) and \
                all(fl["fed"][s] == t for s, t in zip(slots, last_tokens)):
            if fl["slots"] == slots and self._context_bound(slots, 1) == fl["graph"].max_len:
                nxt = self._launch(fl["graph"], slots)           # the step after, before this one is read
                toks = self._read(fl, slots)
                if nxt is not None:
                    nxt["fed"] = dict(zip(slots, toks))
                self._flight = nxt
                return toks
            # some sequences of the step in flight have ended: its tokens for the others are still theirs
            all_toks = dict(zip(fl["slots"], self._read(fl, slots)))
            self._flight = None
            self._inflight.clear()
            toks = [all_toks[s] for s in slots]
            graph = self._arm(slots, toks, options)
            nxt = self._launch(graph, slots)
            if nxt is not None:
                nxt["fed"] = dict(zip(slots, toks))
            self._flight = nxt
            return toks
        self._drain()
        graph = self._arm(slots, last_tokens, options, ahead=2)
        first = self._launch(graph, slots)
        if first is None:
            raise CacheFull("no room for the next position of a sequence")
        nxt = self._launch(graph, slots)
        toks = self._read(first, slots)
        if nxt is not None:
            nxt["fed"] = dict(zip(slots, toks))
        self._flight = nxt
        return toks

    # ------------------------------------------------------------------ graph plumbing
    def _arm(self, slots, last_tokens, options, ahead: int = 1):
        """The graph for this batch size (and for the lengths that the next ``ahead`` steps reach) with its inputs
        set: uploaded when the set of sequences or the graph changed, otherwise already there (the last step fed
        its tokens forward on the device)."""
        cache = self.model.cache
        all_greedy = all(o.greedy for o in options)
        bound = self._context_bound(slots, ahead)
        key = (len(slots), all_greedy, bound)
        graph = self._graphs.get(key)
        if graph is None:
            from .graph import DecodeGraph
            graph = self._graphs[key] = DecodeGraph(self.model, self.sampler, len(slots), all_greedy, bound)
        if self._armed != (key, tuple(slots)):
            params = np.array([[o.temperature, float(o.top_k), o.top_p, o.repeat_penalty] for o in options], dtype=np.float32)
            carried = None
            if last_tokens is None:
                # the tokens are on the device only, in the graph that ran these sequences' last step
                before = self._graphs.get(self._armed[0]) if self._armed and self._armed[1] == tuple(slots) else None
                if before is None:
                    raise ValueError("the next step's tokens are needed: no recorded step of these sequences holds them")
                carried = before.tokens.clone()
            graph.load(slots, last_tokens if carried is None else [0] * len(slots), [cache.length(s) for s in slots], params)
            if carried is not None:
                graph.tokens.copy_(carried)
            self.h2d_bytes += 4 * (6 * len(slots) + 1) + params.nbytes
            self._armed = (key, tuple(slots))
        elif last_tokens is not None:
            graph.feed(last_tokens)
            self.h2d_bytes += 4 * len(slots)
        return graph

    def recorded_launches(self, n_seqs: int) -> int:
        """Kernel launches of this library in one recorded decode step of ``n_seqs`` sequences (the graph used last
        among those of that size)."""
        found = [g for k, g in self._graphs.items() if k[0] == n_seqs and g.graph is not None]
        if not found:
            raise KeyError(f"no decode step of {n_seqs} sequences has been recorded")
        return found[-1].launches_per_step

    def reserve_ahead(self, slots, steps: int) -> None:
        cache = self.model.cache
        for s in slots:
            cache.reserve(s, cache.length(s) + steps)
        cache.flush()

    def _advance_lengths(self, slots, steps: int) -> None:
        cache = self.model.cache
        for s in slots:
            cache.commit(s, cache.length(s) + steps)

    def decode_on_device(self, slots, last_tokens, options, steps: int, reach: Optional[int] = None) -> torch.Tensor:
        """``steps`` decode steps without a host round trip between them (tokens are fed forward on
        the device); returns the last step's chosen tokens (device).  Used to time the device alone.
        ``reach``: how many steps the caller will run in all, this call's included; the graph is chosen for the
        lengths they reach, so that a warm-up and the timed steps after it run the same recorded step."""
        self._drain()
        graph = self._arm(slots, last_tokens, options, ahead=max(steps, reach or 0))
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
        out = tokens.tolist()
        self.model.check_device()
        return out
