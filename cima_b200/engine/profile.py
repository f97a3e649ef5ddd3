"""Time of every launch of a step, measured inside the step, without a profiler.

A step is recorded as CUDA graphs that stop after its n-th launch, for every n; the time of the graph cut
after launch n minus that of the graph cut after launch n - 1 is what launch n adds to the step, with
everything that surrounds it in the real step: the launch before it still finishing, its own first loads
issued early, caches as the step leaves them.  (A launch timed alone between two events lacks all of that.)
Every launch states the bytes it has to move and the operations it has to do (``Kernels._admit``), so each
line reads as a fraction of the measured peaks.  The reference prints the same table from event timers
around its launches: microseconds per launch, launches per token and the weight-streaming floor
(``cima profile``, src/selftest.rs:1201-1331).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch


@dataclass
class Launch:
    name: str
    nbytes: float
    flops: float
    us: float = 0.0


@dataclass
class StepProfile:
    """What ``Kernels`` consults before each launch while a step is profiled."""
    limit: Optional[int] = None        # launches beyond this many are left out (None: all run)
    kv_tokens: float = 0.0             # cached positions that the step's attention reads (each once), all sequences
    qk_pairs: float = 0.0              # (query row, key) pairs of the step's attention
    seen: int = 0
    launches: List[Launch] = field(default_factory=list)

    def admit(self, name: str, nbytes: float, flops: float) -> bool:
        self.seen += 1
        if self.limit is not None and self.seen > self.limit:
            return False
        self.launches.append(Launch(name, float(nbytes), float(flops)))
        return True


def _time_graph(g: torch.cuda.CUDAGraph, reps: int) -> float:
    """Median microseconds of one replay (replays back to back, timed in groups by CUDA events)."""
    groups, per = 5, max(1, reps // 5)
    g.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(groups):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(per):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) * 1e3 / per)
    out.sort()
    return out[len(out) // 2]


def time_launches(kernels, run_step: Callable[[], None], kv_tokens: float = 0.0, qk_pairs: float = 0.0,
                  reps: int = 20) -> List[Launch]:
    """The launches of ``run_step`` (a function that issues one step's work on the current stream, from buffers of
    fixed address) with the time each adds to the step.  ``run_step`` is called once for real, then recorded once
    per launch; what it computes while it is cut short is thrown away."""
    if kernels.profile is not None:
        raise RuntimeError("a step is being profiled already")
    try:
        kernels.profile = whole = StepProfile(None, kv_tokens, qk_pairs)
        run_step()
        torch.cuda.synchronize()
        n = len(whole.launches)
        before = 0.0
        for k in range(1, n + 1):
            kernels.profile = StepProfile(k, kv_tokens, qk_pairs)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                run_step()
            t = _time_graph(g, reps)
            del g
            whole.launches[k - 1].us = t - before
            before = t
    finally:
        kernels.profile = None
    return whole.launches


def table(launches: List[Launch], hbm_gbs: float, tflops: float, tokens: int = 0) -> str:
    """The launches as text: time, share of the step, achieved GB/s and TFLOP/s with their fractions of the given
    peaks, the step's total and, for a decode step of ``tokens`` tokens, launches per token and the floor (the
    time its bytes take at the peak bandwidth)."""
    total = sum(l.us for l in launches) or 1.0
    lines = [f"{'#':>4} {'launch':<28} {'us':>9} {'%':>6} {'MB':>9} {'GB/s':>8} {'of peak':>8} {'TFLOP/s':>8} {'of peak':>8}"]
    for i, l in enumerate(launches):
        us = max(l.us, 1e-3)
        gbs, tf = l.nbytes / us / 1e3, l.flops / us / 1e6
        lines.append(f"{i:>4} {l.name:<28} {l.us:>9.2f} {100 * l.us / total:>6.1f} {l.nbytes / 1e6:>9.2f} {gbs:>8.0f} "
                     f"{gbs / hbm_gbs:>8.2f} {tf:>8.1f} {tf / tflops:>8.2f}")
    nbytes = sum(l.nbytes for l in launches)
    lines.append(f"step: {total:.1f} us in {len(launches)} launches, {nbytes / 1e6:.1f} MB: "
                 f"{nbytes / total / 1e3:.0f} GB/s ({nbytes / total / 1e3 / hbm_gbs:.2f} of {hbm_gbs:.0f}); "
                 f"floor {nbytes / hbm_gbs / 1e3:.1f} us" + (f"; {len(launches) / tokens:.1f} launches a token" if tokens else ""))
    return "\n".join(lines)


def profile_decode(stepper, slots, last_tokens, options, reps: int = 20) -> List[Launch]:
    """One decode step of the sequences in ``slots`` (after their prompts), launch by launch, with the sampler and
    the bookkeeping kernel at its end, as the stepper records it."""
    from .graph import DecodeGraph
    import numpy as np
    model, cache = stepper.model, stepper.model.cache
    stepper._drain()
    stepper._armed = None
    all_greedy = all(o.greedy for o in options)
    ahead = 8 * reps + 16                     # every replay of the whole step moves the sequences on by one position
    graph = DecodeGraph(model, stepper.sampler, len(slots), all_greedy, stepper._context_bound(slots, ahead))
    lengths = [cache.length(s) for s in slots]
    params = np.array([[o.temperature, float(o.top_k), o.top_p, o.repeat_penalty] for o in options], dtype=np.float32)
    graph.load(slots, last_tokens, lengths, params)
    for s, n in zip(slots, lengths):         # room for all of those positions
        cache.reserve(s, min(n + ahead, stepper.max_position))
    cache.flush()
    torch.cuda.synchronize()
    try:
        return time_launches(model.rt.kernels, graph._step, kv_tokens=float(sum(lengths) + len(slots)),
                             qk_pairs=float(sum(lengths) + len(slots)), reps=reps)
    finally:
        torch.cuda.synchronize()


def profile_prompt(model, prompt_lens, reps: int = 6, seed: int = 0) -> List[Launch]:
    """One prompt step (random token ids of the given lengths, logits at each prompt's end), launch by launch."""
    import numpy as np
    from .batch import build_batch, StepEntry
    cache = model.cache
    rng = np.random.default_rng(seed)
    slots = cache.open(len(prompt_lens))
    try:
        entries = [StepEntry(s, rng.integers(0, model.spec.vocab, size=n).tolist(), [n - 1])
                   for s, n in zip(slots, prompt_lens)]
        batch = build_batch(entries, [0] * len(entries), model.spec.vocab, model.rt.device)
        for e in entries:
            cache.reserve(e.slot, len(e.tokens))
        cache.flush()
        torch.cuda.synchronize()
        pairs = float(sum(n * (n + 1) / 2 for n in prompt_lens))
        return time_launches(model.rt.kernels, lambda: model.forward(batch), kv_tokens=float(sum(prompt_lens)),
                             qk_pairs=pairs, reps=reps)
    finally:
        torch.cuda.synchronize()
        cache.close(slots)
