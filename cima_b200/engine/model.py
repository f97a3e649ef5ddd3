"""A model put together from a ModelSpec: embedding, the blocks in the order of the schedule, final
norm and head; its cache; and the one step function that prefill, decoding, generation and trace
replay all go through.

The reference's counterparts: ``Transformer::build`` (src/models/transformer.rs:778-1002),
``forward_chunk_at`` (:1012-1321), ``project_logits`` (:1631-1652); one sequence there, a ragged
batch of sequences here.
"""
from __future__ import annotations

import dataclasses
import sys
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.kv import KVCache, StateRequest
from ..config.registry import lookup_architecture, read_config_json
from ..config.specs import ModelSpec
from ..parts import Linear, Runtime, build_block, build_norm
from ..parts.linear import FOLDED_NORM_ROWS
from ..parts.norm import RowsInfo
from ..weights.loader import TensorSpec, tensor_names
from .batch import StepBatch, StepEntry, build_batch, check_entries
from .fit import STEP_ROWS

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype {d!r} is not one of bfloat16, float32")
    return _DTYPES[d]


def build_plan(spec: ModelSpec, rt: Optional[Runtime] = None) -> Dict[str, TensorSpec]:
    """Every tensor the model reads, by name (needs no GPU: parts are built but not loaded)."""
    rt = rt or Runtime(kernels=None, dtype=torch.bfloat16, device="cpu")
    return Model(spec, rt).plan()


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        for i in spec.schedule:
            if not (0 <= i < len(spec.layers)):
                raise ValueError(f"the schedule names layer {i}; the model has {len(spec.layers)}")
        self.blocks = [build_block(b, i, rt) for i, b in enumerate(spec.layers)]
        self.final_norm = build_norm(spec.final_norm, rt)
        self.config = None                                  # set by load_model
        self.step_rows = STEP_ROWS                          # a step of more rows runs in parts
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self.cache: Optional[KVCache] = None

    # ------------------------------------------------------------------ weights
    def plan(self) -> Dict[str, TensorSpec]:
        s = self.spec
        p: Dict[str, TensorSpec] = {s.embed_name: TensorSpec((s.vocab, s.hidden))}
        for b in self.blocks:
            p.update(b.plan())
        p.update(self.final_norm.plan(s.final_norm_name))
        if not s.tie_head:
            p[s.head_name] = TensorSpec((s.vocab, s.hidden))
        return p

    def ignorable(self) -> List[str]:
        """Names a checkpoint may hold without the model reading them."""
        pats = ["*.rotary_emb.inv_freq"]
        if self.spec.tie_head:
            pats.append(self.spec.head_name)
        return pats

    def load(self, tensors) -> None:
        """``tensors``: name -> tensor, a dict or a ``TensorSource`` that fetches each tensor when it is asked for
        (every name of the plan is asked for once)."""
        s = self.spec
        table = tensors[s.embed_name]
        self.embedding = self.rt.matrix(table)
        if s.tie_head:
            self.head = Linear(self.embedding, None, self.rt)     # one copy on the device serves both
        del table
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors, s.final_norm_name)
        if not s.tie_head:
            self.head = Linear(tensors[s.head_name], None, self.rt)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """Every tensor of the plan by its name, as it is kept on the device (matrices in the model's precision or
        the 32 bits they were stored in, vectors in float32); stacked matrices come back as views of their rows."""
        s = self.spec
        out: Dict[str, torch.Tensor] = {s.embed_name: self.embedding}
        for b in self.blocks:
            out.update(b.state())
        out.update(self.final_norm.state(s.final_norm_name))
        if not s.tie_head:
            out[s.head_name] = self.head.weight
        return out

    @property
    def short_context(self) -> int:
        """The bound of the context class for which decode steps are recorded apart: the smallest that a mixer
        names (``mixer.short_context``), 0 if none does."""
        named = [int(getattr(b.mixer, "short_context", 0) or 0) for b in self.blocks if hasattr(b, "mixer")]
        named = [n for n in named if n > 0]
        return min(named) if named else 0

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step may be recorded as a CUDA graph: every layer's parts and the final norm say so."""
        return all(getattr(b, "graph_safe", False) for b in self.blocks) and getattr(self.final_norm, "graph_safe", False)

    def weight_bytes(self) -> int:
        """Bytes a decode step reads of the weights: every block, final norm and head once
        (embedding rows excluded unless the head shares the table)."""
        return sum(b.nbytes() for b in self.blocks) + self.final_norm.nbytes() + self.head.nbytes()

    # ------------------------------------------------------------------ cache
    def make_cache(self, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = 64,
                   extra_state: Sequence[StateRequest] = ()) -> KVCache:
        # storage belongs to a *site* (an entry of the schedule), weights to a layer: a layer that
        # runs twice keeps the keys and values of each run apart
        sched = self.spec.schedule
        shares = {site: self.spec.layers[layer].mixer.cache_from for site, layer in enumerate(sched)
                  if self.spec.layers[layer].mixer.cache_from is not None}
        self.cache = KVCache([self.blocks[layer].cache_requests(site) for site, layer in enumerate(sched)],
                             max_tokens, self.spec.max_position,
                             self.rt.dtype, self.rt.device, page_size=page_size, max_seqs=max_seqs,
                             shares=shares, extra_state=extra_state)
        return self.cache

    def forecast(self, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = 64,
                 extra_state: Sequence[StateRequest] = ()):
        """Bytes that the weights, a cache of ``max_tokens`` positions and a step's scratch will take."""
        from .fit import forecast
        sched = self.spec.schedule
        shares = [site for site, layer in enumerate(sched) if self.spec.layers[layer].mixer.cache_from is not None]
        widest = max([int(getattr(b, "scratch_row", lambda: 0)()) for b in self.blocks] + [self.spec.hidden])
        return forecast(self.plan(), [self.blocks[layer].cache_requests(site) for site, layer in enumerate(sched)],
                        self.rt.dtype, max_tokens, self.spec.hidden, self.spec.vocab, widest, page_size, shares,
                        extra_state, max_seqs or 0)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the tokens the entries bring, from the cache earlier steps left; float32 logits
        ``[wanted, vocab]`` in the order of the entries and of their ``want``."""
        cache = self.cache
        if cache is None:
            raise RuntimeError("the model has no cache yet: call make_cache first")
        entries = list(entries)
        for e in entries:
            if not cache.slots.is_held(e.slot):
                raise ValueError(f"slot {e.slot} is not open")
        starts = [cache.length(e.slot) for e in entries]
        # the whole step fits or nothing is taken: a step that fails leaves the cache as it found it
        cache.must_fit([(e.slot, s + len(e.tokens)) for e, s in zip(entries, starts)])
        if sum(len(e.tokens) for e in entries) > self.step_rows:
            return self._step_in_parts(entries)
        return self._step_within_bound(entries, starts)

    def _step_within_bound(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> torch.Tensor:
        cache = self.cache
        limit = cache.most_tokens_going_on()
        if limit is not None and any(starts) and max(len(e.tokens) for e in entries) > limit:
            return self._step_in_rounds(entries, limit)
        batch = build_batch(entries, starts, self.spec.vocab, self.rt.device)
        for e, s in zip(entries, starts):
            cache.reserve(e.slot, s + len(e.tokens))
        cache.flush()
        logits = self.forward(batch)
        for e, s in zip(entries, starts):
            cache.commit(e.slot, s + len(e.tokens))
        return logits

    def _step_in_parts(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of more rows than ``step_rows`` (the number the forecast of a step's scratch counts on) as several:
        its sequences in their order, as many at a time as stay within the bound; a sequence that alone exceeds it
        in rounds of ``step_rows`` tokens (its later rounds go on from the cache).  Sequences do not depend on one
        another and a sequence's logits not on how its tokens are cut, so the logits are the step's own, in the
        order of the entries and of their ``want``.  With a window's ring of pages a prompt that starts is left
        whole however long (it reads its own rows, while rounds that go on may add a page at most)."""
        check_entries(entries, self.spec.vocab)
        cache = self.cache
        ring = cache.most_tokens_going_on() is not None
        parts, group, rows = [], [], 0

        def run_group():
            nonlocal group, rows
            if group:
                parts.append(self._step_within_bound(group, [cache.length(e.slot) for e in group]))
            group, rows = [], 0

        for e in entries:
            n = len(e.tokens)
            if n > self.step_rows:
                run_group()
                if ring and cache.length(e.slot) == 0:
                    group = [e]
                    run_group()
                else:
                    parts.append(self._step_in_rounds([e], self.step_rows))
                continue
            if rows + n > self.step_rows:
                run_group()
            group.append(e)
            rows += n
        run_group()
        return torch.cat(parts)

    def _step_in_rounds(self, entries: Sequence[StepEntry], most: int) -> torch.Tensor:
        """The same step as rounds of at most ``most`` tokens a sequence (see ``KVCache.most_tokens_going_on``);
        the logits come back in the order of the entries and of their ``want``, as from one step."""
        for i, e in enumerate(entries):
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"entry {i}: wanted place {w} is outside its {len(e.tokens)} tokens")
        parts, place = [], {}                                 # (entry, index in its want) -> row among all rounds' logits
        done_rows = 0
        for lo in range(0, max(len(e.tokens) for e in entries), most):
            sub = []
            for i, e in enumerate(entries):
                if lo >= len(e.tokens):
                    continue
                want = []
                for k, w in enumerate(e.want):
                    if lo <= w < lo + most:
                        place[(i, k)] = done_rows + sum(len(x.want) for x in sub) + len(want)
                        want.append(w - lo)
                sub.append(StepEntry(e.slot, e.tokens[lo:lo + most], want))
            parts.append(self.step(sub))
            done_rows += parts[-1].shape[0]
        order = [place[(i, k)] for i, e in enumerate(entries) for k in range(len(e.want))]
        logits = torch.cat(parts)
        return logits[torch.as_tensor(order, dtype=torch.long, device=logits.device)] if order else logits

    def check_device(self) -> None:
        """Raise if a bounded wait inside a kernel ran out since the last check (synchronises)."""
        k = self.rt.kernels
        if hasattr(k, "device_errors") and k.device_errors():
            raise RuntimeError("a kernel's bounded wait ran out (TMA or tensor-core pipeline): results are invalid")

    def forward(self, batch: StepBatch) -> torch.Tensor:
        K_, s = self.rt.kernels, self.spec
        x = self.rt.empty(batch.n_rows, s.hidden, dtype=torch.float32)
        # What a kernel leaves behind about the rows it wrote travels along as a RowsInfo, so that norms are
        # folded into the products around them (few rows) or run together with the residual add (many rows).
        info = None
        order = [self.blocks[layer] for layer in s.schedule]
        if batch.n_rows <= FOLDED_NORM_ROWS and not self.rt.full_precision:
            ssq = self.rt.empty(batch.n_rows, 1, dtype=torch.float32)
            first = getattr(order[0], "mixer_norm", None) if order else self.final_norm
            if (getattr(first, "weight", None) is not None and first.spec.kind == "rmsnorm"
                    and first.spec.size == s.hidden):
                xw = self.rt.empty(batch.n_rows, s.hidden)
                K_.embed(batch.tokens, self.embedding, x, s.embed_scale, ssq, first.weight, xw)
                info = RowsInfo(ssq=ssq, xw=xw, xw_norm=first)
            else:
                K_.embed(batch.tokens, self.embedding, x, s.embed_scale, ssq)
                info = RowsInfo(ssq=ssq)
        else:
            K_.embed(batch.tokens, self.embedding, x, s.embed_scale)
        for site, block in enumerate(order):
            if site + 1 < len(order):
                nxt = getattr(order[site + 1], "mixer_norm", None)
            else:
                nxt = self.final_norm if batch.want_all_in_order else None
            info = block.forward(x, batch, self.cache, site, info, nxt)
        return self.project(x, batch, info)

    def project(self, x: torch.Tensor, batch: StepBatch, info=None) -> torch.Tensor:
        """Final norm and head at the wanted rows only."""
        if batch.n_want == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=self.rt.device)
        if not batch.want_all_in_order:
            picked = self.rt.empty(batch.n_want, self.spec.hidden, dtype=torch.float32)
            self.rt.kernels.gather_rows(x, batch.want_rows, picked)
            x, info = picked, None
        if info is not None and getattr(info, "norm", None) is self.final_norm and info.h is not None:
            return self.head.logits(info.h)
        if hasattr(self.final_norm, "lazy"):
            ssq = getattr(info, "ssq", None) if info is not None else None
            xw = info.xw if (info is not None and getattr(info, "xw_norm", None) is self.final_norm) else None
            return self.head.logits(self.final_norm.lazy(x, ssq, xw))
        return self.head.logits(self.final_norm(x))


def settle_head(spec: ModelSpec, stored: Sequence[str], warn=None) -> ModelSpec:
    """The spec with the head tied to the table if the architecture allows a checkpoint without a head
    tensor and this one has none (src/models/transformer.rs:810: tied = the flag, or no lm_head.weight)."""
    names = [spec.head_name] + [spec.head_name[len(p):] for p in spec.optional_prefixes if spec.head_name.startswith(p)]
    if spec.tie_head or not spec.head_may_be_absent or any(n in stored for n in names):
        return spec
    if warn is not None:
        warn(f"{spec.head_name} absent: the embedding table serves as the head")
    return dataclasses.replace(spec, tie_head=True)


def load_model(folder: Optional[str] = None, dtype="bfloat16", max_tokens: int = 4096, max_seqs: Optional[int] = None,
               device="cuda:0", kernels=None, verbose: bool = True, config=None, seed: int = 0,
               draw: str = "cpu") -> Model:
    """A model from a folder with config.json and model.safetensors, or, without a folder, from ``config`` (a
    config.json dict or the architecture's typed configuration) with random weights drawn from ``seed``; its
    class is chosen by the configuration either way, and both go through the same steps: the fit check, the parts'
    ``load`` from a source that hands out one tensor at a time, the cache.  ``draw``: where the random values are
    drawn, "cpu" (the values that ``write_random_model`` stores for this seed) or "device" (the device's own
    generator: other values, seconds instead of a minute for a 7B shape).  The reference's in-memory stand-in for
    a checkpoint takes the same road as a file (src/selftest.rs:23-159)."""
    from ..kernels import Kernels
    from ..weights.loader import CheckpointTensors, RandomTensors
    if (folder is None) == (config is None):
        raise ValueError("load_model takes a model folder or a configuration, one of the two")
    if folder is not None:
        raw = read_config_json(folder)
    else:
        raw = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    entry = lookup_architecture(raw)
    typed = entry.parse(raw)
    spec = entry.spec(typed)
    if folder is not None:
        spec = settle_head(spec, tensor_names(folder),
                           warn=(lambda m: print(f"[cima_b200] {m}", file=sys.stderr, flush=True)) if verbose else None)
    rt = Runtime(kernels=kernels if kernels is not None else Kernels(verbose=verbose),
                 dtype=parse_dtype(dtype), device=device)
    model = Model(spec, rt)
    model.config = typed                                    # the architecture's typed configuration, as parsed
    from ..sampling.sampler import sampler_state
    from .fit import check_fit
    check_fit(model.forecast(max_tokens, max_seqs, extra_state=sampler_state()), device)     # before anything is allocated
    if folder is not None:
        source = CheckpointTensors(folder, model.plan(), ignore=model.ignorable(), optional_prefixes=spec.optional_prefixes)
    else:
        if draw not in ("cpu", "device"):
            raise ValueError(f"draw '{draw}' is neither 'cpu' nor 'device'")
        source = RandomTensors(model.plan(), seed, torch.bfloat16, device if draw == "device" else "cpu")
    with source:
        model.load(source)
    model.load_peak_host_bytes = source.peak_bytes          # most bytes of fetched tensors alive at once while loading
    model.make_cache(max_tokens, max_seqs, extra_state=sampler_state())
    return model
