"""A decode step captured as a CUDA graph: one launch per token instead of a few hundred.

The step's inputs (tokens, positions, lengths, slots, sampling parameters) live in device buffers of
fixed address; the captured step ends with a kernel that feeds the chosen tokens back and moves
every sequence on by one, so replaying needs nothing from the host but the pages that the next
positions need (block tables are updated outside the graph, before the replay).  The reference
arms its decode graph the same way around a device position counter
(src/models/transformer.rs:1467-1494, src/cuda.rs:1069-1097).
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .batch import StepBatch, StepEntry, build_batch


class DecodeGraph:
    """One batch size's captured step.  ``load`` sets its inputs for a set of sequences; ``run``
    does one step (the first run after construction executes eagerly and captures)."""

    def __init__(self, model, sampler, n_seqs: int, all_greedy: bool, max_len: int = 0):
        """``max_len``: the most positions that a sequence may hold after a step of this graph (0: any number).  A
        recorded step fixes its launches; one recorded for short contexts takes the kernels' choices for them
        (the decode attention without splits), and the stepper moves to the unbounded graph when a sequence
        outgrows the bound."""
        self.model, self.sampler = model, sampler
        self.B = B = n_seqs
        self.all_greedy = all_greedy
        self.max_len = max_len
        dev = model.rt.device
        self.meta = torch.zeros(6 * B + 1, dtype=torch.int32, device=dev)
        self.meta_host = torch.zeros(6 * B + 1, dtype=torch.int32).pin_memory()
        m = self.meta
        self.tokens, self.row_pos, self.row_seq = m[0:B], m[B:2 * B], m[2 * B:3 * B]
        self.seq_slot, self.seq_first_row, self.seq_len = m[3 * B:4 * B], m[4 * B:5 * B + 1], m[5 * B + 1:6 * B + 1]
        self.params = torch.zeros(B, 4, dtype=torch.float32, device=dev)
        self.chosen = torch.zeros(B, dtype=torch.int32, device=dev)
        # What a recorded step may know on the host is what every replay shares: the number of sequences and their
        # rows (one each).  Slots, positions and lengths change from replay to replay and exist on the device only
        # (``host_seq_slot`` / ``host_seq_len`` stay None; ``max_len`` is the graph's bound, 0 = unknown).
        self.batch = StepBatch(prefill=False, n_rows=B, n_seqs=B, n_want=B, max_len=max_len, want_all_in_order=True,
                               tokens=self.tokens, row_pos=self.row_pos, row_seq=self.row_seq,
                               seq_slot=self.seq_slot, seq_first_row=self.seq_first_row, seq_len=self.seq_len,
                               want_rows=self.row_seq, max_rows=1, host_seq_first_row=np.arange(B + 1, dtype=np.int32))
        self.graph = None
        self.slots: List[int] = []

    def load(self, slots: Sequence[int], tokens: Sequence[int], lengths: Sequence[int], params: np.ndarray) -> None:
        """Inputs of the next step: sequence i sits in slots[i], holds lengths[i] positions and brings tokens[i]."""
        B = self.B
        h = self.meta_host.numpy()
        h[0:B] = tokens
        h[B:2 * B] = lengths                       # the new token's position
        h[2 * B:3 * B] = np.arange(B)
        h[3 * B:4 * B] = slots
        h[4 * B:5 * B + 1] = np.arange(B + 1)
        h[5 * B + 1:6 * B + 1] = np.asarray(lengths) + 1
        self.meta.copy_(self.meta_host, non_blocking=True)
        self.params.copy_(torch.from_numpy(params), non_blocking=False)
        self.slots = list(slots)

    def feed(self, tokens: Sequence[int]) -> None:
        """The next step's input tokens from the host (pinned memory, one small copy).  The captured step
        has fed its own choices forward already; the host's copy is what a caller that decides the next
        input itself (forced tokens, another sampler) relies on."""
        h = self.meta_host.numpy()
        h[0:self.B] = tokens
        self.tokens.copy_(self.meta_host[0:self.B], non_blocking=True)

    def _step(self) -> None:
        logits = self.model.forward(self.batch)
        self.sampler.sample(logits, self.seq_slot, self.params, self.chosen, self.all_greedy)
        self.model.rt.kernels.decode_advance(self.chosen, self.tokens, self.row_pos, self.seq_len)

    def run(self) -> torch.Tensor:
        """One decode step of the loaded sequences; returns the device tensor of chosen tokens."""
        if self.graph is None:
            self._step()                            # a real step, eagerly; it also warms every kernel up
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            k = self.model.rt.kernels
            before = k.launches
            with torch.cuda.graph(g):               # records the same step for the following ones; runs nothing
                self._step()
            self.launches_per_step = k.launches - before
            self.graph = g
        else:
            self.graph.replay()
        return self.chosen


PROMPT_BUCKETS = (16, 32, 64, 128, 256, 384, 512, 768, 1024, 1536, 2048)    # rows a sequence of a recorded prompt step
PROMPT_ROWS = 256                           # rows (all sequences together) that every model's prompt steps are recorded for


MAX_PROMPT_GRAPHS = 24    # recorded prompt steps kept (by sequences and rows); the one used longest ago gives way


def recorded_prompt_rows(weight_bytes: float, sites: int, element_size: int) -> int:
    """The most rows, all sequences together, for which a prompt step is recorded rather than issued launch by launch:
    the largest bucket whose padded step the device finishes before the host could have issued an unrecorded one.
    ``weight_bytes``: what a step reads of the weights; ``sites``: layers that run; ``element_size``: of a weight.
    The host needs about 145 us a layer for a prompt step's launches whatever the sizes (measured: 3.8 ms for the 24
    layers of the 0.5B shape, 4.0 to 4.4 ms for 28 layers of the 1.5B and the 7B shape), so a small model's prompts
    of some hundred tokens wait for the host (0.5B, 300 tokens: 4.0 ms to the first token, of which the device works
    0.5), while a 7B prompt beyond 256 rows keeps the device busy longer than the host needs (300 tokens: 5.5 ms of
    device work behind 4.3 ms of launches) and would only pay for its padding.  The device's time is put at the
    weights read once at 6 TB/s plus two operations per weight and row at 0.8 PFLOP/s (what the small shapes reach at
    some hundred rows)."""
    host_s = 145e-6 * sites
    best = PROMPT_ROWS
    for rows in PROMPT_BUCKETS:
        if rows > PROMPT_ROWS and weight_bytes / 6e12 + 2.0 * (weight_bytes / element_size) * rows / 0.8e15 <= host_s:
            best = rows
    return best


class PromptGraph:
    """The step of a few short prompts recorded as a graph, for the first token's sake: prompts of some tens of
    tokens are a few milliseconds of device work behind some 250 launches from the host, and the host is the slower
    of the two.  Every prompt is padded at its end to the bucket's rows; the rows of the padding come after the
    sequence's real rows, so no real row sees them (attention is causal and stays inside a sequence), their keys
    land beyond the sequence's committed length, where the next tokens are written over them, and logits are
    gathered at each prompt's last real row only.  Padding changes no result.  (The reference records its decode
    step only, src/models/transformer.rs:1467-1494.)"""

    def __init__(self, model, n_seqs: int, rows: int):
        self.model, self.n_seqs, self.rows = model, n_seqs, rows
        dev = model.rt.device
        self.batch = build_batch([StepEntry(i, [0] * rows, [rows - 1]) for i in range(n_seqs)], [0] * n_seqs,
                                 model.spec.vocab, dev)
        self.batch.host_seq_slot = self.batch.host_seq_len = None       # they change from replay to replay
        self.host = torch.zeros(n_seqs * rows + 2 * n_seqs, dtype=torch.int32).pin_memory()
        self.graph = None
        self.logits = None
        self.uses = 0

    def run(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> torch.Tensor:
        """Float32 logits [sequences, vocab] at each prompt's last token.  The caller has reserved ``rows`` positions
        for every slot and commits the prompts' lengths afterwards."""
        B, R = self.n_seqs, self.rows
        h = self.host.numpy()
        h[:B * R] = 0
        for i, p in enumerate(prompts):
            h[i * R:i * R + len(p)] = p
            h[B * R + i] = slots[i]
            h[B * R + B + i] = i * R + len(p) - 1
        b = self.batch
        b.tokens.copy_(self.host[:B * R], non_blocking=True)
        b.seq_slot.copy_(self.host[B * R:B * R + B], non_blocking=True)
        b.want_rows.copy_(self.host[B * R + B:B * R + 2 * B], non_blocking=True)
        if self.graph is None:
            # The padded step, launch by launch.  A shape's first step is only that; its second is recorded as well
            # (recording costs about one more step's launches, which a shape that never comes back would not
            # repay); from the third on the graph is replayed.  What is computed is the same each time.
            self.uses += 1
            out = self.model.forward(b)
            if self.uses >= 2:
                torch.cuda.current_stream().synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.logits = self.model.forward(b)
                self.graph = g
            return out
        self.graph.replay()
        return self.logits
