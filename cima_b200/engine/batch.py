"""A step's batch: the tokens it brings and where they belong, as the kernels want them.

Rows are flat and ragged: the tokens of all sequences one after another, no padding.  Per row its
absolute position and the index of its sequence in the batch; per sequence its slot, its first row
and its length after the step.  All of it travels to the device in one copy from pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


Q_TILE = 64        # query rows per block of the prefill attention kernel
Q_TILE_TC = 128    # ... and of its tcgen05 variant


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are wanted


@dataclass
class StepBatch:
    prefill: bool                     # True: every sequence starts at position 0 (attention may read the step's own
                                      # keys); False: the rows read the cache (one token each, or sequences that
                                      # go on by several tokens)
    n_rows: int
    n_seqs: int
    n_want: int
    max_len: int                      # longest sequence after the step (host copy, sizes launches)
    want_all_in_order: bool
    tokens: torch.Tensor              # int32 [rows]
    row_pos: torch.Tensor             # int32 [rows]
    row_seq: torch.Tensor             # int32 [rows]
    seq_slot: torch.Tensor            # int32 [seqs]
    seq_first_row: torch.Tensor       # int32 [seqs + 1]
    seq_len: torch.Tensor             # int32 [seqs]
    want_rows: torch.Tensor           # int32 [wanted]
    n_q_tiles: int = 0                # several rows a sequence: blocks of 64 query rows, heaviest first
    q_tile_seq: torch.Tensor = None   # int32 [n_q_tiles] sequence of the block
    q_tile_row0: torch.Tensor = None  # int32 [n_q_tiles] first row of the block among the sequence's rows
    max_rows: int = 0                 # most rows that one sequence brings
    n_q_tiles_tc: int = 0             # the same in blocks of 128 rows
    q_tile_tc_seq: torch.Tensor = None
    q_tile_tc_row0: torch.Tensor = None
    host_seq_slot: np.ndarray = None
    host_seq_first_row: np.ndarray = None
    host_seq_len: np.ndarray = None


def check_entries(entries: Sequence[StepEntry], vocab: Optional[int] = None) -> None:
    """What must hold of a step's entries whatever their sizes; with ``vocab`` also the token ids and the wanted
    places (``build_batch`` checks those while it packs; a step that is run in parts checks them before the first
    part, so that a fault in a later part leaves nothing behind)."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    if len({e.slot for e in entries}) != len(entries):
        raise ValueError("a slot appears twice in one step")
    if any(len(e.tokens) <= 0 for e in entries):
        raise ValueError("every entry of a step brings at least one token")
    if vocab is None:
        return
    for i, e in enumerate(entries):
        tk = np.asarray(e.tokens, dtype=np.int64)
        if tk.min() < 0 or tk.max() >= vocab:
            raise ValueError(f"entry {i}: token ids must lie in [0, {vocab})")
        for p in e.want:
            if not (0 <= p < len(e.tokens)):
                raise ValueError(f"entry {i}: wanted place {p} is outside its {len(e.tokens)} tokens")


def build_batch(entries: List[StepEntry], starts: Sequence[int], vocab: int, device) -> StepBatch:
    """Validate and pack.  ``starts[i]`` is how many positions entry i's slot already holds."""
    check_entries(entries)
    counts = [len(e.tokens) for e in entries]
    if all(c == 1 for c in counts):
        prefill = False                   # one token each: attention over the cache, also at position 0
    elif all(s == 0 for s in starts):
        prefill = True
    else:
        prefill = False                   # some sequence goes on by several tokens: every row reads the cache
    B, T = len(entries), sum(counts)
    W = sum(len(e.want) for e in entries)
    q_tiles = []
    if any(c > 1 for c in counts):        # several rows of a sequence: blocks of query rows, heaviest first
        q_tiles = sorted(((i, r0) for i, c in enumerate(counts) for r0 in range(0, c, Q_TILE)),
                         key=lambda t: -(starts[t[0]] + t[1]))
    NT = len(q_tiles)
    tc_tiles = [t for t in q_tiles if t[1] % Q_TILE_TC == 0]
    NTC = len(tc_tiles)
    buf = np.empty(3 * T + 3 * B + 1 + W + 2 * NT + 2 * NTC, dtype=np.int32)
    tokens, row_pos, row_seq = buf[0:T], buf[T:2 * T], buf[2 * T:3 * T]
    o = 3 * T
    seq_slot, seq_first, seq_len = buf[o:o + B], buf[o + B:o + 2 * B + 1], buf[o + 2 * B + 1:o + 3 * B + 1]
    w0 = o + 3 * B + 1
    want_rows = buf[w0:w0 + W]
    if NT:
        buf[w0 + W:w0 + W + NT] = [t[0] for t in q_tiles]
        buf[w0 + W + NT:w0 + W + 2 * NT] = [t[1] for t in q_tiles]
    t0 = w0 + W + 2 * NT
    if NTC:
        buf[t0:t0 + NTC] = [t[0] for t in tc_tiles]
        buf[t0 + NTC:t0 + 2 * NTC] = [t[1] for t in tc_tiles]
    r = w = 0
    for i, (e, s, c) in enumerate(zip(entries, starts, counts)):
        tk = np.asarray(e.tokens, dtype=np.int64)
        if tk.min() < 0 or tk.max() >= vocab:
            raise ValueError(f"entry {i}: token ids must lie in [0, {vocab})")
        tokens[r:r + c] = tk
        row_pos[r:r + c] = np.arange(s, s + c)
        row_seq[r:r + c] = i
        seq_slot[i], seq_first[i], seq_len[i] = e.slot, r, s + c
        for p in e.want:
            if not (0 <= p < c):
                raise ValueError(f"entry {i}: wanted place {p} is outside its {c} tokens")
            want_rows[w] = r + p
            w += 1
        r += c
    seq_first[B] = T
    host = torch.from_numpy(buf)
    if torch.device(device).type == "cuda":
        dev = host.pin_memory().to(device, non_blocking=True)
    else:
        dev = host.clone()
    all_in_order = W == T and bool(np.array_equal(want_rows, np.arange(T)))
    return StepBatch(prefill=prefill, n_rows=T, n_seqs=B, n_want=W, max_len=int(seq_len.max()),
                     want_all_in_order=all_in_order, max_rows=max(counts),
                     tokens=dev[0:T], row_pos=dev[T:2 * T], row_seq=dev[2 * T:3 * T],
                     seq_slot=dev[o:o + B], seq_first_row=dev[o + B:o + 2 * B + 1],
                     seq_len=dev[o + 2 * B + 1:o + 3 * B + 1], want_rows=dev[w0:w0 + W],
                     n_q_tiles=NT, q_tile_seq=dev[w0 + W:w0 + W + NT], q_tile_row0=dev[w0 + W + NT:w0 + W + 2 * NT],
                     n_q_tiles_tc=NTC, q_tile_tc_seq=dev[t0:t0 + NTC], q_tile_tc_row0=dev[t0 + NTC:t0 + 2 * NTC],
                     host_seq_slot=seq_slot.copy(), host_seq_first_row=seq_first.copy(), host_seq_len=seq_len.copy())
