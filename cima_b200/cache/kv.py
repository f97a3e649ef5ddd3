"""The cache: a slot for each live sequence, keys and values for each layer in pages, and
fixed-size state for each slot beside them.

Layout.  Layers whose mixers ask for the same storage (KV heads, head size, window) form a
*group*.  A group owns ``[layers, pages, 2 (k|v), kv_heads, page_size, head_dim]`` and one block
table ``[slots, width]`` of page ids that all its layers share.  A group that keeps every key
gives a sequence one page per ``page_size`` positions; a group with a window of ``w`` keys gives
it a ring of ``ceil(w / page_size) + 1`` pages, position ``p`` living in ring entry
``(p / page_size) % ring``; those are the pages that can still hold a key within the window of
the newest position.  A slot's pages go back to their pools when the slot is closed and are
handed to later sequences with their old contents, which nothing reads: every kernel is given
the sequence's length.

The reference keeps one sequence: per layer K and V of ``[kv_heads, max_seq, head_dim]`` and one
cursor (src/models/transformer.rs:764, :916-917; src/kernels.cu:440-454), its fixed-size state
(position counter, penalty ring, next token) in separate device buffers (:716-729).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import CacheFull, FreeList


@dataclass(frozen=True)
class KVRequest:
    """What a mixer needs per position: keys and values of ``n_kv_heads`` heads of ``head_dim``;
    ``window`` 0 = all positions are kept, w > 0 = only the last w need to be."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per sequence: a tensor ``[slots, *shape]``, zeroed when a slot is opened."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CapacityError(RuntimeError):
    """A sequence would grow beyond the positions the model or the cache allows."""


@dataclass
class LayerKV:
    """What an attention kernel needs to find a layer's keys and values."""
    storage: torch.Tensor        # [pages, 2, kv_heads, page_size, head_dim] of this layer
    block_table: torch.Tensor    # [slots, width] int32, shared by the group
    page_size: int
    ring_pages: int              # 0 = one table entry per page of positions; R = ring of R entries
    window: int
    group: int


class KVGroup:
    def __init__(self, index: int, request: KVRequest, layers: List[int], n_pages: int, n_slots: int,
                 page_size: int, max_pages_per_seq: int, dtype: torch.dtype, device):
        self.index = index
        self.request = request
        self.layers = layers
        self.page_size = page_size
        ring = -(-request.window // page_size) + 1 if request.window > 0 else 0
        self.ring_pages = ring if 0 < ring < max_pages_per_seq else 0
        self.width = self.ring_pages or max_pages_per_seq
        self.pool = FreeList(n_pages, f"page of group {index}")
        self.pages_of: List[List[int]] = [[] for _ in range(n_slots)]
        self.table_host = np.zeros((n_slots, self.width), dtype=np.int32)
        self.block_table = torch.zeros((n_slots, self.width), dtype=torch.int32, device=device)
        self.storage = torch.zeros((len(layers), n_pages, 2, request.n_kv_heads, page_size, request.head_dim),
                                   dtype=dtype, device=device)
        self.dirty: set = set()

    def pages_needed(self, length: int) -> int:
        n = -(-length // self.page_size)
        return min(n, self.ring_pages) if self.ring_pages else n

    def grow(self, slot: int, length: int) -> int:
        """Take the pages that ``length`` positions need beyond those held; returns how many."""
        held = self.pages_of[slot]
        need = self.pages_needed(length) - len(held)
        if need <= 0:
            return 0
        new = self.pool.take(need)
        for p in new:
            self.table_host[slot, len(held)] = p
            held.append(p)
        self.dirty.add(slot)
        return need

    def shrink(self, slot: int, count: int) -> None:
        """Undo the last ``count`` pages of ``grow`` (used when another group could not grow)."""
        held = self.pages_of[slot]
        back = [held.pop() for _ in range(count)]
        self.pool.give(back)

    def release(self, slot: int) -> None:
        self.pool.give(self.pages_of[slot])
        self.pages_of[slot] = []

    def flush(self) -> None:
        if not self.dirty:
            return
        rows = sorted(self.dirty)
        idx = torch.as_tensor(rows, dtype=torch.long, device=self.block_table.device)
        self.block_table.index_copy_(0, idx, torch.from_numpy(self.table_host[rows]).to(self.block_table.device))
        self.dirty.clear()

    def nbytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


class KVCache:
    """Slots, pages and per-sequence state of one model.

    ``requests[i]`` is what the mixer at site ``i`` (the i-th entry of the model's schedule; "layer"
    below) asks for: a list of ``KVRequest`` / ``StateRequest`` (possibly empty).  ``shares[i] = j``
    lets site ``i`` read site ``j``'s keys and values instead of holding its own.  ``max_tokens`` is the most positions that live
    sequences hold at any time, each sequence's count rounded up to ``page_size``.
    """

    def __init__(self, requests: Sequence[Sequence[object]], max_tokens: int, max_position: int,
                 dtype: torch.dtype, device, page_size: int = 64, max_seqs: Optional[int] = None,
                 shares: Optional[Dict[int, int]] = None, extra_state: Sequence[StateRequest] = ()):
        if page_size <= 0 or page_size % 16:
            raise ValueError(f"page_size {page_size} must be a positive multiple of 16")
        if max_tokens <= 0:
            raise ValueError(f"max_tokens {max_tokens} must be positive")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_tokens = self.n_pages * page_size
        self.max_position = max_position
        self.n_slots = max(1, min(self.n_pages, max_seqs if max_seqs else 4096))
        self.max_pages_per_seq = -(-min(self.max_tokens, max_position) // page_size)
        self.dtype = dtype
        self.device = device
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths = np.zeros(self.n_slots, dtype=np.int64)
        self.groups: List[KVGroup] = []
        self._layer_group: Dict[int, Tuple[int, int]] = {}
        self.state: Dict[str, torch.Tensor] = {}
        self.has_mixer_state = False      # a mixer keeps state of fixed size per sequence (it cannot be rewound)
        shares = dict(shares or {})
        by_key: Dict[KVRequest, List[int]] = {}
        for layer, reqs in enumerate(requests):
            for r in reqs:
                if isinstance(r, KVRequest):
                    if layer in shares:
                        raise ValueError(f"layer {layer} both asks for keys/values and reads layer {shares[layer]}'s")
                    by_key.setdefault(r, []).append(layer)
                elif isinstance(r, StateRequest):
                    self._add_state(r)
                    self.has_mixer_state = True
                else:
                    raise TypeError(f"layer {layer}: unknown cache request {r!r}")
        for r in extra_state:
            self._add_state(r)
        for gi, (req, layers) in enumerate(by_key.items()):
            g = KVGroup(gi, req, layers, self.n_pages, self.n_slots, page_size, self.max_pages_per_seq, dtype, device)
            self.groups.append(g)
            for li, layer in enumerate(layers):
                if layer in self._layer_group:
                    raise ValueError(f"layer {layer} asks for keys and values twice")
                self._layer_group[layer] = (gi, li)
        for layer, src in shares.items():
            if src not in self._layer_group:
                raise ValueError(f"layer {layer} reads the cache of layer {src}, which holds none")
            self._layer_group[layer] = self._layer_group[src]

    # ------------------------------------------------------------------ state
    def _add_state(self, r: StateRequest) -> None:
        if r.name in self.state:
            raise ValueError(f"per-sequence state '{r.name}' is asked for twice")
        self.state[r.name] = torch.zeros((self.n_slots, *r.shape), dtype=r.dtype, device=self.device)

    # ------------------------------------------------------------------ views
    def layer_kv(self, layer: int) -> LayerKV:
        gi, li = self._layer_group[layer]
        g = self.groups[gi]
        return LayerKV(storage=g.storage[li], block_table=g.block_table, page_size=self.page_size,
                       ring_pages=g.ring_pages, window=g.request.window, group=gi)

    def most_tokens_going_on(self) -> Optional[int]:
        """The most tokens that a sequence which already holds positions may add in one step whose rows read the
        cache, or None for no limit.  A window group keeps a ring of ceil(w / page) + 1 pages: the step's keys are
        all appended before any row reads, so a row's oldest key survives only while the step adds at most a page."""
        return self.page_size if any(g.ring_pages for g in self.groups) else None

    def has_kv(self, layer: int) -> bool:
        return layer in self._layer_group

    def nbytes(self) -> int:
        return (sum(g.nbytes() for g in self.groups)
                + sum(t.numel() * t.element_size() for t in self.state.values()))

    # ------------------------------------------------------------------ slots
    def open(self, count: int) -> List[int]:
        """Slots for ``count`` new sequences, empty, their state zeroed."""
        got = self.slots.take(count)
        for s in got:
            assert self.lengths[s] == 0 and all(not g.pages_of[s] for g in self.groups), \
                f"slot {s} was handed out with contents"
        if got and self.state:
            idx = torch.as_tensor(got, dtype=torch.long, device=self.device)
            for t in self.state.values():
                t.index_fill_(0, idx, 0)
        return got

    def reserve(self, slot: int, length: int) -> None:
        """Make room for ``slot`` to hold ``length`` positions; all or nothing."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not open")
        if length > self.max_position:
            raise CapacityError(f"slot {slot}: {length} positions exceed the model's max_position {self.max_position}")
        if length < self.lengths[slot]:
            raise ValueError(f"slot {slot}: a sequence of {self.lengths[slot]} positions cannot shrink to {length}")
        grown: List[Tuple[KVGroup, int]] = []
        try:
            for g in self.groups:
                grown.append((g, g.grow(slot, length)))
        except CacheFull as e:
            for g, n in grown:
                if n:
                    g.shrink(slot, n)
            raise CacheFull(f"slot {slot} cannot grow to {length} positions: {e} "
                            f"(the cache holds {self.max_tokens} positions in pages of {self.page_size})") from e

    def must_fit(self, wanted: Sequence[Tuple[int, int]]) -> None:
        """Raise (``CapacityError`` / ``CacheFull``) unless every (slot, length) of ``wanted`` can be reserved
        together; takes nothing.  A step asks this before it reserves anything, so one that does not fit leaves
        no sequence with pages it did not commit."""
        for slot, length in wanted:
            if length > self.max_position:
                raise CapacityError(f"slot {slot}: {length} positions exceed the model's max_position {self.max_position}")
        for g in self.groups:
            need = sum(max(0, g.pages_needed(length) - len(g.pages_of[slot])) for slot, length in wanted)
            if need > g.pool.free:
                raise CacheFull(f"the step needs {need} more pages of group {g.index}, {g.pool.free} are free "
                                f"(the cache holds {self.max_tokens} positions in pages of {self.page_size})")

    def commit(self, slot: int, length: int) -> None:
        """Record that ``slot`` now holds ``length`` positions (after the step that wrote them)."""
        for g in self.groups:
            if len(g.pages_of[slot]) < g.pages_needed(length):
                raise ValueError(f"slot {slot}: {length} positions committed but not reserved")
        self.lengths[slot] = length

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    def can_rewind(self, slot: int, length: int) -> bool:
        """Whether ``slot`` may go back to its first ``length`` positions and go on from there.  Always to where it
        is; further back only if every group keeps all keys (a ring has overwritten old ones) and no mixer keeps
        state of its own (which belongs to the sequence's end)."""
        held = int(self.lengths[slot])
        if length == held:
            return True
        return 0 <= length < held and not self.has_mixer_state and not any(g.ring_pages for g in self.groups)

    def rewind(self, slot: int, length: int) -> None:
        """Forget the positions from ``length`` on (their pages stay with the slot and are written again)."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not open")
        if not self.can_rewind(slot, length):
            raise ValueError(f"slot {slot} holds {int(self.lengths[slot])} positions and cannot go back to {length}")
        self.lengths[slot] = length

    def free_tokens(self) -> int:
        """Positions that the free pages could still hold (the scarcest group decides)."""
        return min((g.pool.free for g in self.groups), default=self.n_pages) * self.page_size

    def held_tokens(self, slot: int) -> int:
        """Positions that the pages of ``slot`` hold room for (the group with the fewest pages decides)."""
        return min((len(g.pages_of[slot]) for g in self.groups), default=0) * self.page_size

    def close(self, slots: Sequence[int]) -> None:
        """Give the slots and their pages back; later sequences use them again."""
        slots = list(slots)
        for s in slots:
            if not self.slots.is_held(s):
                raise ValueError(f"slot {s} is closed but is not open")
        self.slots.give(slots)
        for s in slots:
            for g in self.groups:
                g.release(s)
            self.lengths[s] = 0

    def flush(self) -> None:
        """Bring the device's block tables up to date with the host's."""
        for g in self.groups:
            g.flush()

    def check(self) -> None:
        """Invariants of the bookkeeping (tests call this after every operation)."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            seen = set()
            for s in range(self.n_slots):
                pages = g.pages_of[s]
                if not self.slots.is_held(s):
                    assert not pages, f"closed slot {s} holds pages in group {g.index}"
                for p in pages:
                    assert p not in seen, f"page {p} of group {g.index} is held twice"
                    assert g.pool.is_held(p), f"page {p} of group {g.index} is in a table but free"
                    seen.add(p)
                assert len(pages) >= g.pages_needed(int(self.lengths[s])), f"slot {s} holds too few pages"
            assert len(seen) == g.pool.held, f"group {g.index}: {g.pool.held - len(seen)} page(s) held by no slot"
