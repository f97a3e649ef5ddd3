"""The step's batch as the kernels get it (host side only): rows, positions, sequences, wanted rows, the blocks of
query rows of the two prefill attention kernels, the columns of the transposed V, and what is refused."""
import numpy as np
import pytest

from cima_b200.engine.batch import Q_TILE, Q_TILE_TC, StepEntry, build_batch


def test_prefill_batch_layout():
    entries = [StepEntry(3, list(range(130)), [0, 129]), StepEntry(0, [7], []), StepEntry(5, list(range(300)), [299])]
    b = build_batch(entries, [0, 0, 0], vocab=1000, device="cpu")
    assert b.prefill and b.n_rows == 431 and b.n_seqs == 3 and b.n_want == 3 and b.max_len == 300
    assert b.seq_first_row.tolist() == [0, 130, 131, 431] and b.seq_len.tolist() == [130, 1, 300]
    assert b.seq_slot.tolist() == [3, 0, 5] and b.want_rows.tolist() == [0, 129, 430]
    assert b.row_pos[:3].tolist() == [0, 1, 2] and b.row_pos[130].item() == 0 and b.row_pos[-1].item() == 299
    assert b.row_seq[129].item() == 0 and b.row_seq[130].item() == 1 and b.row_seq[131].item() == 2
    # blocks of 64 query rows, heaviest (latest rows) first; every row of every sequence is in exactly one
    tiles = list(zip(b.q_tile_seq.tolist(), b.q_tile_row0.tolist()))
    assert len(tiles) == b.n_q_tiles == 3 + 1 + 5 and sorted(t[1] for t in tiles) == sorted([0, 64, 128, 0, 0, 64, 128, 192, 256])
    assert [t[1] for t in tiles] == sorted((t[1] for t in tiles), reverse=True)
    covered = {(s, r0 + i) for s, r0 in tiles for i in range(Q_TILE) if r0 + i < [130, 1, 300][s]}
    assert len(covered) == 431
    # blocks of 128 rows for the tcgen05 kernel, and a sequence's first column in the transposed V
    tc = list(zip(b.q_tile_tc_seq.tolist(), b.q_tile_tc_row0.tolist()))
    assert len(tc) == b.n_q_tiles_tc == 2 + 1 + 3 and all(r0 % Q_TILE_TC == 0 for _, r0 in tc)


def test_decode_batch_and_what_is_refused():
    b = build_batch([StepEntry(2, [5], [0]), StepEntry(9, [6], [0])], [40, 7], vocab=10, device="cpu")
    assert not b.prefill and b.n_q_tiles == 0 and b.n_q_tiles_tc == 0
    assert b.row_pos.tolist() == [40, 7] and b.seq_len.tolist() == [41, 8] and b.want_all_in_order
    with pytest.raises(ValueError, match="twice"):
        build_batch([StepEntry(1, [1]), StepEntry(1, [2])], [0, 0], 10, "cpu")
    # a sequence that goes on by several tokens beside one that starts: rows that read the cache, no prompt blocks
    b = build_batch([StepEntry(1, [1, 2, 3], [2]), StepEntry(2, [2, 4])], [7, 0], 10, "cpu")
    assert not b.prefill and b.n_rows == 5 and b.n_seqs == 2 and b.n_q_tiles_tc == 2 and b.max_rows == 3
    assert list(zip(b.q_tile_seq.tolist(), b.q_tile_row0.tolist())) == [(0, 0), (1, 0)]     # blocks of rows, heaviest first
    assert b.row_pos.tolist() == [7, 8, 9, 0, 1] and b.seq_len.tolist() == [10, 2] and b.want_rows.tolist() == [2]
    with pytest.raises(ValueError, match="token ids"):
        build_batch([StepEntry(1, [10])], [0], 10, "cpu")
    with pytest.raises(ValueError, match="wanted place"):
        build_batch([StepEntry(1, [1, 2], [2])], [0], 10, "cpu")
    with pytest.raises(ValueError, match="at least one"):
        build_batch([StepEntry(1, [])], [0], 10, "cpu")
