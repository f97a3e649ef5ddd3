"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice; rings; shares."""
import random

import pytest
import torch

from cima_b200.cache import CacheFull, CapacityError, FreeList, KVCache, KVRequest, StateRequest


def make(max_tokens=64 * 6, window=0, max_seqs=None, max_position=4096, sites=2, extra=()):
    reqs = [[KVRequest(2, 16, 0)] for _ in range(sites)]
    if window:
        reqs.append([KVRequest(2, 16, window)])
    return KVCache(reqs, max_tokens, max_position, torch.float32, "cpu", max_seqs=max_seqs, extra_state=extra)


def test_free_list_refuses_double_take_and_double_give():
    f = FreeList(3, "slot")
    a = f.take(2)
    assert a == [0, 1] and f.free == 1 and f.held == 2
    with pytest.raises(CacheFull):
        f.take(2)
    assert f.free == 1                         # nothing was taken
    f.give([0])
    with pytest.raises(ValueError, match="not held"):
        f.give([0])
    with pytest.raises(ValueError, match="twice"):
        f.give([1, 1])
    with pytest.raises(ValueError, match="does not exist"):
        f.give([7])
    f.check()
    assert f.take(1) == [0]                    # given back, used again


def test_open_reserve_commit_close_cycle():
    c = make()
    s = c.open(3)
    assert s == [0, 1, 2]
    c.reserve(s[0], 65); c.commit(s[0], 65)
    c.reserve(s[1], 1); c.commit(s[1], 1)
    assert [len(g.pages_of[0]) for g in c.groups] == [2] and c.groups[0].pool.held == 3
    c.check()
    with pytest.raises(ValueError, match="not reserved"):
        c.commit(s[2], 10)
    with pytest.raises(ValueError, match="shrink"):
        c.reserve(s[0], 3)
    c.reserve(s[2], 64 * 3)                    # exactly what is left
    with pytest.raises(CacheFull):
        c.reserve(s[1], 65)
    c.check()
    c.close([s[0]])
    with pytest.raises(ValueError, match="not open"):
        c.close([s[0]])
    with pytest.raises(ValueError, match="not open"):
        c.reserve(s[0], 1)
    c.reserve(s[1], 65)                        # the pages of the closed slot are used again
    (again,) = c.open(1)
    assert again == s[0] and c.length(again) == 0
    c.close([again, s[1], s[2]])
    c.check()
    assert c.slots.held == 0 and all(g.pool.held == 0 for g in c.groups)


def test_all_or_nothing_across_groups():
    """A group that cannot grow undoes what the other groups took in the same call."""
    c = KVCache([[KVRequest(1, 16, 0)], [KVRequest(1, 32, 0)]], 64 * 4, 4096, torch.float32, "cpu")
    assert len(c.groups) == 2
    a, b = c.open(2)
    c.reserve(a, 64 * 3)
    # starve the second group only
    c.groups[1].pool.take(1)
    with pytest.raises(CacheFull):
        c.reserve(b, 64)
    assert c.groups[0].pool.held == 3 and not c.groups[0].pages_of[b] and not c.groups[1].pages_of[b]


def test_window_group_is_a_ring_with_storage_of_its_own():
    c = make(max_tokens=64 * 16, window=100)
    assert len(c.groups) == 2
    full, ring = c.groups
    assert full.ring_pages == 0 and ring.ring_pages == 3 and ring.width == 3 and len(full.layers) == 2
    (s,) = c.open(1)
    c.reserve(s, 1000); c.commit(s, 1000)
    assert len(full.pages_of[s]) == 16 and len(ring.pages_of[s]) == 3
    kv = c.layer_kv(2)
    assert kv.ring_pages == 3 and kv.window == 100 and tuple(kv.storage.shape) == (16, 2, 2, 64, 16)
    assert tuple(c.layer_kv(0).storage.shape) == (16, 2, 2, 64, 16)
    assert c.layer_kv(0).storage.data_ptr() != c.layer_kv(1).storage.data_ptr()
    c.close([s])
    c.check()


def test_a_site_may_read_another_sites_cache():
    c = KVCache([[KVRequest(2, 16, 0)], [], []], 256, 4096, torch.float32, "cpu", shares={2: 0})
    assert c.layer_kv(2).storage.data_ptr() == c.layer_kv(0).storage.data_ptr()
    assert not c.has_kv(1)
    with pytest.raises(ValueError, match="holds none"):
        KVCache([[KVRequest(2, 16, 0)], [], []], 256, 4096, torch.float32, "cpu", shares={2: 1})
    with pytest.raises(ValueError, match="both asks"):
        KVCache([[KVRequest(2, 16, 0)], []], 256, 4096, torch.float32, "cpu", shares={0: 1})


def test_state_is_zeroed_when_a_slot_is_opened():
    c = make(extra=[StateRequest("mine", (3,), torch.float32)])
    (s,) = c.open(1)
    c.state["mine"][s] = 5.0
    c.close([s])
    (t,) = c.open(1)
    assert t == s and c.state["mine"][t].tolist() == [0.0, 0.0, 0.0]
    with pytest.raises(ValueError, match="twice"):
        make(extra=[StateRequest("x", (1,)), StateRequest("x", (1,))])


def test_limits():
    c = make(max_tokens=100)                   # rounded up to pages
    assert c.max_tokens == 128 and c.n_pages == 2 and c.n_slots == 2
    c = make(max_tokens=64 * 100, max_position=128)
    assert c.max_pages_per_seq == 2
    (s,) = c.open(1)
    with pytest.raises(CapacityError):
        c.reserve(s, 129)
    assert make(max_tokens=64 * 10, max_seqs=3).n_slots == 3
    with pytest.raises(CacheFull):
        make(max_tokens=64 * 10, max_seqs=3).open(4)


def test_random_walk_keeps_the_invariants():
    rnd = random.Random(1)
    c = make(max_tokens=64 * 12, window=70, max_seqs=5)
    live = {}
    for _ in range(600):
        op = rnd.random()
        try:
            if op < 0.25 and len(live) < 5:
                (s,) = c.open(1)
                assert s not in live
                live[s] = 0
            elif op < 0.8 and live:
                s = rnd.choice(list(live))
                n = live[s] + rnd.choice([1, 1, 1, 7, 64, 130])
                c.reserve(s, n); c.commit(s, n)
                live[s] = n
            elif live:
                s = rnd.choice(list(live))
                c.close([s])
                del live[s]
        except CacheFull:
            pass
        c.check()
        assert c.slots.held == len(live)
        for s, n in live.items():
            assert c.length(s) == n
        assert c.groups[0].pool.held >= sum(-(-n // 64) for n in live.values())
    c.close(list(live))
    c.check()
    assert all(g.pool.held == 0 for g in c.groups)
