"""The device sampling chain against the plain statement of the reference's sampler, draw by draw."""
import numpy as np
import pytest
import torch

from qwen2_plain import PlainXorshift, plain_sample

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cima_b200.kernels import Kernels
    return Kernels(verbose=False)


CASES = [
    dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1),      # the reference's defaults
    dict(temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0),       # plain temperature sampling
    dict(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0),
    dict(temperature=0.0, top_k=40, top_p=0.9, repeat_penalty=1.3),      # greedy after the penalty
    dict(temperature=2.5, top_k=5, top_p=1.0, repeat_penalty=1.0),
    dict(temperature=0.7, top_k=0, top_p=0.5, repeat_penalty=1.0),
    dict(temperature=1.5, top_k=1, top_p=0.9, repeat_penalty=1.0),
    dict(temperature=1.0, top_k=2000, top_p=0.0, repeat_penalty=1.0),    # top_p 0 keeps one token
    dict(temperature=1.2, top_k=1024, top_p=0.95, repeat_penalty=1.05),  # the most that the fast kernel gathers whole
    dict(temperature=1.2, top_k=1025, top_p=1.0, repeat_penalty=1.0),    # one more: the head stands in for the row
]


def draw_is_consistent(logits, history, c, u, got, eps=2e-4):
    """Whether token ``got`` is a draw that the chain can make from ``u``, judged in float64: the chain sums
    tens of thousands of float32 masses, the host one after the other and the device as a tree, so on a flat
    row the cumulated mass at which a draw lands differs in the fifth digit and the neighbouring token of the
    sorted order may come out.  ``got`` must hold the target u * kept within eps of the total mass."""
    l = np.array(logits, dtype=np.float32).copy()
    rp = np.float32(c["repeat_penalty"])
    if rp != 1.0:
        for t in history[-64:]:
            l[t] = l[t] / rp if l[t] > 0 else l[t] * rp
    order = sorted(range(len(l)), key=lambda i: (-float(l[i]), -i))
    k = len(l) if c["top_k"] == 0 else min(c["top_k"], len(l))
    order = order[:k]
    p = np.exp((l[order].astype(np.float64) - float(l[order[0]])) / max(c["temperature"], 1e-4))
    F = np.cumsum(p) / p.sum()
    cut = min(int(np.searchsorted(F, c["top_p"])), len(F) - 1) if c["top_p"] < 1.0 else len(F) - 1
    if got not in order:
        return False
    g = order.index(got)
    target = u * F[cut]
    before = F[g - 1] if g > 0 else 0.0
    return g <= cut + 1 and before - eps <= target <= F[g] + eps


@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("V,spread", [(777, 3.0), (5000, 3.0), (40003, 3.0), (40003, 12.0)])
def test_chain_matches_the_plain_sampler(K, V, spread, general):
    """Every draw equals the plain sampler's.  With a spread of 3 the rows are flat (with top_k = 0 the draw
    often falls behind the 1024 tokens that the fast kernel gathers, and the general kernel settles the row),
    with 12 they are peaked as a model's are (the fast kernel settles them).  ``general``: the one-block-per-row
    kernel, which otherwise serves only vocabularies too long for the fast kernel."""
    if general and V > 10000 and spread < 10:
        pytest.skip("one size of the long rows is enough for the general kernel")
    n_slots, steps = 12, 12 if V < 10000 else 4
    rows = len(CASES)
    slots = [11, 3, 0, 7, 5, 2, 9, 1, 4, 8]
    gen = torch.Generator().manual_seed(V)
    rng = torch.zeros(n_slots, 1, dtype=torch.int64)
    ring = torch.zeros(n_slots, 64, dtype=torch.int32)
    count = torch.zeros(n_slots, 1, dtype=torch.int32)
    plain_rng, history = [], []
    for i, s in enumerate(slots):
        seed = 1000 + i
        rng[s, 0] = seed
        plain_rng.append(PlainXorshift(seed))
        hist = torch.randint(0, V, (5 + 20 * i,), generator=gen).tolist()    # some longer than the ring
        history.append(hist)
        for j, t in enumerate(hist[-64:]):
            ring[s, (len(hist) - len(hist[-64:]) + j) % 64] = t
        count[s, 0] = len(hist)
    rng, ring, count = rng.cuda(), ring.cuda(), count.cuda()
    params = torch.tensor([[c["temperature"], c["top_k"], c["top_p"], c["repeat_penalty"]] for c in CASES],
                          dtype=torch.float32).cuda()
    row_slot = torch.tensor(slots, dtype=torch.int32).cuda()
    work = torch.empty(rows, V, device="cuda")
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    for step in range(steps):
        logits = torch.randn(rows, V, generator=gen) * spread
        logits[:, 5] = logits[:, 400]                  # ties in value
        K.sample(logits.cuda(), row_slot, params, rng, ring, count, work, tokens, general=general)
        got = tokens.tolist()
        for i, c in enumerate(CASES):
            whole_row = c["temperature"] > 0 and (c["top_k"] == 0 or c["top_k"] > 1024)
            if V > 10000 and whole_row:
                # tens of thousands of masses are summed: equal up to the sums' rounding (see draw_is_consistent)
                u = plain_rng[i].next_f32()
                assert draw_is_consistent(logits[i].tolist(), history[i], c, u, got[i]), (V, spread, step, i, c)
                history[i].append(got[i])
                continue
            want = plain_sample(logits[i].tolist(), history[i], c, plain_rng[i])
            assert got[i] == want, (V, spread, step, i, c)
            history[i].append(want)
    # the generators advanced alike (greedy rows draw nothing)
    for i, s in enumerate(slots):
        assert int(np.array(int(rng[s, 0]), dtype=np.int64).astype(np.uint64)) == plain_rng[i].state


def test_draws_follow_the_distribution(K):
    """Frequencies of many draws from one row against the softmax (a check that does not share the
    chain's order of summation)."""
    V, n = 50, 4000
    logits = torch.linspace(-2, 2, V)[None, :].repeat(n, 1).contiguous()
    rng = (torch.arange(n, dtype=torch.int64)[:, None] * 7919 + 12345).cuda()
    ring = torch.zeros(n, 64, dtype=torch.int32).cuda()
    count = torch.zeros(n, 1, dtype=torch.int32).cuda()
    params = torch.tensor([[1.0, 0, 1.0, 1.0]], dtype=torch.float32).repeat(n, 1).cuda()
    row_slot = torch.arange(n, dtype=torch.int32).cuda()
    work = torch.empty(n, V, device="cuda")
    tokens = torch.empty(n, dtype=torch.int32, device="cuda")
    freq = torch.zeros(V)
    for _ in range(5):
        K.sample(logits.cuda(), row_slot, params, rng, ring, count, work, tokens)
        freq += torch.bincount(tokens.cpu().long(), minlength=V).float()
    p = torch.softmax(logits[0], 0)
    # 20000 draws: standard error of a frequency is sqrt(p (1 - p) / N) <= 0.0016
    assert (freq / freq.sum() - p).abs().max().item() < 5 * 0.0016
