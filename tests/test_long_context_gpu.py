"""Contexts as long as the configuration allows (32,768 positions), at the 7B layer shape with 2 layers: the
tcgen05 attention over hundreds of key tiles, prompts that go on from hundreds of pages, split decode over 512
pages, sequences of very unequal lengths in one batch, and the last position the model may hold.  At these
lengths the plain implementation (a loop over queries) is out of reach, so the bfloat16 engine is compared with
the 32-bit engine, whose kernels are others (one warp per row and head, no tensor core) and which the shorter
tests compare with the plain implementation."""
import tempfile

import pytest
import torch

import cima_b200
from cima_b200.cache.kv import CapacityError
from cima_b200.engine import StepEntry, load_model
from helpers import random_tokens

pytestmark = pytest.mark.gpu

REL_BF16 = 2e-2 / 0.28            # the tiny models' bfloat16 tolerance as a fraction of the logits' spread
MAXPOS = 32768
SHAPE = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584,
             num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
             vocab_size=20008, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
             use_sliding_window=False, max_position_embeddings=MAXPOS)
TOKENS = random_tokens(SHAPE["vocab_size"], MAXPOS, seed=77)
PLACES = [0, 63, 64, 4095, 16383, 16384, 24000, MAXPOS - 2, MAXPOS - 1]


@pytest.fixture(scope="module")
def folder():
    d = tempfile.mkdtemp(prefix="cima_long_")
    cima_b200.write_random_model(d, SHAPE, seed=5)
    return d


def whole(model, tokens, places):
    (slot,) = model.cache.open(1)
    try:
        out = model.step([StepEntry(slot, tokens, places)]).float().cpu()
        model.check_device()
        return out
    finally:
        model.cache.close([slot])


@pytest.fixture(scope="module")
def exact(folder):
    """The 32-bit engine's logits of the whole 32,768-token prompt at PLACES."""
    m = load_model(folder, dtype="float32", max_tokens=MAXPOS + 64, verbose=False)
    m.step_rows = MAXPOS                           # one step
    out = whole(m, TOKENS, PLACES)
    del m
    torch.cuda.empty_cache()
    return out


@pytest.fixture(scope="module")
def m16(folder):
    return load_model(folder, dtype="bfloat16", max_tokens=MAXPOS + 16384 + 4096 + 256, max_seqs=4, verbose=False)


def test_the_longest_prompt_whole(m16, exact):
    """As the engine runs it (a step of more than 16,384 rows in parts: the second half goes on from 256 pages) and as
    one step of 32,768 rows (the tcgen05 attention over up to 512 key tiles of the step's own rows)."""
    got = whole(m16, TOKENS, PLACES)
    assert (got - exact).abs().max().item() <= REL_BF16 * exact.std().item()
    again = whole(m16, TOKENS, PLACES)              # from other pages' contents left behind: the same bits
    assert torch.equal(got, again)
    bound, m16.step_rows = m16.step_rows, MAXPOS
    try:
        one = whole(m16, TOKENS, PLACES)
    finally:
        m16.step_rows = bound
    assert (one - exact).abs().max().item() <= REL_BF16 * exact.std().item()


def test_the_longest_prompt_in_pieces_and_its_tail_one_by_one(m16, exact):
    """16,384 tokens, then 16,000 that go on from 256 pages, then 380 more, then the last 4 one by one (split decode
    over 512 pages), with the logits at the same places as the whole prompt's; the 32,769th position is refused
    and the refusal takes nothing."""
    cuts = [0, 16384, 32384, MAXPOS - 4]
    (slot,) = m16.cache.open(1)
    try:
        outs = []
        for lo, hi in zip(cuts, cuts[1:]):
            want = [p - lo for p in PLACES if lo <= p < hi]
            outs.append(m16.step([StepEntry(slot, TOKENS[lo:hi], want)]).float().cpu())
        for p in range(MAXPOS - 4, MAXPOS):
            o = m16.step([StepEntry(slot, [TOKENS[p]], [0])]).float().cpu()
            if p in PLACES:
                outs.append(o)
        m16.check_device()
        got = torch.cat(outs)
        assert got.shape == exact.shape
        assert (got - exact).abs().max().item() <= REL_BF16 * exact.std().item()
        free = m16.cache.free_tokens()
        with pytest.raises(CapacityError):
            m16.step([StepEntry(slot, [1], [0])])
        assert m16.cache.length(slot) == MAXPOS and m16.cache.free_tokens() == free
    finally:
        m16.cache.close([slot])
    m16.cache.check()


def test_sequences_of_very_unequal_lengths_decode_together(m16):
    """Prompts of 30,000, 5,000, 130 and 1 tokens in one step, then 6 decode steps of the four together: every
    sequence's logits as when it runs alone (the split of the keys is chosen for the longest; the shortest has
    one page)."""
    lens = [30000, 5000, 130, 1]
    seqs = [TOKENS[i * 100:i * 100 + n + 6] for i, n in enumerate(lens)]

    def run(idx):
        slots = m16.cache.open(len(idx))
        try:
            outs = [m16.step([StepEntry(s, seqs[i][:lens[i]], [lens[i] - 1]) for s, i in zip(slots, idx)]).float().cpu()]
            for k in range(6):
                outs.append(m16.step([StepEntry(s, [seqs[i][lens[i] + k]], [0]) for s, i in zip(slots, idx)]).float().cpu())
            m16.check_device()
            return torch.stack(outs)                 # [7, sequences, vocab]
        finally:
            m16.cache.close(slots)

    together = run([0, 1, 2, 3])
    for i in range(4):
        alone = run([i])[:, 0]
        assert (together[:, i] - alone).abs().max().item() <= REL_BF16 * alone.std().item(), lens[i]
    m16.cache.check()
    assert m16.cache.slots.held == 0


def test_long_tail_in_32_bit(folder, exact):
    """The 32-bit engine: the last 3 of the 32,768 tokens one by one after the rest in two pieces give the whole
    prompt's bits (its attention adds a row's keys in one order, however the tokens were cut)."""
    m = load_model(folder, dtype="float32", max_tokens=MAXPOS + 64, verbose=False)
    (slot,) = m.cache.open(1)
    try:
        m.step([StepEntry(slot, TOKENS[:20000], [])])
        m.step([StepEntry(slot, TOKENS[20000:MAXPOS - 3], [])])
        outs = [m.step([StepEntry(slot, [TOKENS[p]], [0])]).float().cpu() for p in range(MAXPOS - 3, MAXPOS)]
        m.check_device()
    finally:
        m.cache.close([slot])
    got = torch.cat(outs[1:])
    assert torch.equal(got, exact[-2:])


def test_a_window_of_4096_over_20000_positions(tmp_path):
    """The second layer keeps a window of 4,096 keys in a ring of 65 pages: a 20,000-token prompt whole (the window's
    first key tile is far from the block's own), then 700 tokens that go on (rounds of a page), then three tokens
    one by one; bfloat16 against the 32-bit engine, and the 32-bit engine's tail against its own whole prompt."""
    cfg = dict(SHAPE, use_sliding_window=True, sliding_window=4096, max_window_layers=1)
    folder = str(tmp_path / "w")
    cima_b200.write_random_model(folder, cfg, seed=6)
    n, more, tail = 20000, 700, 3
    toks = TOKENS[:n + more + tail]
    places = [0, 4095, 4096, 4097, 8191, 12345, n - 1]

    def run(dtype):
        m = load_model(folder, dtype=dtype, max_tokens=MAXPOS, verbose=False)
        assert any(g.ring_pages for g in m.cache.groups)
        (slot,) = m.cache.open(1)
        try:
            outs = [m.step([StepEntry(slot, toks[:n], places)]).float().cpu()]
            outs.append(m.step([StepEntry(slot, toks[n:n + more], [0, 63, 64, more - 1])]).float().cpu())
            for p in range(n + more, n + more + tail):
                outs.append(m.step([StepEntry(slot, [toks[p]], [0])]).float().cpu())
            m.check_device()
        finally:
            m.cache.close([slot])
        m.cache.check()
        got = torch.cat(outs)
        (slot,) = m.cache.open(1)                    # the whole sequence as one prompt: the same places
        try:
            allp = places + [n, n + 63, n + 64, n + more - 1] + list(range(n + more, n + more + tail))
            one = m.step([StepEntry(slot, toks, allp)]).float().cpu()
        finally:
            m.cache.close([slot])
        del m
        torch.cuda.empty_cache()
        return got, one

    got32, one32 = run("float32")
    assert (got32 - one32).abs().max().item() <= 1e-4          # sums of thousands of float32 terms in another order
    got16, one16 = run("bfloat16")
    tol = REL_BF16 * one32.std().item()
    assert (got16 - one32).abs().max().item() <= tol and (one16 - one32).abs().max().item() <= tol


@pytest.mark.parametrize("dtype,max_tokens", [("bfloat16", 2_700_000), ("float32", 1_400_000)])
def test_pages_far_into_a_large_cache(folder, dtype, max_tokens):
    """A cache of more than 5 GB a layer (2.7 million positions in bfloat16): with the low pages taken away, sequences
    get pages whose bytes lie beyond 4 GB of their layer's storage.  A prompt whole, one in pieces (rows that read the
    pages through the tensor map or the block table), then decode steps of the two together: bit for bit the logits of
    the same run on the first pages, so no kernel cuts a page's address to 32 bits."""
    m = load_model(folder, dtype=dtype, max_tokens=max_tokens, max_seqs=4, verbose=False)
    elt = 2 if dtype == "bfloat16" else 4
    page_bytes = 2 * SHAPE["num_key_value_heads"] * 64 * SHAPE["head_dim"] * elt
    a, b = TOKENS[:700], TOKENS[1000:1600]

    def run():
        slots = m.cache.open(2)
        try:
            outs = [m.step([StepEntry(slots[0], a, [0, 699])]).float().cpu()]
            outs.append(m.step([StepEntry(slots[1], b[:100], [99])]).float().cpu())
            outs.append(m.step([StepEntry(slots[1], b[100:], [0, 499])]).float().cpu())       # goes on by 500 rows
            for k in range(3):
                outs.append(m.step([StepEntry(slots[0], [TOKENS[2000 + k]], [0]),
                                    StepEntry(slots[1], [TOKENS[3000 + k]], [0])]).float().cpu())
            m.check_device()
            pages = [p for g in m.cache.groups for s in slots for p in g.pages_of[s]]
            return torch.cat(outs), min(pages)
        finally:
            m.cache.close(slots)

    low, first_low = run()
    assert first_low == 0
    ballast = [g.pool.take(g.pool.free - 40) for g in m.cache.groups]
    try:
        high, first_high = run()
    finally:
        for g, held in zip(m.cache.groups, ballast):
            g.pool.give(held)
    assert first_high * page_bytes > 5 * 2 ** 30
    assert torch.equal(low, high)
    m.cache.check()
    assert m.cache.slots.held == 0
