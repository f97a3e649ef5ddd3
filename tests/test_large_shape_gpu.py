"""The Qwen2.5-7B layer shape (hidden 3584, 28/4 heads of 128, intermediate 18944) with two layers and a
smaller vocabulary: the kernels at the sizes the benchmark runs them, against the plain implementation
(float64, CPU) and against each other in every cutting."""
import tempfile

import pytest
import torch

import cima_b200
from cima_b200.engine import load_model
from helpers import random_tokens, run_batched, run_tail_one_by_one, run_whole
from qwen2_plain import plain_forward, plain_load

pytestmark = pytest.mark.gpu

# The tiny models' bfloat16 tolerance (2e-2 on logits whose standard deviation is 0.28) as a fraction of
# the logits' standard deviation; at this width the logits are about four times larger.
REL_BF16 = 2e-2 / 0.28

SHAPE = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584,
             num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
             vocab_size=20008, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
             use_sliding_window=False, max_position_embeddings=4096)


@pytest.fixture(scope="module")
def folder():
    d = tempfile.mkdtemp(prefix="cima_7bshape_")
    cima_b200.write_random_model(d, SHAPE, seed=11)
    return d


def test_7b_layer_shape_in_every_cutting(folder):
    cfg, W = plain_load(folder)
    toks = random_tokens(SHAPE["vocab_size"], 100, seed=1)
    want = plain_forward(W, cfg, toks).float()
    m32 = load_model(folder, dtype="float32", max_tokens=4096, verbose=False)
    whole32 = run_whole(m32, toks)
    # sums over 3584 to 18944 float32 terms, two layers, logits of magnitude about 1
    assert (whole32 - want).abs().max().item() <= 1e-4
    assert torch.equal(run_tail_one_by_one(m32, toks, 32), whole32)
    del m32
    torch.cuda.empty_cache()
    m16 = load_model(folder, dtype="bfloat16", max_tokens=4096, verbose=False)
    tol = REL_BF16 * want.std().item()
    whole16 = run_whole(m16, toks)
    assert (whole16 - want).abs().max().item() <= tol
    assert (run_tail_one_by_one(m16, toks, 32) - want).abs().max().item() <= tol
    seqs = [random_tokens(SHAPE["vocab_size"], n, seed=20 + n) for n in (70, 9, 130, 31)] + [toks]
    got = run_batched(m16, seqs, [60, 1, 100, 20, 68])
    assert (got[4] - want).abs().max().item() <= tol
    for q, g in zip(seqs[:2], got[:2]):
        assert (g - plain_forward(W, cfg, q).float()).abs().max().item() <= tol
    m16.cache.check()


def test_long_context_decode_against_whole_prompt(folder):
    """3,000 positions: the last 8 tokens one by one (split-KV decode attention over 47 pages) against the
    same positions of the whole prompt (flash prefill), bfloat16; both against float32 at the end."""
    toks = random_tokens(SHAPE["vocab_size"], 3000, seed=3)
    m16 = load_model(folder, dtype="bfloat16", max_tokens=4096, verbose=False)
    (slot,) = m16.cache.open(1)
    from cima_b200.engine import StepEntry
    try:
        whole = m16.step([StepEntry(slot, toks, list(range(2992, 3000)))]).float().cpu()
    finally:
        m16.cache.close([slot])
    (slot,) = m16.cache.open(1)
    try:
        m16.step([StepEntry(slot, toks[:2992], [])])
        tail = torch.cat([m16.step([StepEntry(slot, [t], [0])]).float().cpu() for t in toks[2992:]])
    finally:
        m16.cache.close([slot])
    tol = REL_BF16 * whole.std().item()
    assert (tail - whole).abs().max().item() <= tol
    del m16
    torch.cuda.empty_cache()
    m32 = load_model(folder, dtype="float32", max_tokens=4096, verbose=False)
    (slot,) = m32.cache.open(1)
    try:
        ref = m32.step([StepEntry(slot, toks, list(range(2992, 3000)))]).float().cpu()
    finally:
        m32.cache.close([slot])
    assert (whole - ref).abs().max().item() <= tol and (tail - ref).abs().max().item() <= tol


WIDER = {"14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824),
         "32b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648)}


@pytest.mark.parametrize("name", ["14b", "32b"])
def test_wider_layer_shapes(name, tmp_path):
    """One layer of the Qwen2.5-14B and -32B shapes (hidden 5120: 320 partial sums per row for the folded norm,
    more than the 256 a lane's registers take; 40/8 heads; intermediate 13,824 or 27,648): a prompt whole, its
    last 16 tokens one by one, and a 300-token prompt (the tcgen05 attention) in bfloat16 against float32."""
    shape = dict(SHAPE, num_hidden_layers=1, vocab_size=5000, **WIDER[name])
    folder = str(tmp_path / name)
    cima_b200.write_random_model(folder, shape, seed=13)
    cfg, W = plain_load(folder)
    toks = random_tokens(shape["vocab_size"], 72, seed=2)
    want = plain_forward(W, cfg, toks).float()
    long_toks = random_tokens(shape["vocab_size"], 300, seed=4)
    m32 = load_model(folder, dtype="float32", max_tokens=1024, verbose=False)
    whole32 = run_whole(m32, toks)
    assert (whole32 - want).abs().max().item() <= 1e-4
    # 32-bit: the last 16 one by one and a batch of three unequal requests, bit for bit the whole prompt's logits
    assert torch.equal(run_tail_one_by_one(m32, toks, 16), whole32)
    others = [random_tokens(shape["vocab_size"], n, seed=50 + n) for n in (9, 40)]
    got = run_batched(m32, [toks] + others, [60, 1, 33])
    assert torch.equal(got[0], whole32)
    for q, g in zip(others, got[1:]):
        assert (g - plain_forward(W, cfg, q).float()).abs().max().item() <= 1e-4
    long32 = run_whole(m32, long_toks)
    del m32
    torch.cuda.empty_cache()
    m16 = load_model(folder, dtype="bfloat16", max_tokens=1024, verbose=False)
    tol = REL_BF16 * want.std().item()
    assert (run_whole(m16, toks) - want).abs().max().item() <= tol
    assert (run_tail_one_by_one(m16, toks, 16) - want).abs().max().item() <= tol
    assert (run_whole(m16, long_toks) - long32).abs().max().item() <= REL_BF16 * long32.std().item()
    m16.check_device()


def test_ragged_long_prompts_in_one_step(folder):
    """Five prompts of 1 to 700 tokens in one step (the longest decides that the tcgen05 attention runs: blocks
    of 128 query rows, sequences that end inside a block, one of a single token), bfloat16 against float32, at
    every sequence's last position and at a few inside."""
    from cima_b200.engine import StepEntry
    lens = [700, 130, 1, 257, 300]
    seqs = [random_tokens(SHAPE["vocab_size"], n, seed=40 + n) for n in lens]
    wants = [sorted({0, n // 2, max(0, n - 2), n - 1}) for n in lens]

    def run(dtype):
        m = load_model(folder, dtype=dtype, max_tokens=2048, verbose=False)
        slots = m.cache.open(len(seqs))
        try:
            out = m.step([StepEntry(s, t, w) for s, t, w in zip(slots, seqs, wants)]).float().cpu()
            m.check_device()
        finally:
            m.cache.close(slots)
        del m
        torch.cuda.empty_cache()
        return out

    got16, got32 = run("bfloat16"), run("float32")
    assert got16.shape == got32.shape == (sum(len(w) for w in wants), SHAPE["vocab_size"])
    assert (got16 - got32).abs().max().item() <= REL_BF16 * got32.std().item()


def test_a_300_token_prompt_at_the_7b_layer_shape_against_the_plain_implementation(folder):
    """One 300-token prompt through two layers in bfloat16, directly against the plain implementation (not by way of
    the 32-bit engine): the attention on its tcgen05 kernel, the gated projection on the library (its 300 rows would
    leave most of a second tile of 256 empty); then the prompt's first 256 tokens, whose gated projection runs on the
    tcgen05 pair kernel, against the same logits; then the 32-bit engine beside it."""
    from cima_b200.engine.profile import StepProfile
    cfg, W = plain_load(folder)
    toks = random_tokens(SHAPE["vocab_size"], 300, seed=6)
    want = plain_forward(W, cfg, toks).float()
    m16 = load_model(folder, dtype="bfloat16", max_tokens=1024, verbose=False)
    K = m16.rt.kernels
    for n, pair in ((300, False), (256, True)):
        K.profile = seen = StepProfile()
        try:
            got = run_whole(m16, toks[:n])
        finally:
            K.profile = None
        m16.check_device()
        names = {l.name for l in seen.launches}
        assert ("gemm_tcgen05_pair[2]" in names) == pair and "attention_prefill_tc" in names, names
        # The tolerance bounds the largest error among the 10^5 logits or so that the other tests compare.  Among the six
        # million of 300 rows at this vocabulary the largest error of a sound run reaches it (measured: 0.084 with the
        # kernel and 0.091 with the library product, of 0.086; 5.9 and 6.1 times the error's standard deviation, on
        # different rows from seed to seed).  So it is asked of the rows at the ends and at the tiles' edges, and every
        # row is held to its root mean square instead (measured 0.008 to 0.019, 0.015 over all; a faulty row's is 1).
        tol = REL_BF16 * want.std().item()
        err = got - want[:n]
        edges = [r for r in (0, 1, 127, 128, 255, 256, n - 2, n - 1) if r < n]
        assert err[edges].abs().max().item() <= tol, n
        assert err.pow(2).mean(dim=1).sqrt().max().item() <= tol / 3 and err.pow(2).mean().sqrt().item() <= tol / 4, n
    del m16
    torch.cuda.empty_cache()
    m32 = load_model(folder, dtype="float32", max_tokens=1024, verbose=False)
    assert (run_whole(m32, toks) - want).abs().max().item() <= 1e-4


def test_64_sequences_decode_together_at_the_7b_layer_shape(folder):
    """One decode step of 64 sequences (and of 9 and 16) after prompts of unequal lengths: the schedule for more
    than 8 rows at the benchmark's widths, bfloat16 against the 32-bit engine and, for a few sequences, against the
    plain implementation."""
    from cima_b200.engine import StepEntry
    cfg, W = plain_load(folder)
    gen = torch.Generator().manual_seed(3)
    lens = [int(x) for x in torch.randint(1, 200, (64,), generator=gen)]
    lens[0], lens[1], lens[2] = 1, 64, 199
    seqs = [random_tokens(SHAPE["vocab_size"], n + 3, seed=300 + i) for i, n in enumerate(lens)]

    def run(dtype, count):
        m = load_model(folder, dtype=dtype, max_tokens=64 * 4 * 64, max_seqs=64, verbose=False)
        slots = m.cache.open(count)
        try:
            for i in range(0, count, 16):
                m.step([StepEntry(s, q[:n], []) for s, q, n in zip(slots[i:i + 16], seqs[i:i + 16], lens[i:i + 16])])
            outs = [m.step([StepEntry(s, [q[n + k]], [0]) for s, q, n in zip(slots, seqs, lens)]).float().cpu()
                    for k in range(3)]
        finally:
            m.cache.close(slots)
        del m
        torch.cuda.empty_cache()
        return torch.stack(outs)                      # [3 steps, count, vocab]

    want32 = run("float32", 64)
    tol = REL_BF16 * want32.std().item()
    for i in (0, 1, 2, 63):
        plain = plain_forward(W, cfg, seqs[i]).float()
        for k in range(3):
            assert (want32[k, i] - plain[lens[i] + k]).abs().max().item() <= 1e-4
    for count in (64, 16, 9):
        got = run("bfloat16", count)
        assert (got - want32[:, :count]).abs().max().item() <= tol, count


def test_256_sequences_generate_together_at_the_7b_layer_shape(folder):
    """256 prompts of 1 to 300 tokens as ONE batch through the entry point (recorded decode steps of 256 rows, the
    device sampler's chain and the argmax on 256 rows, sequences that stop at different steps), greedy and through
    the default sampling chain with a generator per request: in 32-bit every request's tokens are those it gets
    in a batch of its own; in bfloat16 every token lies within the tolerance of the 32-bit logits' best."""
    gen = torch.Generator().manual_seed(9)
    lens = [int(x) for x in torch.randint(1, 300, (256,), generator=gen)]
    lens[0], lens[255] = 1, 299
    prompts = [random_tokens(SHAPE["vocab_size"], n, seed=700 + i) for i, n in enumerate(lens)]
    budgets = [1 + (i * 7) % 6 for i in range(256)]
    from cima_b200.sampling import GenOptions
    for chain in (dict(temperature=0.0, repeat_penalty=1.0), dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1)):
        opts = [GenOptions(max_tokens=b, ignore_eos=True, seed=i + 1, **chain) for i, b in enumerate(budgets)]
        lm = cima_b200.load(folder, dtype="float32", max_tokens=256 * 320, max_seqs=256, max_batch=256, verbose=False)
        got = lm.generate(prompts, opts)
        assert lm.stats.batches == 1 and [len(r.tokens) for r in got] == budgets
        for i in (0, 1, 77, 128, 254, 255):
            alone = lm.generate([prompts[i]], [opts[i]])[0]
            assert alone.tokens == got[i].tokens, (i, chain)
        lm.model.cache.check()
        assert lm.model.cache.slots.held == 0
        lm.model.check_device()
        del lm
        torch.cuda.empty_cache()
    # bfloat16, greedy: each token against the 32-bit logits of the same history
    opts = [GenOptions(max_tokens=b, ignore_eos=True, temperature=0.0, repeat_penalty=1.0) for b in budgets]
    lm = cima_b200.load(folder, dtype="bfloat16", max_tokens=256 * 320, max_seqs=256, max_batch=256, verbose=False)
    got = lm.generate(prompts, opts)
    assert lm.stats.batches == 1 and [len(r.tokens) for r in got] == budgets
    lm.model.check_device()
    del lm
    torch.cuda.empty_cache()
    m32 = load_model(folder, dtype="float32", max_tokens=4096, verbose=False)
    from cima_b200.engine import StepEntry
    for i in (0, 5, 77, 128, 200, 255):
        seq = prompts[i] + got[i].tokens
        (slot,) = m32.cache.open(1)
        try:
            places = list(range(len(prompts[i]) - 1, len(seq) - 1))
            lg = m32.step([StepEntry(slot, seq[:-1], places)]).float().cpu()
        finally:
            m32.cache.close([slot])
        tol = REL_BF16 * lg.std().item()
        for k, t in enumerate(got[i].tokens):
            # the chosen token's and the best token's logits are each off by at most the tolerance
            assert lg[k, t].item() >= lg[k].max().item() - 2 * tol, (i, k)


def test_gated_feed_forward_in_row_chunks(folder, monkeypatch):
    """A step whose [rows, 2 x intermediate] scratch would exceed its bound runs the feed-forward in row chunks: with
    the bound set so low that a 300-token prompt takes three chunks, the 32-bit logits are bit for bit those of
    the run in one piece, and bfloat16 stays within its tolerance of them."""
    import cima_b200.parts.feed_forward as ff
    toks = random_tokens(SHAPE["vocab_size"], 300, seed=8)
    outs = {}
    for dtype in ("float32", "bfloat16"):
        m = load_model(folder, dtype=dtype, max_tokens=1024, verbose=False)
        outs[dtype, "whole"] = run_whole(m, toks)
        monkeypatch.setattr(ff, "_SCRATCH_ELEMS", 2 * SHAPE["intermediate_size"] * 128)
        outs[dtype, "chunks"] = run_whole(m, toks)
        monkeypatch.undo()
        del m
        torch.cuda.empty_cache()
    assert torch.equal(outs["float32", "whole"], outs["float32", "chunks"])
    # bfloat16: chunks of 128 rows take the library product and the activation kernel where the whole prompt takes
    # the tcgen05 product with the activation in its epilogue; everything else is the same kernels on the same
    # values, so the two runs differ by the rounding of one layer part and stay within the tolerance of each other,
    # and the chunked run is on average as close to the 32-bit logits as the whole one
    tol = REL_BF16 * outs["float32", "whole"].std().item()
    assert (outs["bfloat16", "chunks"] - outs["bfloat16", "whole"]).abs().max().item() <= tol
    err_chunks = (outs["bfloat16", "chunks"] - outs["float32", "whole"]).abs().mean().item()
    err_whole = (outs["bfloat16", "whole"] - outs["float32", "whole"]).abs().mean().item()
    assert err_chunks <= 1.1 * err_whole


def test_the_full_vocabulary_head_argmax_and_sampler():
    """One layer of the 7B shape with the whole vocabulary of 152,064: the head through the kernel for few rows (1 and
    8 rows) and through the library branch (9 and 64 rows), the argmax and the sampling chain at that width (the
    default chain and temperature only), against the plain implementation: float64 logits of the same rows, and the
    plain sampler on the engine's own float32 logits, draw for draw."""
    import numpy as np
    from cima_b200.engine import StepEntry
    from cima_b200.sampling import GenOptions
    from qwen2_plain import PlainXorshift, plain_sample
    shape = dict(SHAPE, num_hidden_layers=1, vocab_size=152064)
    lm = cima_b200.load(config=shape, seed=17, dtype="bfloat16", max_tokens=64 * 2 * 64, max_seqs=64, verbose=False)
    W = {k: v.detach().cpu().double() for k, v in lm.state_dict().items()}      # float64 once: plain_forward keeps it
    cfg = shape
    V = shape["vocab_size"]
    seqs = [random_tokens(V, 3 + (i % 5), seed=700 + i) for i in range(64)]
    plain_last = {}

    def plain_row(i):
        if i not in plain_last:
            plain_last[i] = plain_forward(W, cfg, seqs[i])[-1].float()
        return plain_last[i]

    K = lm.model.rt.kernels
    for count in (1, 8, 9, 64):
        slots = lm.model.cache.open(count)
        try:
            lm.step([StepEntry(s, q[:-1], []) for s, q in zip(slots, seqs)])
            logits = lm.step([StepEntry(s, [q[-1]], [0]) for s, q in zip(slots, seqs)])       # a decode step of `count` rows
        finally:
            lm.model.cache.close(slots)
        host = logits.float().cpu()
        tol = REL_BF16 * host.std().item()
        for i in sorted({0, count // 2, count - 1}):
            assert (host[i] - plain_row(i)).abs().max().item() <= tol, (count, i)
        # argmax at this width: the reference's tie rule (the higher index) on the engine's own logits
        tokens = torch.empty(count, dtype=torch.int32, device=logits.device)
        K.argmax(logits, tokens)
        for i in range(count):
            row = host[i].numpy()
            best = int(np.flatnonzero(row == row.max())[-1])
            assert int(tokens[i]) == best, (count, i)
    # the sampling chain through generate: every draw is the plain sampler's on the same logits.  The logits of the
    # engine are taken from a step of the same rows; generate then must choose what the plain chain chooses on them
    for opts in (dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=5),
                 dict(temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=6)):
        prompts = seqs[:8]
        slots = lm.model.cache.open(8)
        try:
            logits = lm.step([StepEntry(s, q, [len(q) - 1]) for s, q in zip(slots, prompts)]).float().cpu()
        finally:
            lm.model.cache.close(slots)
        got = lm.generate(prompts, max_tokens=1, **opts)
        from test_sampling_gpu import draw_is_consistent
        for i, (p, r) in enumerate(zip(prompts, got)):
            want = plain_sample(logits[i].tolist(), list(p), opts, PlainXorshift(opts["seed"]))
            # over a flat row of 152,064 masses the device's tree of float32 sums and the host's running sum
            # may land on neighbouring tokens of the sorted order: then the draw must be one the chain can make
            assert r.tokens == [want] or (opts["top_k"] == 0 and draw_is_consistent(
                logits[i].tolist(), list(p), opts, PlainXorshift(opts["seed"]).next_f32(), r.tokens[0])), (opts, i)


def test_unequal_batch_of_prompts_of_1024_to_2048_tokens(folder):
    """The benchmark's own kind of batch: prompts of 1,024, 1,500 and 2,048 tokens in one step, then eight tokens
    each, the shortest request ending first; bfloat16 (tcgen05 attention and gated product, then the decode
    kernels over 16 to 33 pages) against the 32-bit engine at every decoded position and at the prompts' ends."""
    from cima_b200.engine import StepEntry
    lens = [1024, 1500, 2048]
    tails = [3, 8, 6]
    seqs = [random_tokens(SHAPE["vocab_size"], n + t, seed=900 + n) for n, t in zip(lens, tails)]

    def run(dtype):
        m = load_model(folder, dtype=dtype, max_tokens=64 * 80, max_seqs=3, verbose=False)
        slots = m.cache.open(3)
        outs = []
        try:
            outs.append(m.step([StepEntry(s, q[:n], [0, n // 2, n - 1]) for s, q, n in zip(slots, seqs, lens)]).float().cpu())
            for k in range(max(tails)):
                live = [i for i in range(3) if k < tails[i]]
                outs.append(m.step([StepEntry(slots[i], [seqs[i][lens[i] + k]], [0]) for i in live]).float().cpu())
            m.check_device()
        finally:
            m.cache.close(slots)
        m.cache.check()
        del m
        torch.cuda.empty_cache()
        return torch.cat(outs)

    got16, got32 = run("bfloat16"), run("float32")
    assert got16.shape == got32.shape == (9 + sum(tails), SHAPE["vocab_size"])
    assert (got16 - got32).abs().max().item() <= REL_BF16 * got32.std().item()
