"""The engine on the GPU against the plain implementation: every way of cutting the same requests,
in 32-bit and in bfloat16, on three tiny configurations that differ in every size and option."""
import numpy as np
import pytest
import torch

from helpers import (TINY, gpu_model, model_folder, random_tokens, run_batched, run_tail_one_by_one, run_whole)
from qwen2_plain import plain_forward, plain_load
from cima_b200.engine import StepEntry

pytestmark = pytest.mark.gpu

# float32: rounding of float32 sums over a few hundred terms and a few layers, on logits of
# magnitude about 1.  bfloat16: activations are rounded to 8 bits of mantissa (2^-8 relative)
# several times per layer.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENGTHS = {"A": 40, "B": 150, "C": 300}

_models = {}


def model_of(name, dtype, max_tokens=2048):
    key = (name, dtype, max_tokens)
    if key not in _models:
        _models[key] = gpu_model(name, dtype, max_tokens=max_tokens)
    return _models[key]


_plain = {}


def plain_logits(name, toks):
    key = (name, tuple(toks))
    if key not in _plain:
        cfg, W = plain_load(model_folder(name))
        _plain[key] = plain_forward(W, cfg, toks).float()
    return _plain[key]


def close(a, b, tol):
    return (a - b).abs().max().item() <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_request(name, dtype):
    toks = random_tokens(TINY[name]["vocab_size"], LENGTHS[name], seed=3)
    m = model_of(name, dtype)
    got = run_whole(m, toks)
    assert close(got, plain_logits(name, toks), TOL[dtype])
    m.cache.check()
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_one_by_one(name, dtype):
    toks = random_tokens(TINY[name]["vocab_size"], LENGTHS[name], seed=3)
    m = model_of(name, dtype)
    got = run_tail_one_by_one(m, toks, 32)
    assert close(got, plain_logits(name, toks), TOL[dtype])
    if dtype == "float32":
        # the 32-bit kernels are row-independent with a fixed order of summation
        assert torch.equal(got, run_whole(m, toks))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(name, dtype):
    """Batches of unequal lengths whose shorter requests end earlier, on a cache with so few slots
    and pages that the second and third batch get slots and pages the first one used."""
    V = TINY[name]["vocab_size"]
    lens = {"A": [7, 1, 13, 40], "B": [1, 9, 30, 64], "C": [130, 3, 70, 41]}[name]
    decode = {"A": 10, "B": 16, "C": 20}[name]
    m = gpu_model(name, dtype, max_tokens=64 * 8, max_seqs=4)
    for rnd in range(3):
        seqs = [random_tokens(V, n + (decode if i != 1 else 2), seed=100 * rnd + i) for i, n in enumerate(lens)]
        got = run_batched(m, seqs, lens)
        for q, g in zip(seqs, got):
            assert close(g, plain_logits(name, q), TOL[dtype]), (name, dtype, rnd, len(q))
        m.cache.check()
        assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """A short prompt, then every further token one by one up to the model's last position."""
    name = "B"
    toks = random_tokens(TINY[name]["vocab_size"], 256, seed=9)
    m = model_of(name, dtype)
    got = run_tail_one_by_one(m, toks, 250)
    assert close(got, plain_logits(name, toks), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_first_tokens(name, dtype):
    """Positions 0, 1, 2 fed one by one from an empty slot, and a one-token prompt."""
    toks = random_tokens(TINY[name]["vocab_size"], 3, seed=5)
    m = model_of(name, dtype)
    got = run_tail_one_by_one(m, toks, 3)
    assert close(got, plain_logits(name, toks), TOL[dtype])
    assert close(run_whole(m, toks[:1]), plain_logits(name, toks[:1]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_does_not_change_a_row(dtype):
    """The same request alone and among others, in another slot: float32 bit for bit."""
    name = "C"
    V = TINY[name]["vocab_size"]
    m = model_of(name, dtype)
    a = random_tokens(V, 90, seed=21)
    alone = run_whole(m, a)
    others = [random_tokens(V, n, seed=30 + n) for n in (5, 200, 64)]
    slots = m.cache.open(4)
    try:
        entries = [StepEntry(slots[0], others[0], []), StepEntry(slots[1], others[1], []),
                   StepEntry(slots[3], a, list(range(len(a)))), StepEntry(slots[2], others[2], [])]
        among = m.step(entries).float().cpu()
    finally:
        m.cache.close(slots)
    if dtype == "float32":
        assert torch.equal(alone, among)
    else:
        assert close(alone, among, TOL[dtype])


def test_wanted_rows_only():
    m = model_of("B", "float32")
    toks = random_tokens(1000, 50, seed=2)
    full = run_whole(m, toks)
    (slot,) = m.cache.open(1)
    try:
        some = m.step([StepEntry(slot, toks, [49, 0, 7])]).float().cpu()
        none = m.step([StepEntry(slot, [1], [])])
    finally:
        m.cache.close([slot])
    assert torch.equal(some, full[[49, 0, 7]])
    assert tuple(none.shape) == (0, 1000)


def test_step_refuses_bad_tokens_and_overflow():
    from cima_b200.cache import CacheFull, CapacityError
    m = gpu_model("A", "float32", max_tokens=128, max_seqs=2)
    s = m.cache.open(2)
    try:
        m.step([StepEntry(s[0], [1, 2, 3], [])])
        with pytest.raises(ValueError):
            m.step([StepEntry(s[0], [4, 5], []), StepEntry(s[0], [1, 2], [])])   # a slot twice
        with pytest.raises(ValueError):
            m.step([StepEntry(s[0], [600], [])])                                   # token id out of range
        with pytest.raises(CacheFull):
            m.step([StepEntry(s[1], list(range(100)), [])])                        # 2 pages wanted, 1 free
        with pytest.raises(CapacityError):
            m2 = gpu_model("A", "float32", max_tokens=1024)
            (t,) = m2.cache.open(1)
            m2.step([StepEntry(t, list(range(129)), [])])                          # beyond max_position 128
    finally:
        m.cache.close(s)
    m.cache.check()


ODD = [dict(hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16, intermediate_size=130, vocab_size=333),
       dict(hidden_size=104, num_attention_heads=2, num_key_value_heads=1, head_dim=48, intermediate_size=99, vocab_size=1001),
       # head sizes above the tensor-core attention kernels' 128: the plain attention serves both precisions
       dict(hidden_size=96, num_attention_heads=2, num_key_value_heads=1, head_dim=160, intermediate_size=72, vocab_size=300),
       dict(hidden_size=64, num_attention_heads=3, num_key_value_heads=3, head_dim=256, intermediate_size=48, vocab_size=129)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("over", ODD)
def test_widths_and_head_sizes_off_the_fast_paths(over, dtype, tmp_path):
    """Hidden and intermediate widths and a vocabulary that fit none of the 16-byte paths, and head sizes up to
    the largest allowed: a prompt whole, then ten tokens one by one, against the plain implementation."""
    import cima_b200
    from cima_b200.engine import load_model
    cfg = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, rope_theta=10000.0,
               rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False, max_position_embeddings=256, **over)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=3)
    c, W = plain_load(folder)
    toks = random_tokens(cfg["vocab_size"], 70, 0)
    want = plain_forward(W, c, toks).float()
    m = load_model(folder, dtype=dtype, max_tokens=512, device="cuda:0", verbose=False)
    (slot,) = m.cache.open(1)
    try:
        assert close(m.step([StepEntry(slot, toks[:60], list(range(60)))]).cpu(), want[:60], TOL[dtype])
        for t in range(60, 70):
            assert close(m.step([StepEntry(slot, [toks[t]], [0])]).cpu()[0], want[t], TOL[dtype]), t
    finally:
        m.cache.close([slot])


def test_a_head_size_outside_the_steps_of_16_is_refused(tmp_path):
    import cima_b200
    cfg = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=1, hidden_size=100,
               num_attention_heads=5, num_key_value_heads=5, head_dim=20, intermediate_size=64, vocab_size=50)
    with pytest.raises(ValueError, match="head_dim 20 must be a multiple of 16"):
        cima_b200.write_random_model(str(tmp_path / "m"), cfg, seed=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sequences_may_go_on_by_several_tokens(name, dtype):
    """Prompts fed in pieces beside sequences that start or go on by one token (in C through the window's ring,
    a long piece in rounds of a page): the logits of the whole sequences."""
    from helpers import run_in_pieces
    cfg = TINY[name]
    m = model_of(name, dtype)
    lens = {"A": [100, 37, 64], "B": [150, 33, 90], "C": [230, 41, 130]}[name]
    seqs = [random_tokens(cfg["vocab_size"], n, seed=20 + i) for i, n in enumerate(lens)]
    cuts = [[20, 33, 34, lens[0] - 10], [1, 2, 30], [max(3, lens[2] - 70)]]
    got = run_in_pieces(m, seqs, cuts)
    for q, g_ in zip(seqs, got):
        assert close(g_, plain_logits(name, q), TOL[dtype])
    m.cache.check()
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,first_windowed", [(1, 0), (64, 1), (65, 2), (128, 0), (16, 3)])
def test_windows_at_the_edges_of_pages(window, first_windowed, dtype, tmp_path):
    """Windows of one key, of exactly one and two pages, and one key more than a page, on all layers or on the later
    ones: whole, the last 150 tokens one by one, in pieces, and in a batch of unequal lengths."""
    import cima_b200
    from helpers import run_in_pieces
    from cima_b200.engine import load_model
    cfg = dict(TINY["C"], sliding_window=window, max_window_layers=first_windowed)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=1)
    c, W = plain_load(folder)
    toks = random_tokens(cfg["vocab_size"], 300, 5)
    want = plain_forward(W, c, toks).float()
    m = load_model(folder, dtype=dtype, max_tokens=2048, device="cuda:0", verbose=False)
    assert close(run_whole(m, toks), want, TOL[dtype])
    assert close(run_tail_one_by_one(m, toks, 150), want, TOL[dtype])
    assert close(run_in_pieces(m, [toks], [[10, 100, 101, 250]])[0], want, TOL[dtype])
    for got in run_batched(m, [toks, toks[:77], toks[:130]], [200, 1, 64]):
        assert close(got, want[:got.shape[0]], TOL[dtype])
    m.cache.check()
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,stored", [("B", "float32"), ("A", "float32"), ("C", "mixed"), ("B", "float16")])
def test_checkpoint_stored_in_32_bit(name, stored, dtype, tmp_path):
    """A tensor stored in 32-bit stays 32-bit on both paths (on the bfloat16 path its products run through the plain
    kernel with bfloat16 activations).  ``mixed``: every second matrix and all vectors in 32-bit, the rest bfloat16.
    ``float16``: random values of 11 bits stored as float16 must reach the 32-bit path exactly (by way of bfloat16
    they would lose three bits); the bfloat16 path rounds them to bfloat16 by design and is not compared."""
    import json
    from safetensors.torch import load_file, save_file
    from cima_b200.engine import load_model
    src = model_folder(name)
    tensors = load_file(f"{src}/model.safetensors")
    out = {}
    if stored == "float16":
        if dtype == "bfloat16":
            pytest.skip("float16 weights are rounded to bfloat16 on the bfloat16 path")
        gen = torch.Generator().manual_seed(3)
        for n, t in sorted(tensors.items()):
            noise = torch.randn(t.shape, generator=gen) * 0.004      # bits that bfloat16 does not hold
            out[n] = (t.float() * (1 + noise)).to(torch.float16).contiguous()
    for i, (n, t) in enumerate(sorted(tensors.items())):
        if stored == "float16":
            break
        wide = stored == "float32" or t.dim() == 1 or i % 2 == 0
        out[n] = t.float().contiguous() if wide else t.contiguous()
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY[name]))
    save_file(out, str(folder / "model.safetensors"))
    c, W = plain_load(str(folder))
    toks = random_tokens(TINY[name]["vocab_size"], 90, 7)
    want = plain_forward(W, c, toks).float()
    m = load_model(str(folder), dtype=dtype, max_tokens=1024, device="cuda:0", verbose=False)
    kept = {t.dtype for b in m.blocks for t in (b.mixer.qkv.weight, b.mixer.out.weight)}
    assert torch.float32 in kept
    if stored == "float16":
        assert torch.equal(m.blocks[0].mixer.out.weight.cpu(), out["model.layers.0.self_attn.o_proj.weight"].float())
    assert close(run_whole(m, toks), want, TOL[dtype])
    assert close(run_tail_one_by_one(m, toks, 32), want, TOL[dtype])
    for got in run_batched(m, [toks, toks[:17], toks[:50]], [60, 1, 40]):
        assert close(got, want[:got.shape[0]], TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_at_head_size_64(dtype, tmp_path):
    """Prompts past 256 tokens at head_dim 64 (in bfloat16 the tcgen05 attention serves them): two ragged prompts in
    one step, then tokens one by one."""
    import cima_b200
    from cima_b200.engine import load_model
    cfg = dict(TINY["B"], max_position_embeddings=1024, num_attention_heads=4, num_key_value_heads=2, hidden_size=256)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=2)
    c, W = plain_load(folder)
    seqs = [random_tokens(cfg["vocab_size"], n, seed=n) for n in (420, 300)]
    m = load_model(folder, dtype=dtype, max_tokens=2048, device="cuda:0", verbose=False)
    got = run_batched(m, seqs, [400, 290])
    for q, g_ in zip(seqs, got):
        assert close(g_, plain_forward(W, c, q).float(), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n_seqs", [("A", 12), ("B", 20), ("A", 64), ("B", 64)])
def test_many_sequences_decode_together(name, n_seqs, dtype):
    """9 to 64 sequences in one decode step (in bfloat16 that is another schedule than for up to 8: library
    products with their own residual, norm and activation kernels, fewer splits of the attention): prompts of 1 to
    64 tokens in one step, then a token each; the shorter ones end earlier; three rounds on a cache with exactly as
    many slots as sequences, so that every slot and most pages are used again."""
    V = TINY[name]["vocab_size"]
    gen = np.random.default_rng(1000 + n_seqs)
    m = gpu_model(name, dtype, max_tokens=64 * 2 * n_seqs, max_seqs=n_seqs)
    for rnd in range(3):
        lens = [int(x) for x in gen.integers(1, 65, size=n_seqs)]
        lens[rnd % n_seqs], lens[(rnd + 5) % n_seqs] = 1, 64
        tails = [int(x) for x in gen.integers(1, 13, size=n_seqs)]
        tails[0], tails[-1] = 12, 2
        seqs = [random_tokens(V, n + t, seed=7000 + 100 * rnd + i) for i, (n, t) in enumerate(zip(lens, tails))]
        got = run_batched(m, seqs, lens)
        for i, (q, g) in enumerate(zip(seqs, got)):
            assert close(g, plain_logits(name, q), TOL[dtype]), (name, dtype, rnd, i, len(q))
        if dtype == "float32" and rnd == 0:
            for i in range(0, n_seqs, 7):
                assert torch.equal(got[i], run_whole(m, seqs[i])), i      # alone and whole: bit for bit
        m.cache.check()
        assert m.cache.slots.held == 0


def standout_model(folder):
    """Tiny B with weights made so that single keys carry a row: five marker tokens S_i (ids 901..905) and a query
    token Q (id 900).  An S_i's embedding has one large component in a dimension of its own (all other tokens have
    0 there); layer 0's key projection turns any of those dimensions into one large component of the key, in the
    rotary pair of the lowest frequency (so that the distance between query and key hardly matters); its value
    projection turns each into a large vector of its own; Q's embedding has such a dimension that layer 0's query
    projection turns into the matching component of every head's query.  A Q row's score with an S key then stands
    about 4 above its scores with ordinary keys, and the S keys before it hold two thirds of its weight."""
    import json
    from safetensors.torch import load_file, save_file
    name, hd = "B", 64
    W = dict(load_file(f"{model_folder(name)}/model.safetensors"))
    Q, dq, S, dks = 900, 7, [901, 902, 903, 904, 905], [11, 12, 13, 14, 15]
    alpha, beta, big, vscale, r = 0.2, 0.9, 0.5, 0.15, hd // 2 - 1
    E = W["model.embed_tokens.weight"].float().clone()
    wq, wk, wv = (W[f"model.layers.0.self_attn.{n}_proj.weight"].float().clone() for n in "qkv")
    n1 = W["model.layers.0.input_layernorm.weight"].float().clone()
    gen = torch.Generator().manual_seed(1)
    for d in [dq] + dks:
        E[:, d] = 0
        wq[:, d] = 0
        wk[:, d] = 0
        n1[d] = 1
    E[Q, dq] = big
    for h in range(TINY[name]["num_attention_heads"]):
        wq[h * hd + r, dq] = alpha
    for t, d in zip(S, dks):
        E[t, d] = big
        wk[r, d] = beta
        wv[:, d] = torch.randn(hd, generator=gen) * vscale
    W["model.embed_tokens.weight"] = E.to(torch.bfloat16)
    for n, w in zip("qkv", (wq, wk, wv)):
        W[f"model.layers.0.self_attn.{n}_proj.weight"] = w.to(torch.bfloat16)
    W["model.layers.0.input_layernorm.weight"] = n1.to(torch.bfloat16)
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY[name]))
    save_file({k: v.contiguous() for k, v in W.items()}, str(folder / "model.safetensors"))
    return Q, S


def test_keys_that_stand_out_in_bfloat16(tmp_path):
    """A masking fault of one key moves a bfloat16 logit by less than the model tests' tolerance while every key
    weighs about 1/300.  Here single keys carry a fifth to a whole of a row's weight (``standout_model``), at the
    places where tiles, pages and splits begin and end: positions 0, 63, 64, 127, 128, read by query rows at 1, 65,
    129, 130 and the last position.  First the plain side shows that forgetting any one of those keys moves the
    rows' logits by more than ten times the tolerance; then every cutting must agree with the plain logits."""
    import math
    import qwen2_plain
    from helpers import run_in_pieces
    from cima_b200.engine import load_model
    Q, S = standout_model(tmp_path / "m")
    cfg, W = plain_load(str(tmp_path / "m"))
    toks = random_tokens(900, 200, seed=77)
    spos, qpos = [0, 63, 64, 127, 128], [1, 65, 129, 130, 199]
    for p, t in zip(spos, S):
        toks[p] = t
    for p in qpos:
        toks[p] = Q
    want = plain_forward(W, cfg, toks).float()
    tol = TOL["bfloat16"]

    def without_key(j):
        def attention(q, k, v, window=0):
            T, nh, hd = q.shape
            out = torch.zeros_like(q)
            for h in range(nh):
                for p in range(T):
                    keep = [i for i in range(p + 1) if not (i == j and p > j)]
                    w = torch.softmax((k[keep, h // (nh // k.shape[1]), :] @ q[p, h, :]) / math.sqrt(hd), dim=0)
                    out[p, h, :] = w @ v[keep, h // (nh // k.shape[1]), :]
            return out
        return attention

    whole = qwen2_plain.plain_attention
    try:
        for j in spos:
            qwen2_plain.plain_attention = without_key(j)
            moved = (plain_forward(W, cfg, toks).float() - want).abs().max(dim=1).values
            assert all(moved[p].item() > 10 * tol for p in qpos if p > j), (j, moved[qpos])
    finally:
        qwen2_plain.plain_attention = whole

    m = load_model(str(tmp_path / "m"), dtype="bfloat16", max_tokens=4096, device="cuda:0", verbose=False)
    assert close(run_whole(m, toks), want, tol)
    assert close(run_tail_one_by_one(m, toks, 140), want, tol)          # decoding across the page edges 64, 128, 192
    assert close(run_in_pieces(m, [toks], [[63, 64, 65, 128, 129]])[0], want, tol)
    # in batches: 13 sequences (the schedule for more than 8 rows) that decode across the marked places
    seqs = [toks, toks[:66], toks[:131], toks[:2]] + [toks[:140 + 5 * i] for i in range(9)]
    for got in run_batched(m, seqs, [120, 64, 128, 1] + [60 + i for i in range(9)]):
        assert close(got, want[:got.shape[0]], tol)
    for got in run_batched(m, seqs[:5], [127, 63, 129, 1, 100]):
        assert close(got, want[:got.shape[0]], tol)


def test_a_step_that_does_not_fit_takes_nothing():
    """A step whose second entry overflows the cache leaves the first entry's slot without pages it did not
    commit; a long piece that would be run in rounds is refused before its first round."""
    from cima_b200.cache import CacheFull
    m = gpu_model("A", "float32", max_tokens=64 * 3, max_seqs=3)
    s = m.cache.open(2)
    try:
        free = m.cache.free_tokens()
        with pytest.raises(CacheFull):
            m.step([StepEntry(s[0], list(range(100)), []), StepEntry(s[1], list(range(100)), [])])   # 4 pages, 3 free
        assert m.cache.free_tokens() == free and m.cache.length(s[0]) == 0 and m.cache.held_tokens(s[0]) == 0
        m.cache.check()
    finally:
        m.cache.close(s)
    m = gpu_model("C", "float32", max_tokens=64 * 4, max_seqs=2)        # windows: a long piece runs in rounds of a page
    s = m.cache.open(2)
    try:
        m.step([StepEntry(s[0], list(range(10)), []), StepEntry(s[1], list(range(10)), [])])
        free = m.cache.free_tokens()
        with pytest.raises(CacheFull):
            m.step([StepEntry(s[0], list(range(150)), []), StepEntry(s[1], list(range(100)), [])])
        assert m.cache.free_tokens() == free and m.cache.length(s[0]) == 10 and m.cache.length(s[1]) == 10
        m.cache.check()
    finally:
        m.cache.close(s)
