"""The package's host logic (cache, block tables, step function) driven on the CPU through plain
statements of the kernels, compared with the plain implementation."""
import torch
import pytest

from helpers import TINY, cpu_model, model_folder, random_tokens, run_batched, run_tail_one_by_one, run_whole
from qwen2_plain import plain_forward, plain_load
from cima_b200.engine import StepEntry


@pytest.mark.parametrize("name,length", [("A", 21), ("B", 70), ("C", 150)])
def test_whole_tail_and_batch_match_plain(name, length):
    cfg, W = plain_load(model_folder(name))
    model = cpu_model(name, max_tokens=1024)
    toks = random_tokens(cfg["vocab_size"], length, seed=3)
    want = plain_forward(W, cfg, toks).float()
    whole = run_whole(model, toks)
    assert torch.allclose(whole, want, atol=2e-4, rtol=1e-4)
    tail = run_tail_one_by_one(model, toks, min(32, length - 1))
    assert torch.allclose(tail, want, atol=2e-4, rtol=1e-4)
    model.cache.check()
    assert model.cache.slots.held == 0


def test_unequal_batches_reuse_slots():
    name = "C"
    cfg, W = plain_load(model_folder(name))
    model = cpu_model(name, max_tokens=64 * 8, max_seqs=3)
    for rnd in range(2):
        seqs = [random_tokens(cfg["vocab_size"], n, seed=10 * rnd + i) for i, n in enumerate([70, 9, 33])]
        starts = [60, 1, 20]
        got = run_batched(model, seqs, starts)
        for q, g in zip(seqs, got):
            assert torch.allclose(g, plain_forward(W, cfg, q).float(), atol=2e-4, rtol=1e-4)
        model.cache.check()
        assert model.cache.slots.held == 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sequences_may_go_on_by_several_tokens(name):
    """A step may bring several tokens to a sequence that already holds some (a prompt fed in pieces, a second turn
    of a conversation), beside sequences that start or go on by one: the logits are those of the whole sequence.
    In C the later layers keep a ring of pages for their window: pieces longer than a page are fed in rounds."""
    from helpers import run_in_pieces
    cfg, W = plain_load(model_folder(name))
    model = cpu_model(name, max_tokens=1024)
    lens = {"A": [100, 37, 64], "B": [150, 33, 90], "C": [230, 41, 130]}[name]
    seqs = [random_tokens(cfg["vocab_size"], n, seed=20 + i) for i, n in enumerate(lens)]
    cuts = [[20, 33, 34, lens[0] - 10], [1, 2, 30], [max(3, lens[2] - 70)]]      # the third: a start and one long piece
    got = run_in_pieces(model, seqs, cuts)
    for q, g in zip(seqs, got):
        assert torch.allclose(g, plain_forward(W, cfg, q).float(), atol=2e-4, rtol=1e-4)
    model.cache.check()
    assert model.cache.slots.held == 0
    # wanted places out of order and across the rounds of a long piece
    (slot,) = model.cache.open(1)
    try:
        q = seqs[2]
        model.step([StepEntry(slot, q[:5], [])])
        want = [len(q) - 6, 0, min(70, len(q) - 7), 3]
        lg = model.step([StepEntry(slot, q[5:], want)]).float().cpu()
        ref = plain_forward(W, cfg, q).float()
        assert torch.allclose(lg, ref[[5 + w for w in want]], atol=2e-4, rtol=1e-4)
    finally:
        model.cache.close([slot])


@pytest.mark.parametrize("name", ["B", "C"])
def test_a_step_of_more_rows_than_the_bound_runs_in_parts(name):
    """Sequences of 7, 25, 4, 11 and 30 tokens with a bound of 10 rows a step: the short ones run grouped in their
    order, the long ones in rounds (C keeps a window's ring, so its long prompts that start stay whole); two of the
    sequences go on from positions they hold.  The logits are those of the unbounded step, in its order; a token
    outside the vocabulary in the last sequence is refused before any part has run."""
    cfg = TINY[name]
    m = cpu_model(name, max_tokens=1024)
    lens, held = [7, 25, 4, 11, 30], [0, 3, 0, 0, 65]
    seqs = [random_tokens(cfg["vocab_size"], h + n, seed=50 + i) for i, (n, h) in enumerate(zip(lens, held))]
    wants = [[0, n - 1] if i != 2 else [] for i, n in enumerate(lens)]

    def run(bound, spoil=False):
        m.step_rows = bound
        slots = m.cache.open(len(seqs))
        try:
            for s, q, h in zip(slots, seqs, held):
                if h:
                    m.step([StepEntry(s, q[:h], [])])
            entries = [StepEntry(s, list(q[h:]), w) for s, q, h, w in zip(slots, seqs, held, wants)]
            if spoil:
                entries[-1].tokens[-1] = cfg["vocab_size"]
                with pytest.raises(ValueError, match="token ids"):
                    m.step(entries)
                assert [m.cache.length(s) for s in slots] == held
                return None
            out = m.step(entries)
            assert [m.cache.length(s) for s in slots] == [h + n for h, n in zip(held, lens)]
            return out
        finally:
            m.cache.close(slots)
            m.cache.check()

    one = run(1 << 20)
    cut = run(10)
    assert one.shape == cut.shape == (8, cfg["vocab_size"])
    assert (one - cut).abs().max().item() <= 2e-5
    for i, k in ((0, 0), (1, 2), (3, 4), (4, 6)):          # and against the plain implementation, sequence by sequence
        c, W = plain_load(model_folder(name))
        want = plain_forward(W, c, seqs[i]).float()
        assert (cut[k] - want[held[i]]).abs().max().item() <= 2e-5
        assert (cut[k + 1] - want[-1]).abs().max().item() <= 2e-5
    run(10, spoil=True)


def test_bfloat16_plumbing_with_folded_norms():
    """The bfloat16 path's host logic (pending norms handed to the products, sums of squares handed on)
    on the stand-in kernels: one-by-one decoding agrees with whole prompts and with the plain logits."""
    name = "B"
    cfg, W = plain_load(model_folder(name))
    model = cpu_model(name, dtype="bfloat16", max_tokens=512)
    toks = random_tokens(cfg["vocab_size"], 40, seed=4)
    want = plain_forward(W, cfg, toks).float()
    whole = run_whole(model, toks)
    tail = run_tail_one_by_one(model, toks, 20)
    assert (whole - want).abs().max().item() <= 2e-2
    assert (tail - want).abs().max().item() <= 2e-2


def test_a_checkpoint_without_a_head_uses_the_table(tmp_path, capsys):
    """An untied configuration whose file holds no lm_head.weight: the table is the head, with a warning
    (src/models/transformer.rs:810, :839-841); a tied configuration that also stores a head ignores it."""
    import json
    import cima_b200
    from cima_b200.engine import load_model
    from cima_b200.weights import SafetensorsFile, write_safetensors
    from reference_kernels import ReferenceKernels
    src = model_folder("B")                                   # untied, stores lm_head.weight
    sf = SafetensorsFile(f"{src}/model.safetensors")
    tensors = {n: sf.read(n).clone() for n in sf.names()}
    sf.close()
    cfg = dict(TINY["B"])
    toks = random_tokens(cfg["vocab_size"], 20, seed=1)

    def folder(name, cfg_, tensors_):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(cfg_))
        write_safetensors(str(d / "model.safetensors"), tensors_)
        return str(d)

    headless = folder("headless", cfg, {n: t for n, t in tensors.items() if n != "lm_head.weight"})
    model = load_model(headless, dtype="float32", max_tokens=256, device="cpu", kernels=ReferenceKernels())
    assert "lm_head.weight absent" in capsys.readouterr().err
    c, W = plain_load(headless)
    assert torch.allclose(run_whole(model, toks), plain_forward(W, c, toks).float(), atol=2e-4, rtol=1e-4)
    tied_with_head = folder("tied", dict(cfg, tie_word_embeddings=True), tensors)
    model = load_model(tied_with_head, dtype="float32", max_tokens=256, device="cpu", kernels=ReferenceKernels())
    c, W = plain_load(tied_with_head)
    got = run_whole(model, toks)
    assert torch.allclose(got, plain_forward(W, c, toks).float(), atol=2e-4, rtol=1e-4)
    head = plain_forward(dict(W, **{"model.embed_tokens.weight": W["model.embed_tokens.weight"]}), dict(c, tie_word_embeddings=False), toks)
    assert not torch.allclose(got, head.float(), atol=1e-2)   # the stored head was not used


def _lm(name, retain, max_tokens=1024, **kw):
    import cima_b200
    return cima_b200.LM(cpu_model(name, max_tokens=max_tokens, **kw), retain=retain, pipeline=False)


@pytest.mark.parametrize("opts", [dict(temperature=0, repeat_penalty=1.0), dict(temperature=0.9, top_k=20, seed=7)])
def test_finished_sequences_are_taken_up_again(opts):
    """With ``retain`` a finished sequence stays in the cache; a prompt that begins with its tokens runs only what is
    new, and the answers are those of a model that runs everything (src/models/mod.rs:1022-1058 does so for its
    one sequence)."""
    V = TINY["B"]["vocab_size"]
    lm, plain = _lm("B", retain=2), _lm("B", retain=0)
    p1 = random_tokens(V, 40, 1)
    r1 = lm.generate([p1], max_tokens=8, **opts)[0]
    assert lm.stats.reused_tokens == 0 and lm.model.cache.slots.held == 1
    # the next turn: everything so far and something new
    p2 = p1 + r1.tokens + random_tokens(V, 10, 2)
    r2 = lm.generate([p2], max_tokens=8, **opts)[0]
    assert lm.stats.reused_tokens == len(p1) + len(r1.tokens) - 1        # the last token of the answer was never run
    assert r2.tokens == plain.generate([p2], max_tokens=8, **opts)[0].tokens
    # a prompt that shares only the first 30 tokens: the sequence goes back to there
    p3 = p2[:30] + random_tokens(V, 25, 3)
    # ... beside one that shares nothing and one that is all old but for its last token
    p4, p5 = random_tokens(V, 33, 4), p1[:20]
    got = lm.generate([p3, p4, p5], max_tokens=6, **opts)
    assert lm.stats.reused_tokens == 30                                   # p5 found its sequence taken by p3
    want = plain.generate([p3, p4, p5], max_tokens=6, **opts)
    assert [g.tokens for g in got] == [w.tokens for w in want]
    assert lm.model.cache.slots.held == 2                                 # the newest two stay
    lm.model.cache.check()
    lm.stepper.drop_retained()
    assert lm.model.cache.slots.held == 0
    lm.model.cache.check()


def test_kept_sequences_give_way_and_rings_do_not_go_back():
    V = TINY["C"]["vocab_size"]
    opts = dict(temperature=0, repeat_penalty=1.0)
    # C's later layers keep a ring for their window: a sequence is taken up only where it ended
    lm, plain = _lm("C", retain=4, max_tokens=512), _lm("C", retain=0, max_tokens=512)
    p1 = random_tokens(V, 100, 1)
    r1 = lm.generate([p1], max_tokens=5, **opts)[0]
    p2 = p1 + r1.tokens[:-1] + random_tokens(V, 80, 2)                    # goes on where the cache ends
    r2 = lm.generate([p2], max_tokens=5, **opts)[0]
    assert lm.stats.reused_tokens == 104
    assert r2.tokens == plain.generate([p2], max_tokens=5, **opts)[0].tokens
    p3 = p2[:50] + random_tokens(V, 20, 3)                                # would have to go back: runs whole
    r3 = lm.generate([p3], max_tokens=5, **opts)[0]
    assert lm.stats.reused_tokens == 0
    assert r3.tokens == plain.generate([p3], max_tokens=5, **opts)[0].tokens
    # the cache holds 512 positions; the kept sequences (189 and 75 positions: 3 + 2 pages) give way to a batch of 448
    big = [random_tokens(V, 200, 10 + i) for i in range(2)]
    got = lm.generate(big, max_tokens=20, **opts)
    assert [g.tokens for g in got] == [w.tokens for w in plain.generate(big, max_tokens=20, **opts)]
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 2
