"""Generation through the Python entry point and trace replay through bin/trace_run, on the GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import cima_b200
from helpers import TINY, model_folder, random_tokens
from qwen2_plain import PlainXorshift, plain_forward, plain_load, plain_sample

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_generate(name, prompt, opts, n, stop=()):
    cfg, W = plain_load(model_folder(name))
    rng = PlainXorshift(opts.get("seed", 0xC0FFEE))
    seq, out = list(prompt), []
    for _ in range(n):
        logits = plain_forward(W, cfg, seq)[-1].float()
        t = plain_sample(logits.tolist(), seq, opts, rng)
        if t in stop:
            return out, "stop"
        out.append(t)
        seq.append(t)
    return out, "length"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lens,steps", [("A", [7, 1, 13], 10), ("B", [1, 9, 30, 64], 16)])
def test_greedy_generation_matches_plain(name, lens, steps, dtype):
    V = TINY[name]["vocab_size"]
    prompts = [random_tokens(V, n, seed=40 + n) for n in lens]
    lm = cima_b200.load(model_folder(name), dtype=dtype, max_tokens=1024, verbose=False)
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=steps)
    cfg, W = plain_load(model_folder(name))
    for p, r in zip(prompts, got):
        assert r.finish_reason == "length" and len(r.tokens) == steps
        if dtype == "float32":
            assert r.tokens == plain_generate(name, p, dict(temperature=0.0), steps)[0]
        else:
            # bfloat16 may pick another token where two logits are closer than its rounding: every
            # chosen token must be within that of the plain maximum, given the same history
            seq = list(p)
            for t in r.tokens:
                lg = plain_forward(W, cfg, seq)[-1]
                assert lg[t] >= lg.max() - 4e-2
                seq.append(t)
    assert lm.model.cache.slots.held == 0


def test_entry_point_exposes_config_and_step():
    """``lm.config`` is the typed configuration, ``lm.step`` the step function that generation runs on."""
    from cima_b200.engine import StepEntry
    lm = cima_b200.load(model_folder("B"), dtype="float32", max_tokens=256, verbose=False)
    assert lm.config.num_key_value_heads == 1 and lm.config.rope_theta == TINY["B"]["rope_theta"]
    toks = random_tokens(TINY["B"]["vocab_size"], 12, seed=5)
    cfg, W = plain_load(model_folder("B"))
    (slot,) = lm.model.cache.open(1)
    try:
        got = lm.step([StepEntry(slot, toks, [11])]).cpu()
    finally:
        lm.model.cache.close([slot])
    assert torch.allclose(got[0], plain_forward(W, cfg, toks)[-1].float(), atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("name,temp", [("A", 0.8), ("B", 1.0)])
def test_sampled_generation_matches_plain_in_float32(name, temp):
    V = TINY[name]["vocab_size"]
    lens = [7, 1, 13] if name == "A" else [1, 9, 30, 64]
    prompts = [random_tokens(V, n, seed=60 + n) for n in lens]
    lm = cima_b200.load(model_folder(name), dtype="float32", max_tokens=1024, verbose=False)
    opts = dict(temperature=temp, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=1234)
    got = lm.generate(prompts, max_tokens=10, **opts)
    for p, r in zip(prompts, got):
        assert r.tokens == plain_generate(name, p, opts, 10)[0]
    # the reference's default chain too (top-k 40, top-p 0.9, penalty 1.1)
    opts = dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=7)
    got = lm.generate(prompts[:2], max_tokens=8, **opts)
    for p, r in zip(prompts[:2], got):
        assert r.tokens == plain_generate(name, p, opts, 8)[0]


def test_stop_tokens_early_finishers_and_many_batches():
    """More requests than a batch holds; some stop early on a stop token; slots are used again."""
    name = "A"
    prompts = [random_tokens(512, 3 + (i % 5), seed=80 + i) for i in range(7)]
    lm = cima_b200.load(model_folder(name), dtype="float32", max_tokens=64 * 3, max_seqs=3, max_batch=3, verbose=False)
    free = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=12)
    assert lm.stats.batches == 3
    # make the 4th token of request 2 and the 1st of request 5 stop tokens
    stops = (free[2].tokens[3], free[5].tokens[0])
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=12, stop=stops)
    for i, (f, r) in enumerate(zip(free, got)):
        cut = next((j for j, t in enumerate(f.tokens) if t in stops), None)
        if cut is None:
            assert r.tokens == f.tokens and r.finish_reason == "length"
        else:
            assert r.tokens == f.tokens[:cut] and r.finish_reason == "stop", i
    assert got[5].tokens == []
    ignored = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=12, stop=stops, ignore_eos=True)
    assert [r.tokens for r in ignored] == [f.tokens for f in free]
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0


# ---------------------------------------------------------------------------- trace replay
def run_trace(folder, dtype, steps, out_dir, max_tokens):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]


def read_step(out_dir, step, V):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, V).copy())


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_trace_run_three_ways(tmp_path, dtype, tol):
    name = "C"
    V = TINY[name]["vocab_size"]
    folder = model_folder(name)
    cfg, W = plain_load(folder)
    reqs = {f"r{i}": random_tokens(V, n, seed=90 + i) for i, n in enumerate([150, 40, 97])}
    want = {k: plain_forward(W, cfg, v).float() for k, v in reqs.items()}
    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(reqs.items())]
    run_trace(folder, dtype, steps, tmp_path / "whole", 192)
    for i, k in enumerate(reqs):
        assert (read_step(tmp_path / "whole", i, V) - want[k]).abs().max().item() <= tol
    # 2. the last 32 tokens one by one
    steps, n = [], 0
    for k, v in reqs.items():
        head = len(v) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": v[:head], "want": [head - 1]}], "end": []}); n += 1
        for j in range(head, len(v)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [v[j]], "want": [0]}],
                          "end": [k] if j == len(v) - 1 else []}); n += 1
    run_trace(folder, dtype, steps, tmp_path / "tail", 192)
    n = 0
    for k, v in reqs.items():
        head = len(v) - 32
        assert (read_step(tmp_path / "tail", n, V)[0] - want[k][head - 1]).abs().max().item() <= tol; n += 1
        for j in range(head, len(v)):
            assert (read_step(tmp_path / "tail", n, V)[0] - want[k][j]).abs().max().item() <= tol, (k, j); n += 1
    # 3. one batch of unequal lengths; the shorter requests end earlier; then a second batch reuses the cache
    steps, n = [], 0
    for rnd in range(2):
        ids = {k: f"{k}_{rnd}" for k in reqs}
        heads = {k: len(v) - 20 for k, v in reqs.items()}
        steps.append({"step": n, "entries": [{"id": ids[k], "tokens": v[:heads[k] + (5 if k == "r1" else 0)], "want": [0, heads[k] - 1]}
                                             for k, v in reqs.items()], "end": []}); n += 1
        pos = {k: heads[k] + (5 if k == "r1" else 0) for k in reqs}
        while any(pos[k] < len(reqs[k]) for k in reqs):
            live = [k for k in reqs if pos[k] < len(reqs[k])]
            steps.append({"step": n, "entries": [{"id": ids[k], "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                          "end": [ids[k] for k in live if pos[k] == len(reqs[k]) - 1]}); n += 1
            for k in live:
                pos[k] += 1
    run_trace(folder, dtype, steps, tmp_path / "batch", 64 * 6)
    # every wanted place against the plain logits at its position (tokens fed so far + place)
    fed = {}
    for s in steps:
        got = read_step(tmp_path / "batch", s["step"], V)
        r = 0
        for e in s["entries"]:
            k = e["id"].split("_")[0]
            start = fed.get(e["id"], 0)
            for w in e["want"]:
                assert (got[r] - want[k][start + w]).abs().max().item() <= tol, (s["step"], e["id"], start + w)
                r += 1
            fed[e["id"]] = start + len(e["tokens"])


def test_trace_run_answers_each_step_before_the_next_is_sent(tmp_path):
    """The driver sends a step only after ``done <step>`` of the one before: nothing may wait for more input or
    sit in a buffer; a step's file is complete when its line arrives."""
    name = "A"
    V = TINY[name]["vocab_size"]
    cfg, W = plain_load(model_folder(name))
    toks = random_tokens(V, 12, seed=5)
    want = plain_forward(W, cfg, toks).float()
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder(name), "--dtype",
                          "float32", "--out", str(tmp_path), "--max-tokens", "64"], stdin=subprocess.PIPE,
                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
    try:
        steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:9], "want": [8]}], "end": []},
                 {"step": 1, "entries": [{"id": "x", "tokens": [toks[9]], "want": [0]}], "end": []},
                 {"step": 2, "entries": [{"id": "x", "tokens": toks[10:], "want": [1]}], "end": ["x"]}]
        for s, place in zip(steps, (8, 9, 11)):
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline()
            while line and not line.startswith("done"):
                line = p.stdout.readline()
            assert line.strip() == f"done {s['step']}"
            assert (read_step(tmp_path, s["step"], V)[0] - want[place]).abs().max().item() <= 2e-5
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()


def test_pipelined_and_plain_decoding_give_the_same_tokens():
    """Run-ahead decoding (the default) against the step-by-step loop: greedy and sampled, early stops."""
    name = "B"
    prompts = [random_tokens(1000, n, seed=70 + n) for n in (3, 17, 40, 9, 1)]
    outs = []
    for pipeline in (True, False):
        lm = cima_b200.load(model_folder(name), dtype="bfloat16", max_tokens=2048, verbose=False, pipeline=pipeline)
        free = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=40)
        stops = (free[1].tokens[5], free[3].tokens[20])
        a = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=40, stop=stops)
        b = lm.generate(prompts, temperature=0.9, top_k=20, top_p=0.95, repeat_penalty=1.1, seed=5, max_tokens=30)
        c = lm.generate(prompts[:2], temperature=0, repeat_penalty=1.0, max_tokens=230)      # up to the last position
        outs.append([[r.tokens for r in x] + [[r.finish_reason for r in x]] for x in (free, a, b, c)])
        lm.model.cache.check()
        assert lm.model.cache.slots.held == 0
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pipeline", [True, False])
def test_finished_sequences_are_taken_up_again(dtype, pipeline):
    """``retain``: the next turn of a conversation runs only its new tokens (decoding through graphs, with and
    without run-ahead); the answers are those of a model that runs everything."""
    V = TINY["B"]["vocab_size"]
    opts = dict(temperature=0, repeat_penalty=1.0)
    lm = cima_b200.load(model_folder("B"), dtype=dtype, max_tokens=1024, verbose=False, retain=2, pipeline=pipeline)
    plain = cima_b200.load(model_folder("B"), dtype=dtype, max_tokens=1024, verbose=False, pipeline=pipeline)
    p1 = random_tokens(V, 40, 1)
    r1 = lm.generate([p1], max_tokens=12, **opts)[0]
    assert r1.tokens == plain.generate([p1], max_tokens=12, **opts)[0].tokens
    p2 = p1 + r1.tokens + random_tokens(V, 10, 2)
    q2 = random_tokens(V, 21, 9)
    r2 = lm.generate([p2, q2], max_tokens=12, **opts)
    assert lm.stats.reused_tokens == len(p1) + len(r1.tokens) - 1
    assert [r.tokens for r in r2] == [r.tokens for r in plain.generate([p2, q2], max_tokens=12, **opts)]
    p3 = p2[:30] + random_tokens(V, 25, 3)                    # goes back to 30 tokens in common
    r3 = lm.generate([p3], max_tokens=12, **opts)[0]
    assert lm.stats.reused_tokens == 30
    assert r3.tokens == plain.generate([p3], max_tokens=12, **opts)[0].tokens
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 2
    lm.stepper.drop_retained()
    assert lm.model.cache.slots.held == 0


@pytest.mark.parametrize("name,n_prompts,pipeline", [("A", 20, True), ("B", 64, True), ("B", 20, False), ("A", 64, False)])
def test_many_prompts_generate_as_the_plain_loop_does(name, n_prompts, pipeline):
    """20 and 64 prompts of unequal lengths through ``generate`` in 32-bit (decode graphs of 9 to 64 sequences, with
    run-ahead and without): greedy, and the reference's default sampling chain on a part of them, token for token
    what the plain implementation generates; some stop early on stop tokens, so that the batch shrinks on the way."""
    V = TINY[name]["vocab_size"]
    gen = np.random.default_rng(n_prompts)
    prompts = [random_tokens(V, int(n), seed=500 + i) for i, n in enumerate(gen.integers(1, 40, size=n_prompts))]
    lm = cima_b200.load(model_folder(name), dtype="float32", max_tokens=64 * 2 * n_prompts, verbose=False, pipeline=pipeline)
    steps = 6
    free = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=steps)
    want = [plain_generate(name, p, dict(temperature=0.0), steps)[0] for p in prompts]
    assert [r.tokens for r in free] == want
    stops = (want[3][2], want[11][4], want[0][0])
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=steps, stop=stops)
    for w, r in zip(want, got):
        cut = next((j for j, t in enumerate(w) if t in stops), None)
        assert r.tokens == (w if cut is None else w[:cut])
    opts = dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=11)
    some = prompts[:12]
    got = lm.generate(some, max_tokens=5, **opts)
    for p, r in zip(some, got):
        assert r.tokens == plain_generate(name, p, opts, 5)[0]
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0


def test_batch_sizes_in_any_order_through_recorded_steps():
    """Recorded decode steps keep the addresses of the scratch they were recorded with (the attention's splits, the
    sampler's row copies).  Batches of 1, 8, 1, then 8 shrinking to 4 and 8 again, with sampling on, on ONE model
    must give what each call gives on a model of its own (which has recorded nothing before), and logits that a
    caller kept from an earlier step must stay as they were."""
    from cima_b200.engine import StepEntry
    name = "B"
    V = TINY[name]["vocab_size"]
    prompts = [random_tokens(V, 5 + 3 * i, seed=900 + i) for i in range(8)]
    opts = dict(temperature=0.9, top_k=30, top_p=0.95, repeat_penalty=1.1, seed=21)
    greedy = dict(temperature=0, repeat_penalty=1.0)

    def fresh():
        return cima_b200.load(model_folder(name), dtype="bfloat16", max_tokens=4096, verbose=False)

    probe = fresh().generate(prompts, max_tokens=20, **opts)
    stops = tuple(probe[i].tokens[3 + i] for i in range(4))       # four of the eight stop early: 8 -> 4 sequences
    calls = [(prompts[:1], dict(opts)), (prompts, dict(opts)), (prompts[:1], dict(opts)), (prompts, dict(opts, stop=stops)),
             (prompts, dict(opts)), (prompts[:3], dict(greedy)), (prompts, dict(greedy))]
    want = [[r.tokens for r in fresh().generate(ps, max_tokens=20, **o)] for ps, o in calls]
    lm = fresh()
    assert lm.stepper.use_graphs
    (slot,) = lm.model.cache.open(1)
    kept = lm.step([StepEntry(slot, prompts[0], [len(prompts[0]) - 1])])
    lm.model.cache.close([slot])
    before = kept.clone()
    got = [[r.tokens for r in lm.generate(ps, max_tokens=20, **o)] for ps, o in calls]
    assert torch.equal(kept, before)
    assert got == want
    assert any(len(t) < 20 for t in got[3])
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0


def test_other_tokens_than_the_chosen_ones_may_be_fed_back():
    """A caller of the stepper that feeds back tokens of its own choosing (forced tokens) while run-ahead is on: the
    step that was queued with the chosen tokens is dropped, and the next one starts from the cache's lengths."""
    from cima_b200.engine import StepEntry
    from cima_b200.sampling import GenOptions
    name = "B"
    V = TINY[name]["vocab_size"]
    lm = cima_b200.load(model_folder(name), dtype="float32", max_tokens=1024, verbose=False, pipeline=True)
    st = lm.stepper
    greedy = GenOptions(temperature=0.0, repeat_penalty=1.0)
    prompts = [random_tokens(V, n, seed=300 + n) for n in (9, 4)]
    forced = [random_tokens(V, 6, seed=1), random_tokens(V, 6, seed=2)]
    slots = st.open(2)
    try:
        st.prefill(slots, prompts, [greedy, greedy])
        got = []
        for k in range(6):
            got.append(st.decode(slots, [forced[0][k], forced[1][k]], [greedy, greedy]))
    finally:
        st.close(slots)
    cfg, W = plain_load(model_folder(name))
    for i in range(2):
        seq = list(prompts[i])
        for k in range(6):
            seq.append(forced[i][k])
            assert got[k][i] == int(torch.argmax(plain_forward(W, cfg, seq)[-1].float()))
    lm.model.cache.check()


def test_cima_run_generates_what_the_plain_loop_does(tmp_path):
    """``bin/cima run`` as a user calls it: token ids on the command line and in a prompts file, options by the
    reference's names; the generated ids on standard output are the plain implementation's (32-bit, greedy and
    sampled).  Then the same command on a shape with random weights in memory."""
    name = "A"
    folder = model_folder(name)
    exe = [sys.executable, os.path.join(ROOT, "bin", "cima"), "run"]
    p = subprocess.run(exe + [folder, "5", "17", "3", "--temp", "0", "--repeat-penalty", "1.0", "--max-tokens", "8", "--dtype",
                              "float32"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == plain_generate(name, [5, 17, 3], dict(temperature=0.0), 8)[0]
    assert "3 prompt tok | 8 gen tok" in p.stderr
    (tmp_path / "prompts.txt").write_text("5 17 3\n42\n7,7,7,300,2\n")
    opts = dict(temperature=0.7, top_k=20, top_p=0.9, repeat_penalty=1.2, seed=99)
    p = subprocess.run(exe + [folder, "--prompts", str(tmp_path / "prompts.txt"), "--temperature", "0.7", "--top-k", "20",
                              "--top-p", "0.9", "--repeat-penalty", "1.2", "--seed", "99", "--max-tokens", "6", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(t) for t in l.split()] for l in p.stdout.strip().split("\n")]
    assert lines == [plain_generate(name, q, opts, 6)[0] for q in ([5, 17, 3], [42], [7, 7, 7, 300, 2])]
    p = subprocess.run(exe + ["--random-shape", "tiny-b", "--weights-seed", "4", "1", "2", "3", "--temp", "0", "--max-tokens", "5"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.split()) == 5
    # --stream: every token as its step is read, "<prompt>:<token>" a line, the same tokens
    p = subprocess.run(exe + [folder, "5", "17", "3", "--stream", "--temp", "0", "--repeat-penalty", "1.0", "--max-tokens", "8",
                              "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(l.split(":")[1]) for l in p.stdout.split()] == plain_generate(name, [5, 17, 3], dict(temperature=0.0), 8)[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_model_from_a_configuration_in_memory_equals_the_folder(dtype, tmp_path):
    """``load(config=, seed=)`` draws the values that ``write_random_model`` stores for the seed and goes through
    the same loader: logits bit for bit those of the folder's model; ``state_dict`` gives the tensors back by name."""
    from cima_b200.engine import StepEntry, build_plan
    from cima_b200.weights import random_tensors
    cfg = TINY["C"]
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=6)
    a = cima_b200.load(folder, dtype=dtype, max_tokens=512, verbose=False)
    b = cima_b200.load(config=cfg, seed=6, dtype=dtype, max_tokens=512, verbose=False)
    toks = random_tokens(cfg["vocab_size"], 120, seed=8)
    outs = []
    for lm in (a, b):
        (slot,) = lm.model.cache.open(1)
        try:
            outs.append(lm.step([StepEntry(slot, toks, list(range(len(toks))))]).clone())
        finally:
            lm.model.cache.close([slot])
    assert torch.equal(outs[0], outs[1])
    want = random_tensors(build_plan(b.spec), 6)
    sd = b.state_dict()
    assert sorted(sd) == sorted(want)
    for n, t in want.items():
        assert torch.equal(sd[n].float().cpu(), t.float()), n
    # drawn on the device: other values, the same road
    c = cima_b200.load(config=cfg, seed=6, dtype=dtype, max_tokens=512, verbose=False, draw="device")
    assert len(c.generate([toks[:9]], temperature=0, max_tokens=4)[0].tokens) == 4


def test_loading_holds_one_group_of_tensors_on_the_host_not_the_checkpoint():
    """While a model loads, the fetched host tensors alive at once stay within the largest group that a part
    stacks (the table, gate | up, or q | k | v), far below the checkpoint: each is uploaded and dropped."""
    from cima_b200.engine import build_plan, load_model
    m = load_model(model_folder("B"), dtype="bfloat16", max_tokens=256, verbose=False)
    cfg = m.config
    total = sum(2 * int(np.prod(s.shape)) for s in build_plan(m.spec).values())
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    group = max(2 * V * H, 2 * 2 * I * H, 2 * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim * H)
    assert 0 < m.load_peak_host_bytes <= group + 4096
    assert m.load_peak_host_bytes < total / 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_through_recorded_prompt_steps(dtype):
    """One short prompt at a time takes a recorded prompt step whose rows are padded to 16, 32 or 64: lengths at and
    around the buckets' edges, each three times (a shape's first step is issued as it is, its second is recorded,
    its third replayed), then batches, then longer ones.
    32-bit: the tokens of the plain implementation; bfloat16: maxima of the plain logits within its rounding.
    The padding's keys lie beyond the sequence's length and are written over by the tokens that follow."""
    name = "B"
    V = TINY[name]["vocab_size"]
    cfg, W = plain_load(model_folder(name))
    lm = cima_b200.load(model_folder(name), dtype=dtype, max_tokens=2048, verbose=False)
    for n in (1, 2, 15, 16, 17, 31, 33, 64, 65, 100):
        for rep in range(3):
            p = random_tokens(V, n, seed=3000 + n + 7 * rep)
            r = lm.generate([p], temperature=0, repeat_penalty=1.0, max_tokens=6)[0]
            if dtype == "float32":
                assert r.tokens == plain_generate(name, p, dict(temperature=0.0), 6)[0], (n, rep)
            else:
                seq = list(p)
                for t in r.tokens:
                    lg = plain_forward(W, cfg, seq)[-1]
                    assert lg[t] >= lg.max() - 4e-2, (n, rep)
                    seq.append(t)
    assert sorted(lm.stepper._prompt_graphs) == [(1, 16), (1, 32), (1, 64), (1, 128)]
    # several short prompts in one recorded step: padded to the longest one's bucket, each gathered at its own end
    for lens in ([3, 16, 9], [40, 1, 33, 64], [5, 5, 5, 5, 5, 5, 5, 5], [100, 128]):
        ps = [random_tokens(V, n, seed=4000 + 13 * i + n) for i, n in enumerate(lens)]
        for rep in range(3):
            got = lm.generate(ps, temperature=0, repeat_penalty=1.0, max_tokens=4)
            for p, r in zip(ps, got):
                if dtype == "float32":
                    assert r.tokens == plain_generate(name, p, dict(temperature=0.0), 4)[0], (lens, rep)
                else:
                    seq = list(p)
                    for t in r.tokens:
                        lg = plain_forward(W, cfg, seq)[-1]
                        assert lg[t] >= lg.max() - 4e-2, (lens, rep)
                        seq.append(t)
    assert {(3, 16), (4, 64), (8, 16), (2, 128)} <= set(lm.stepper._prompt_graphs)
    opts = dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=4)
    if dtype == "float32":
        p = random_tokens(V, 20, seed=1)
        assert lm.generate([p], max_tokens=6, **opts)[0].tokens == plain_generate(name, p, opts, 6)[0]
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_longer_prompts_of_a_small_model_through_recorded_prompt_steps(dtype, tmp_path):
    """A small model's prompt steps are recorded up to 2,048 rows (the host would be the slower side): prompts of 257
    to 2,040 tokens at and around the buckets' edges, one at a time and two together, each three times (issued as it
    is, recorded, replayed).
    32-bit: the tokens of the plain implementation; bfloat16: maxima of the plain logits within its rounding."""
    cfg = dict(TINY["B"], max_position_embeddings=2048)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=8)
    c, W = plain_load(folder)
    if dtype == "float32":
        W = {k: v.double() for k, v in W.items()}
    V = cfg["vocab_size"]
    lm = cima_b200.load(folder, dtype=dtype, max_tokens=3 * 2048, verbose=False)
    assert lm.stepper.prompt_rows == 2048

    def check(prompts, tag):
        got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=3)
        for p, r in zip(prompts, got):
            seq = list(p)
            for t in r.tokens:
                lg = plain_forward(W, c, seq)[-1].float()
                assert lg[t] >= lg.max() - (0.0 if dtype == "float32" else 4e-2), (tag, len(p))
                seq.append(t)

    for n in (257, 384, 385, 1000, 2040):
        p = random_tokens(V, n, seed=5000 + n)
        for rep in range(3):
            check([p], rep)
    assert {(1, 384), (1, 512), (1, 1024), (1, 2048)} <= set(lm.stepper._prompt_graphs)
    pair = [random_tokens(V, n, seed=5100 + n) for n in (700, 300)]
    for rep in range(3):
        check(pair, rep)
    assert (2, 768) in lm.stepper._prompt_graphs
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0
    lm.model.check_device()


@pytest.mark.parametrize("pipeline", [True, False])
def test_sequences_that_outgrow_the_short_context_change_graphs(pipeline, tmp_path):
    """Decode steps of sequences within the short-context bound are recorded without splits of the attention; when
    a sequence outgrows that bound the stepper goes on with the unbounded graph.  Generation across the bound (prompts
    that end 3 to 42 tokens before it, 60 new ones), with run-ahead and without, in bfloat16: the same tokens as step-by-step decoding
    without graphs, whose every step chooses its kernels from the lengths it sees; and on the device without the
    host in between (``decode_on_device``) across the bound as well."""
    from cima_b200.sampling import GenOptions
    cfg = dict(TINY["B"], max_position_embeddings=1024)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=4)
    V = cfg["vocab_size"]
    from cima_b200.kernels import short_context
    SHORT_CONTEXT = short_context(cfg["head_dim"])
    prompts = [random_tokens(V, n, seed=600 + n) for n in (SHORT_CONTEXT - 42, SHORT_CONTEXT - 3, SHORT_CONTEXT - 12)]
    outs = []
    for use_graphs in (True, False):
        lm = cima_b200.load(folder, dtype="bfloat16", max_tokens=4096, verbose=False, pipeline=pipeline, use_graphs=use_graphs)
        outs.append([r.tokens for r in lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=60)])
        if use_graphs:
            assert {k[2] for k in lm.stepper._graphs} == {SHORT_CONTEXT, 0}
            st = lm.stepper
            greedy = [GenOptions(temperature=0.0, repeat_penalty=1.0)] * 3
            slots = st.open(3)
            try:
                first = st.prefill(slots, prompts, greedy)
                nxt = st.decode(slots, first, greedy)
                st.decode_on_device(slots, nxt, greedy, 2)                 # stays within the bound
                last = st.decode_on_device(slots, None, greedy, 50).tolist()   # crosses it: the tokens travel on the device
            finally:
                st.close(slots)
            assert last == [t[1 + 2 + 50] for t in outs[0]]
    assert outs[0] == outs[1]


def test_short_prompts_of_a_windowed_model_keep_their_window(tmp_path):
    """A windowed group keeps its keys in a ring of pages: rows padded onto a prompt would land on ring entries that
    positions inside the window still need (129 tokens padded to 256 rows with a window of 40: the padding at 217..255
    falls on the places of 89..127).  Such a model's prompts therefore run unpadded; generation from prompts of 129 to
    200 tokens equals the plain loop's."""
    name = "C"
    V = TINY[name]["vocab_size"]
    lm = cima_b200.load(model_folder(name), dtype="float32", max_tokens=4096, verbose=False)
    for n in (129, 150, 200, 16):
        p = random_tokens(V, n, seed=7000 + n)
        got = lm.generate([p], temperature=0, repeat_penalty=1.0, max_tokens=8)[0]
        assert got.tokens == plain_generate(name, p, dict(temperature=0.0), 8)[0], n
    assert not lm.stepper._prompt_graphs


def test_cima_profile_prints_every_launch_of_a_step():
    """``bin/cima profile``: the launches of one decode step and of one prompt step with their times, from a shape
    with random weights in memory."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "cima"), "profile", "--random-shape", "tiny-b", "--batch", "2",
                        "--prompt-len", "40"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "decode step, batch 2, context 40" in p.stdout and "prompt step, one prompt of 40 tokens" in p.stdout
    assert "qkv_rope_skinny" in p.stdout and "attention_decode" in p.stdout and "launches a token" in p.stdout


def test_cima_bench_reports_a_decode_rate():
    """``bin/cima bench`` as the reference's bench command: greedy, stop tokens ignored, one discarded warm-up, the
    median of the iterations' decode rates as one JSON line."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "cima"), "bench", model_folder("A"), "-n", "12", "--iters", "2",
                        "--batch", "2", "--prompt-len", "9"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().split("\n")[-1])
    assert line["batch"] == 2 and line["gen_tokens"] == 12 and line["prompt_tokens"] == 9
    assert line["decode_tok_per_s_p50"] >= line["decode_tok_per_s_min"] > 0 and line["ttft_ms"] > 0
