"""Configurations drawn at random (every size and option that config.json gives) against the plain implementation,
in both precisions and in ways of cutting drawn at random too: whole, a tail one by one, pieces, unequal batches."""
import os
import random

import pytest
import torch

import cima_b200
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole
from qwen2_plain import plain_forward, plain_load
from cima_b200.engine import load_model

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2e-2}
SEEDS = list(range(int(os.environ.get("CIMA_RANDOM_CONFIGS", "8"))))


def draw_config(rng: random.Random) -> dict:
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 128, 160, 256])
    kv_heads = rng.choice([1, 2, 3, 4])
    heads = kv_heads * rng.choice([1, 2, 3, 7])
    hidden = rng.choice([64, 72, 100, 128, 136, 192, 200, 256])       # some are no multiple of 8
    cfg = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=rng.randint(1, 4),
               hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
               intermediate_size=rng.choice([48, 99, 128, 130, 264, 328]), vocab_size=rng.choice([129, 333, 512, 1001, 2048]),
               rope_theta=rng.choice([100.0, 10000.0, 1000000.0]), rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=1024)
    if rng.random() < 0.5:
        cfg.update(use_sliding_window=True, sliding_window=rng.choice([1, 7, 40, 64, 65, 128, 200]),
                   max_window_layers=rng.randint(0, cfg["num_hidden_layers"]))
    return cfg


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(seed, tmp_path):
    rng = random.Random(1000 + seed)
    cfg = draw_config(rng)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=seed)
    c, W = plain_load(folder)
    n = rng.choice([40, 130, 300])
    toks = random_tokens(cfg["vocab_size"], n, seed)
    want = plain_forward(W, c, toks).float()
    cuts = sorted(rng.sample(range(1, n), 3))
    lens = [n, rng.randint(1, n), rng.randint(1, n)]
    starts = [rng.randint(1, l) for l in lens]
    for dtype in ("float32", "bfloat16"):
        m = load_model(folder, dtype=dtype, max_tokens=2048, device="cuda:0", verbose=False)
        tol = TOL[dtype]
        what = (seed, dtype, cfg)
        assert (run_whole(m, toks) - want).abs().max().item() <= tol, what
        assert (run_tail_one_by_one(m, toks, min(32, n - 1)) - want).abs().max().item() <= tol, what
        assert (run_in_pieces(m, [toks], [cuts])[0] - want).abs().max().item() <= tol, (what, cuts)
        for got, l in zip(run_batched(m, [toks[:l] for l in lens], starts), lens):
            assert (got - want[:l]).abs().max().item() <= tol, (what, lens, starts)
        m.cache.check()
        assert m.cache.slots.held == 0
        m.check_device()


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration_generates_as_the_plain_loop(seed, tmp_path):
    """Generation through the entry point on a configuration drawn at random, in 32-bit: a random number of prompts
    of random lengths (one prompt alone takes a recorded prompt step, more than 8 the schedule for many rows),
    greedy or through the reference's default sampling chain, with run-ahead on or off and stop tokens taken from a
    first run: token for token what the plain implementation generates, twice over so that slots, pages, recorded
    steps and kept sequences are used again."""
    from qwen2_plain import PlainXorshift, plain_sample
    rng = random.Random(5000 + seed)
    cfg = draw_config(rng)
    cfg["max_position_embeddings"] = 256
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=seed)
    c, W = plain_load(folder)
    W = {k: v.double() for k, v in W.items()}
    n_prompts = rng.choice([1, 1, 2, 5, 9, 12])
    prompts = [random_tokens(cfg["vocab_size"], rng.choice([1, 2, 15, 16, 17, 40, 64, 65, 70, 129, 150, 200]), seed * 100 + i) for i in range(n_prompts)]
    opts = rng.choice([dict(temperature=0.0, repeat_penalty=1.0), dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=seed + 1)])
    steps = 5

    def plain_generate(p, stops):
        gen, seq, out = PlainXorshift(opts.get("seed", 0)), list(p), []
        for _ in range(steps):
            t = plain_sample(plain_forward(W, c, seq)[-1].float().tolist(), seq, opts, gen)
            if t in stops:
                break
            out.append(t)
            seq.append(t)
        return out

    lm = cima_b200.load(folder, dtype="float32", max_tokens=4096, verbose=False, pipeline=rng.random() < 0.5,
                        retain=rng.choice([0, 0, 2]))
    free = [plain_generate(p, ()) for p in prompts]
    what = (seed, cfg, [len(p) for p in prompts], opts)
    assert [r.tokens for r in lm.generate(prompts, max_tokens=steps, **opts)] == free, what
    stops = tuple({free[0][min(2, len(free[0]) - 1)], free[-1][0]})
    want = [plain_generate(p, stops) for p in prompts]
    for _ in range(2):
        got = lm.generate(prompts, max_tokens=steps, stop=stops, **opts)
        assert [r.tokens for r in got] == want, (what, stops)
    lm.stepper.drop_retained()
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0
    lm.model.check_device()
