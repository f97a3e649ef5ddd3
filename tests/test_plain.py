"""The plain implementation checked against statements that do not share its code (no GPU)."""
import math

import torch

from helpers import TINY, model_folder, random_tokens
from qwen2_plain import (PlainXorshift, plain_attention, plain_forward, plain_load, plain_rmsnorm, plain_rope,
                         plain_sample, plain_swiglu_mlp)


def test_attention_equals_dense_masked_softmax():
    torch.manual_seed(0)
    T, nh, nkv, hd = 23, 6, 2, 16
    q, k, v = torch.randn(T, nh, hd, dtype=torch.float64), torch.randn(T, nkv, hd, dtype=torch.float64), torch.randn(T, nkv, hd, dtype=torch.float64)
    for window in (0, 5, 1):
        kk, vv = k.repeat_interleave(nh // nkv, dim=1), v.repeat_interleave(nh // nkv, dim=1)
        s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(hd)
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
        s = s.masked_fill(~mask, float("-inf"))
        want = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
        assert torch.allclose(plain_attention(q, k, v, window), want, atol=1e-12)


def test_rope_is_complex_multiplication():
    torch.manual_seed(1)
    T, H, hd, theta = 9, 3, 32, 1e6
    u = torch.randn(T, H, hd, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 3, 50, 51, 1000, 4095, 7])
    f = theta ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    z = torch.complex(u[..., :hd // 2], u[..., hd // 2:]) * torch.polar(torch.ones(T, hd // 2, dtype=torch.float64), pos.double()[:, None] * f)[:, None]
    assert torch.allclose(plain_rope(u, pos, theta), torch.cat([z.real, z.imag], -1), atol=1e-12)
    # a rotation keeps lengths, and position 0 changes nothing
    assert torch.allclose(plain_rope(u, pos, theta).norm(dim=-1), u.norm(dim=-1))
    assert torch.equal(plain_rope(u[:1], pos[:1], theta), u[:1])


def test_rmsnorm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    assert torch.allclose(plain_rmsnorm(x, w, 0.0), torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    got = plain_swiglu_mlp(h, eye, 2 * eye, eye)
    silu = lambda t: t / (1 + math.exp(-t))
    assert torch.allclose(got, torch.tensor([[silu(1.0) * 2.0, silu(-2.0) * -4.0]], dtype=torch.float64))


def test_causality_and_window_of_the_whole_model():
    for name in ("A", "C"):
        cfg, W = plain_load(model_folder(name))
        toks = random_tokens(cfg["vocab_size"], 60, seed=1)
        full = plain_forward(W, cfg, toks)
        assert torch.allclose(plain_forward(W, cfg, toks[:25]), full[:25], atol=1e-10)   # later tokens change nothing earlier
    cfg, W = plain_load(model_folder("C"))
    toks = random_tokens(cfg["vocab_size"], 60, seed=1)
    nowin = plain_forward(W, dict(cfg, use_sliding_window=False), toks)
    win = plain_forward(W, cfg, toks)
    assert torch.allclose(nowin[:40], win[:40], atol=1e-10) and not torch.allclose(nowin[45:], win[45:], atol=1e-6)


def test_tied_head_is_the_embedding():
    cfg, W = plain_load(model_folder("A"))
    toks = random_tokens(512, 5, seed=2)
    W2 = dict(W)
    W2["lm_head.weight"] = W["model.embed_tokens.weight"].clone()
    assert torch.equal(plain_forward(W, cfg, toks), plain_forward(W2, dict(cfg, tie_word_embeddings=False), toks))


def test_sampler_properties():
    """The properties the reference's sampler tests assert (src/models/mod.rs:2537-2591)."""
    logits = [0.1, 2.0, -1.0, 2.0, 0.5]
    assert plain_sample(logits, [], dict(temperature=0.0), PlainXorshift(1)) == 3           # greedy = argmax, ties to the higher index
    a = [plain_sample(logits, [], dict(temperature=1.0, top_k=0, top_p=1.0), PlainXorshift(9)) for _ in range(3)]
    assert a[0] == a[1] == a[2]                                                             # same seed, same draw
    r1, r2 = PlainXorshift(5), PlainXorshift(5)
    assert [r1.next_f32() for _ in range(4)] == [r2.next_f32() for _ in range(4)]
    seen = set()
    rng = PlainXorshift(3)
    for _ in range(400):
        seen.add(plain_sample(logits, [], dict(temperature=1.5, top_k=0, top_p=1.0), rng))
    assert seen == {0, 1, 2, 3, 4}                                                          # top_p = 1 reaches any candidate
    rng = PlainXorshift(3)
    assert {plain_sample(logits, [], dict(temperature=1.5, top_k=2, top_p=1.0), rng) for _ in range(100)} == {1, 3}
    assert plain_sample(logits, [], dict(temperature=1.0, top_k=1), PlainXorshift(2)) == 3
    # penalty: once per occurrence, sign-aware
    assert plain_sample([1.0, 1.05, -5.0], [1], dict(temperature=0.0, repeat_penalty=1.1), PlainXorshift(1)) == 0
    assert plain_sample([1.0, 1.15, -5.0], [1], dict(temperature=0.0, repeat_penalty=1.1), PlainXorshift(1)) == 1
    assert plain_sample([1.0, 1.15, -5.0], [1, 1], dict(temperature=0.0, repeat_penalty=1.1), PlainXorshift(1)) == 0
    assert plain_sample([-1.0, -0.95, -5.0], [1], dict(temperature=0.0, repeat_penalty=1.1), PlainXorshift(1)) == 0
