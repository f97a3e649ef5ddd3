"""Each part of a layer alone, on inputs that the test chooses, against the plain function of the same
part: norm, position encoding, mixer (attention with its projections, over a prompt and then token by token
from the cache), feed-forward, and the block that arranges them.  The parts are built by the registries from
the tiny configurations' specs and loaded with the random weights of a model folder; no other part runs."""

import pytest
import torch

from helpers import TINY, gpu_model, model_folder
from qwen2_plain import (plain_attention, plain_block, plain_layer_window, plain_linear, plain_load, plain_rmsnorm,
                         plain_rope, plain_swiglu_mlp)
from cima_b200.engine.batch import StepEntry, build_batch

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 6e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def err(got, want):
    return (got.detach().double().cpu() - want.double()).abs().max().item()


def rows(T, H, seed, scale=1.0):
    return torch.randn(T, H, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale


def prepared(model, lengths, starts=None):
    """Open slots, reserve the rows' places and return (slots, batch) for entries of the given lengths."""
    slots = model.cache.open(len(lengths))
    starts = starts or [0] * len(lengths)
    entries = [StepEntry(s, [1] * n, []) for s, n in zip(slots, lengths)]
    batch = build_batch(entries, starts, model.spec.vocab, model.rt.device)
    for s, st, n in zip(slots, starts, lengths):
        model.cache.reserve(s, st + n)
    model.cache.flush()
    return slots, batch


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_norm_alone(name, dtype):
    cfg = TINY[name]
    m = gpu_model(name, dtype)
    _, W = plain_load(model_folder(name))
    x = rows(37, cfg["hidden_size"], 1, scale=3.0)
    for part, wname in ((m.blocks[0].mixer_norm, "model.layers.0.input_layernorm.weight"),
                        (m.blocks[1].ffn_norm, "model.layers.1.post_attention_layernorm.weight"),
                        (m.final_norm, "model.norm.weight")):
        got = part(x.cuda())
        assert got.dtype is DT[dtype]
        assert err(got, plain_rmsnorm(x.double(), W[wname].double(), cfg["rms_norm_eps"])) <= TOL[dtype]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_position_encoding_alone(name):
    """The part's table of inverse frequencies, used the way the kernels use it (angle = position * inv_freq,
    pairs (i, i + d/2)), gives the plain rotation."""
    cfg = TINY[name]
    m = gpu_model(name, "float32")
    pos_part = m.blocks[0].mixer.position
    hd = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    assert pos_part.rotary_dim == hd and pos_part.inv_freq.dtype is torch.float32
    u = torch.randn(9, 2, hd, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    positions = torch.tensor([0, 1, 2, 3, 50, 51, 100, 127, 64])
    want = plain_rope(u, positions, cfg["rope_theta"])
    inv = pos_part.inv_freq.double().cpu()
    ang = positions.double()[:, None] * inv[None, :]
    a, b = u[..., :hd // 2], u[..., hd // 2:]
    got = torch.cat([a * ang.cos()[:, None] - b * ang.sin()[:, None], a * ang.sin()[:, None] + b * ang.cos()[:, None]], -1)
    assert err(got, want) <= 1e-5        # inv_freq is rounded to float32 once


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("activation", ["gelu_pytorch_tanh", "gelu", "relu", "silu"])
@pytest.mark.parametrize("T", [1, 7, 40, 300])
def test_gated_feed_forward_with_other_activations(activation, T, dtype):
    """The gated feed-forward built from a spec of the test's own (sizes that no tiny configuration has, any of the
    gate's activations), loaded from tensors of the test's making, for few rows (the skinny product with the
    activation in its epilogue), more (the library product and the activation kernel) and 300 (which still takes
    that road at this width): x += (act(h Wg^T) * (h Wu^T)) Wd^T against float64."""
    import math
    from cima_b200.config import FeedForwardSpec
    from cima_b200.kernels import Kernels
    from cima_b200.parts import Runtime, build_feed_forward
    H, I = 136, 264
    gen = torch.Generator().manual_seed(11)
    W = {"f.g.weight": torch.randn(I, H, generator=gen) / math.sqrt(H), "f.u.weight": torch.randn(I, H, generator=gen) / math.sqrt(H),
         "f.d.weight": torch.randn(H, I, generator=gen) / math.sqrt(I)}
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    rt = Runtime(kernels=Kernels(verbose=False), dtype=DT[dtype], device="cuda:0")
    ffn = build_feed_forward(FeedForwardSpec("gated_mlp", H, I, activation), 0, rt)
    names = {"gate": "g", "up": "u", "down": "d"}
    assert sorted(ffn.plan("f.", names)) == sorted(W)
    ffn.load(W, "f.", names)
    h, x0 = rows(T, H, 3), rows(T, H, 4)
    x = x0.cuda()
    ffn.forward(h.to(DT[dtype]).cuda(), x, None)
    hd = h.to(DT[dtype]).double()
    g_, u_ = hd @ W["f.g.weight"].double().t(), hd @ W["f.u.weight"].double().t()
    act = {"gelu_pytorch_tanh": lambda g: 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))),
           "gelu": lambda g: 0.5 * g * (1 + torch.erf(g / math.sqrt(2))), "relu": lambda g: g.clamp(min=0),
           "silu": lambda g: g / (1 + torch.exp(-g))}[activation]
    want = x0.double() + (act(g_) * u_) @ W["f.d.weight"].double().t()
    assert err(x, want) <= TOL[dtype]
    with pytest.raises(ValueError, match="is not one of"):
        build_feed_forward(FeedForwardSpec("gated_mlp", H, I, "softsign"), 0, rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 2), ("C", 1), ("C", 3)])      # C's layers 2, 3 have a window
def test_mixer_alone_over_a_prompt_and_from_the_cache(name, layer, dtype):
    """x += attention(h): two prompts of unequal length in one step, then one more token each from the
    cache.  h is an input of the test, not a norm's output."""
    cfg = TINY[name]
    m = gpu_model(name, dtype)
    _, W = plain_load(model_folder(name))
    mixer = m.blocks[layer].mixer
    site = m.spec.schedule.index(layer)
    H, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim", H // nh)
    p = f"model.layers.{layer}.self_attn."
    lens = [70, 45]
    h_all = [rows(n + 1, H, 10 + i) for i, n in enumerate(lens)]       # the last row is the decode step's

    def plain_out(h, upto):
        hh = h[:upto].double()
        T = hh.shape[0]
        pos = torch.arange(T)
        q = plain_rope(plain_linear(hh, W[p + "q_proj.weight"].double(), W[p + "q_proj.bias"].double()).view(T, nh, hd), pos, cfg["rope_theta"])
        k = plain_rope(plain_linear(hh, W[p + "k_proj.weight"].double(), W[p + "k_proj.bias"].double()).view(T, nkv, hd), pos, cfg["rope_theta"])
        v = plain_linear(hh, W[p + "v_proj.weight"].double(), W[p + "v_proj.bias"].double()).view(T, nkv, hd)
        att = plain_attention(q, k, v, plain_layer_window(cfg, layer)).reshape(T, nh * hd)
        return plain_linear(att, W[p + "o_proj.weight"].double())

    slots, batch = prepared(m, lens)
    try:
        h = torch.cat([h_all[0][:lens[0]], h_all[1][:lens[1]]]).to(DT[dtype]).cuda()
        x = torch.zeros(sum(lens), H, device="cuda")
        mixer.forward(h, x, batch, m.cache, site)
        want = torch.cat([plain_out(h_all[0], lens[0]), plain_out(h_all[1], lens[1])])
        assert err(x, want) <= TOL[dtype] * 2
        for s, n in zip(slots, lens):
            m.cache.commit(s, n)
        # one more token each, from the cache
        entries = [StepEntry(s, [1], []) for s in slots]
        batch1 = build_batch(entries, lens, m.spec.vocab, m.rt.device)
        for s, n in zip(slots, lens):
            m.cache.reserve(s, n + 1)
        m.cache.flush()
        h1 = torch.stack([h_all[0][lens[0]], h_all[1][lens[1]]]).to(DT[dtype]).cuda()
        x1 = torch.zeros(2, H, device="cuda")
        mixer.forward(h1, x1, batch1, m.cache, site)
        want1 = torch.stack([plain_out(h_all[0], lens[0] + 1)[-1], plain_out(h_all[1], lens[1] + 1)[-1]])
        assert err(x1, want1) <= TOL[dtype] * 2
    finally:
        m.cache.close(slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,T", [("A", 1), ("A", 50), ("B", 9), ("C", 130)])
def test_feed_forward_alone(name, T, dtype):
    cfg = TINY[name]
    m = gpu_model(name, dtype)
    _, W = plain_load(model_folder(name))
    ffn = m.blocks[1].feed_forward
    p = "model.layers.1.mlp."
    h = rows(T, cfg["hidden_size"], 3)
    x0 = rows(T, cfg["hidden_size"], 4)
    x = x0.cuda()
    ffn.forward(h.to(DT[dtype]).cuda(), x, None)
    want = x0.double() + plain_swiglu_mlp(h.to(DT[dtype]).double(), W[p + "gate_proj.weight"].double(),
                                          W[p + "up_proj.weight"].double(), W[p + "down_proj.weight"].double())
    assert err(x, want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("A", 1), ("B", 0), ("C", 2)])
def test_block_alone(name, layer, dtype):
    """A block on a residual stream of the test's making: a prompt in one step, then a token from the cache
    (in bfloat16 that step takes the folded norms and the fused projection)."""
    cfg = TINY[name]
    m = gpu_model(name, dtype)
    _, W = plain_load(model_folder(name))
    Wd = {k: v.double() for k, v in W.items()}
    block = m.blocks[layer]
    site = m.spec.schedule.index(layer)
    T = 60
    x0 = rows(T + 1, cfg["hidden_size"], 7)
    want = plain_block(x0.double(), Wd, cfg, layer, torch.arange(T + 1))
    slots, batch = prepared(m, [T])
    try:
        x = x0[:T].clone().cuda()
        block.forward(x, batch, m.cache, site)
        assert err(x, plain_block(x0[:T].double(), Wd, cfg, layer, torch.arange(T))) <= TOL[dtype] * 2
        m.cache.commit(slots[0], T)
        batch1 = build_batch([StepEntry(slots[0], [1], [])], [T], m.spec.vocab, m.rt.device)
        m.cache.reserve(slots[0], T + 1)
        m.cache.flush()
        x1 = x0[T:T + 1].clone().cuda()
        block.forward(x1, batch1, m.cache, site)
        assert err(x1, want[T:T + 1]) <= TOL[dtype] * 2
    finally:
        m.cache.close(slots)
