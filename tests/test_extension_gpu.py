"""Generality of the parts: a toy mixer with state of its own, defined here, is registered, built
into a toy architecture (also registered here) and stepped, without any change to the package.
The toy model also runs one layer twice (each run with storage of its own) and lets one attention
layer read another layer's keys and values.  A second toy architecture has a feed-forward with routing
(top-1 of three experts) and a position encoding of its own (partial rotary with scaled frequencies) in
some layers and the package's parts in the others, and scales the embedding rows (``ModelSpec.embed_scale``)."""
import json
import math
import os
import tempfile

import pytest
import torch

import cima_b200
from cima_b200.cache import StateRequest
from cima_b200.config import (ArchitectureEntry, BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec,
                              PositionSpec, register_architecture)
from cima_b200.engine import StepEntry, build_plan, load_model
from cima_b200.parts import register_mixer
from cima_b200.weights import TensorSpec, write_random_model
from helpers import random_tokens, run_tail_one_by_one, run_whole
from qwen2_plain import (plain_attention, plain_embed, plain_linear, plain_rmsnorm, plain_rope, plain_swiglu_mlp)

pytestmark = pytest.mark.gpu


class CausalMean:
    """x += gain * mean of h over the positions so far.  Its state per sequence is the running sum."""

    def __init__(self, spec, layer, rt):
        self.spec, self.layer, self.rt = spec, layer, rt
        self.gain = None

    def plan(self, prefix, names):
        return {f"{prefix}mix.gain": TensorSpec((self.spec.hidden,), init="ones_normal")}

    def load(self, tensors, prefix, names):
        self.gain = self.rt.vector(tensors[f"{prefix}mix.gain"])

    def nbytes(self):
        return self.gain.numel() * 4

    def cache_requests(self, site):
        return [StateRequest(f"causal_mean.sum.{site}", (self.spec.hidden,), torch.float32)]

    def forward(self, h, x, batch, cache, site):
        state = cache.state[f"causal_mean.sum.{site}"]
        hf = h.float()
        for i in range(batch.n_seqs):
            r0, r1 = int(batch.host_seq_first_row[i]), int(batch.host_seq_first_row[i + 1])
            slot = int(batch.host_seq_slot[i])
            c = torch.cumsum(hf[r0:r1], dim=0) + state[slot]
            x[r0:r1] += self.gain * c / (batch.row_pos[r0:r1].float() + 1.0)[:, None]
            state[slot] = c[-1]


class CausalMeanOnDevice(CausalMean):
    """The same mixer, fit for a recorded decode step: when every sequence brings one row it finds its state through
    the batch's device arrays only (no host value enters the recorded work); other steps take the host's road."""
    graph_safe = True

    def forward(self, h, x, batch, cache, site):
        if batch.n_rows != batch.n_seqs:
            return super().forward(h, x, batch, cache, site)
        state = cache.state[f"causal_mean.sum.{site}"]
        slots = batch.seq_slot.long()
        c = h.float() + state.index_select(0, slots)
        x += self.gain * c / (batch.row_pos.float() + 1.0)[:, None]
        state.index_copy_(0, slots, c)


def toy_spec(cfg) -> ModelSpec:
    H, nh, nkv, hd = cfg["hidden_size"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    pos = PositionSpec("rope", hd, hd, cfg["theta"])
    names = {"q": "attn.q", "k": "attn.k", "v": "attn.v", "o": "attn.o", "gate": "ffn.gate", "up": "ffn.up",
             "down": "ffn.down", "mixer_norm": "norm1", "ffn_norm": "norm2"}
    norm = NormSpec("rmsnorm", H, cfg["eps"])
    ffn = FeedForwardSpec("gated_mlp", H, cfg["intermediate"], "silu")
    layers = []
    for i, kind in enumerate(cfg["layer_kinds"]):
        if kind == "causal_mean":
            mixer = MixerSpec(cfg.get("mean_kind", "causal_mean"), H)       # no heads: only kind and width
        else:
            mixer = MixerSpec("attention", H, nh, nkv, hd, True, False, 0, 1.0 / math.sqrt(hd), pos,
                              cache_from=cfg["reads_site"] if kind == "attention_shared" else None)
        layers.append(BlockSpec("prenorm", mixer, ffn, norm, norm, f"blocks.{i}.", names))
    return ModelSpec("ToyMixForCausalLM", cfg["vocab_size"], H, cfg["max_positions"], layers, list(cfg["schedule"]),
                     norm, True, "embed.weight", "final_norm.weight", "head.weight")


TOY = dict(architectures=["ToyMixForCausalLM"], model_type="toymix", hidden_size=96, vocab_size=300, heads=4,
           kv_heads=2, head_dim=32, intermediate=160, eps=1e-5, theta=10000.0, max_positions=256,
           layer_kinds=["attention", "causal_mean", "attention_shared"], schedule=[0, 1, 2, 1], reads_site=0)


def toy_plain(W, cfg, tokens):
    """The toy model, whole sequence, float64, from the plain parts."""
    W = {k: v.double() for k, v in W.items()}
    T = len(tokens)
    nh, nkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    posn = torch.arange(T)
    x = plain_embed(W["embed.weight"], tokens)
    site_kv = {}
    for site, layer in enumerate(cfg["schedule"]):
        p = f"blocks.{layer}."
        h = plain_rmsnorm(x, W[p + "norm1.weight"], cfg["eps"])
        kind = cfg["layer_kinds"][layer]
        if kind == "causal_mean":
            x = x + W[p + "mix.gain"] * torch.cumsum(h, 0) / (posn.double() + 1)[:, None]
        else:
            q = plain_rope(plain_linear(h, W[p + "attn.q.weight"], W[p + "attn.q.bias"]).view(T, nh, hd), posn, cfg["theta"])
            if kind == "attention_shared":
                k, v = site_kv[cfg["reads_site"]]
            else:
                k = plain_rope(plain_linear(h, W[p + "attn.k.weight"], W[p + "attn.k.bias"]).view(T, nkv, hd), posn, cfg["theta"])
                v = plain_linear(h, W[p + "attn.v.weight"], W[p + "attn.v.bias"]).view(T, nkv, hd)
                site_kv[site] = (k, v)
            x = x + plain_linear(plain_attention(q, k, v).reshape(T, nh * hd), W[p + "attn.o.weight"])
        h = plain_rmsnorm(x, W[p + "norm2.weight"], cfg["eps"])
        x = x + plain_swiglu_mlp(h, W[p + "ffn.gate.weight"], W[p + "ffn.up.weight"], W[p + "ffn.down.weight"])
    return plain_linear(plain_rmsnorm(x, W["final_norm.weight"], cfg["eps"]), W["embed.weight"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype, tol):
    register_mixer("causal_mean", CausalMean)
    register_architecture(ArchitectureEntry("ToyMixForCausalLM", "toymix", parse=lambda raw: raw, spec=toy_spec))
    folder = tempfile.mkdtemp(prefix="cima_toy_")
    write_random_model(folder, TOY, build_plan(toy_spec(TOY)), seed=5)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    model = load_model(folder, dtype=dtype, max_tokens=1024, verbose=False)
    assert len(model.cache.groups) == 1 and len(model.cache.groups[0].layers) == 1     # only site 0 stores keys
    assert {"causal_mean.sum.1", "causal_mean.sum.3"} <= set(model.cache.state)
    toks = random_tokens(300, 90, seed=1)
    want = toy_plain(W, TOY, toks).float()
    assert (run_whole(model, toks) - want).abs().max().item() <= tol
    assert (run_tail_one_by_one(model, toks, 32) - want).abs().max().item() <= tol
    # a second sequence in the slot the first one used: its state starts from zero again
    toks2 = random_tokens(300, 40, seed=2)
    assert (run_tail_one_by_one(model, toks2, 10) - toy_plain(W, TOY, toks2).float()).abs().max().item() <= tol
    # two sequences of unequal length in one batch
    slots = model.cache.open(2)
    try:
        lg = model.step([StepEntry(slots[0], toks2, [39]), StepEntry(slots[1], toks, [89])]).float().cpu()
    finally:
        model.cache.close(slots)
    assert (lg[0] - toy_plain(W, TOY, toks2).float()[39]).abs().max().item() <= tol
    assert (lg[1] - want[89]).abs().max().item() <= tol


# ---------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, both defined here.
# ---------------------------------------------------------------------------------------------
class Top1Experts:
    """x += expert_e(h) for the expert e whose router logit is largest (ties to the lower index); every expert is
    a small gated MLP.  Router logits in float32.  Plain tensor operations: it shows the interface, not speed."""

    def __init__(self, spec, layer, rt):
        self.spec, self.layer, self.rt = spec, layer, rt
        self.E = spec.params["experts"]

    def plan(self, prefix, names):
        s = self.spec
        p = {f"{prefix}moe.router.weight": TensorSpec((self.E, s.hidden))}
        for e in range(self.E):
            p[f"{prefix}moe.{e}.gate.weight"] = TensorSpec((s.intermediate, s.hidden))
            p[f"{prefix}moe.{e}.up.weight"] = TensorSpec((s.intermediate, s.hidden))
            p[f"{prefix}moe.{e}.down.weight"] = TensorSpec((s.hidden, s.intermediate))
        return p

    def load(self, tensors, prefix, names):
        self.router = tensors[f"{prefix}moe.router.weight"].to(self.rt.device, torch.float32)
        self.w = [tuple(self.rt.matrix(tensors[f"{prefix}moe.{e}.{n}.weight"]) for n in ("gate", "up", "down"))
                  for e in range(self.E)]

    def nbytes(self):
        return self.router.numel() * 4 + sum(t.numel() * t.element_size() for w in self.w for t in w)

    def forward(self, h, x, batch):
        choice = torch.argmax(h.float() @ self.router.t(), dim=1)        # first maximum = lower index
        for e, (wg, wu, wd) in enumerate(self.w):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                he = h[rows].to(wg.dtype)
                g, u = (he @ wg.t()).float(), (he @ wu.t()).float()
                a = (g / (1 + torch.exp(-g)) * u).to(wd.dtype)
                x[rows] += (a @ wd.t()).float()


class ScaledRope:
    """Rotary encoding over the first rotary_dim dimensions with every frequency divided by ``factor``."""

    def __init__(self, spec, rt):
        self.spec, self.rotary_dim = spec, spec.rotary_dim
        i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / spec.rotary_dim) / spec.params["factor"]
        self.inv_freq = inv.to(torch.float32).to(rt.device).contiguous()


def toy2_spec(cfg) -> ModelSpec:
    H, nh, nkv, hd = cfg["hidden_size"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    names = {"q": "attn.q", "k": "attn.k", "v": "attn.v", "o": "attn.o", "gate": "ffn.gate", "up": "ffn.up",
             "down": "ffn.down", "mixer_norm": "norm1", "ffn_norm": "norm2"}
    norm = NormSpec("rmsnorm", H, cfg["eps"])
    layers = []
    for i in range(cfg["layers"]):
        pos = (PositionSpec("toy_scaled_rope", hd, cfg["rotary_dim"], cfg["theta"], {"factor": cfg["factor"]}) if i % 2 == 0
               else PositionSpec("rope", hd, hd, cfg["theta"]))
        mixer = MixerSpec("attention", H, nh, nkv, hd, True, False, 0, 1.0 / math.sqrt(hd), pos)
        ffn = (FeedForwardSpec("toy_top1_experts", H, cfg["expert_intermediate"], "silu", False, {"experts": cfg["experts"]})
               if i % 2 == 0 else FeedForwardSpec("gated_mlp", H, cfg["intermediate"], "silu"))
        layers.append(BlockSpec("prenorm", mixer, ffn, norm, norm, f"blocks.{i}.", names))
    return ModelSpec("ToyRoutedForCausalLM", cfg["vocab_size"], H, cfg["max_positions"], layers, list(range(cfg["layers"])),
                     norm, False, "embed.weight", "final_norm.weight", "head.weight", embed_scale=cfg["embed_scale"])


TOY2 = dict(embed_scale=3.0, architectures=["ToyRoutedForCausalLM"], model_type="toyrouted", hidden_size=80, vocab_size=211, heads=5,
            kv_heads=1, head_dim=32, rotary_dim=16, factor=4.0, intermediate=120, expert_intermediate=48, experts=3,
            eps=1e-6, theta=5000.0, max_positions=256, layers=3)


def toy2_plain(W, cfg, tokens):
    W = {k: v.double() for k, v in W.items()}
    T = len(tokens)
    nh, nkv, hd, rd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["rotary_dim"]
    posn = torch.arange(T)

    def scaled_partial_rope(u):
        i = torch.arange(rd // 2, dtype=torch.float64)
        ang = posn.double()[:, None] * (cfg["theta"] ** (-2.0 * i / rd) / cfg["factor"])[None, :]
        a, b = u[..., :rd // 2], u[..., rd // 2:rd]
        c, s = ang.cos()[:, None], ang.sin()[:, None]
        return torch.cat([a * c - b * s, a * s + b * c, u[..., rd:]], dim=-1)

    x = plain_embed(W["embed.weight"], tokens) * cfg["embed_scale"]       # the table's rows are scaled as they enter
    for i in range(cfg["layers"]):
        p = f"blocks.{i}."
        h = plain_rmsnorm(x, W[p + "norm1.weight"], cfg["eps"])
        q = plain_linear(h, W[p + "attn.q.weight"], W[p + "attn.q.bias"]).view(T, nh, hd)
        k = plain_linear(h, W[p + "attn.k.weight"], W[p + "attn.k.bias"]).view(T, nkv, hd)
        v = plain_linear(h, W[p + "attn.v.weight"], W[p + "attn.v.bias"]).view(T, nkv, hd)
        if i % 2 == 0:
            q, k = scaled_partial_rope(q), scaled_partial_rope(k)
        else:
            q, k = plain_rope(q, posn, cfg["theta"]), plain_rope(k, posn, cfg["theta"])
        x = x + plain_linear(plain_attention(q, k, v).reshape(T, nh * hd), W[p + "attn.o.weight"])
        h = plain_rmsnorm(x, W[p + "norm2.weight"], cfg["eps"])
        if i % 2 == 0:
            choice = torch.argmax(h @ W[p + "moe.router.weight"].t(), dim=1)
            y = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                y[t] = plain_swiglu_mlp(h[t:t + 1], W[p + f"moe.{e}.gate.weight"], W[p + f"moe.{e}.up.weight"],
                                        W[p + f"moe.{e}.down.weight"])[0]
            x = x + y
        else:
            x = x + plain_swiglu_mlp(h, W[p + "ffn.gate.weight"], W[p + "ffn.up.weight"], W[p + "ffn.down.weight"])
    return plain_linear(plain_rmsnorm(x, W["final_norm.weight"], cfg["eps"]), W["head.weight"]), None


def test_toy_routed_feed_forward_and_another_position_encoding():
    """A feed-forward with routing and a position encoding of the test's own (partial rotary with scaled
    frequencies) are registered from here, built layer by layer beside the package's own parts, and stepped in
    every cutting.  32-bit only: a near-tie between two router logits may fall the other way in bfloat16, which
    says nothing about the interface."""
    from cima_b200.parts import register_feed_forward, register_position
    register_feed_forward("toy_top1_experts", Top1Experts)
    register_position("toy_scaled_rope", ScaledRope)
    register_architecture(ArchitectureEntry("ToyRoutedForCausalLM", "toyrouted", parse=lambda raw: raw, spec=toy2_spec))
    folder = tempfile.mkdtemp(prefix="cima_toy2_")
    write_random_model(folder, TOY2, build_plan(toy2_spec(TOY2)), seed=9)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    model = load_model(folder, dtype="float32", max_tokens=1024, verbose=False)
    toks = random_tokens(TOY2["vocab_size"], 100, seed=4)
    want = toy2_plain(W, TOY2, toks)[0].float()
    assert (run_whole(model, toks) - want).abs().max().item() <= 2e-5
    assert (run_tail_one_by_one(model, toks, 32) - want).abs().max().item() <= 2e-5
    toks2 = random_tokens(TOY2["vocab_size"], 33, seed=5)
    slots = model.cache.open(2)
    try:
        lg = model.step([StepEntry(slots[0], toks2, [32]), StepEntry(slots[1], toks, [99])]).float().cpu()
    finally:
        model.cache.close(slots)
    assert (lg[0] - toy2_plain(W, TOY2, toks2)[0].float()[32]).abs().max().item() <= 2e-5
    assert (lg[1] - want[99]).abs().max().item() <= 2e-5


# ---------------------------------------------------------------------------------------------
# Generation with the toy architectures through the package's entry point.
# ---------------------------------------------------------------------------------------------
def toy_generate(plain, W, cfg, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        lg = plain(W, cfg, seq)
        lg = (lg[0] if isinstance(lg, tuple) else lg)[-1].float()
        best = max(range(lg.numel()), key=lambda i: (float(lg[i]), i))        # ties to the higher index
        out.append(best)
        seq.append(best)
    return out


@pytest.mark.parametrize("mean_kind,pipeline", [("causal_mean", True), ("causal_mean_on_device", True),
                                                ("causal_mean_on_device", False)])
def test_toy_architecture_with_state_generates_through_the_entry_point(mean_kind, pipeline):
    """``cima_b200.load(...).generate`` with the stateful toy mixer: the variant that reads the batch on the host is
    decoded step by step (it does not declare itself fit for recording), the other through recorded steps; neither
    runs ahead (a step too many would leave its running sum one token ahead of the cache).  A finished sequence is
    kept (``retain``) and the next turn goes on from its keys and its state; every token equals the plain model's."""
    register_mixer("causal_mean", CausalMean)
    register_mixer("causal_mean_on_device", CausalMeanOnDevice)
    register_architecture(ArchitectureEntry("ToyMixForCausalLM", "toymix", parse=lambda raw: raw, spec=toy_spec))
    cfg = dict(TOY, mean_kind=mean_kind)
    folder = tempfile.mkdtemp(prefix="cima_toy_gen_")
    cima_b200.write_random_model(folder, cfg, seed=5)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    lm = cima_b200.load(folder, dtype="float32", max_tokens=2048, verbose=False, pipeline=pipeline, retain=1)
    assert lm.stepper.use_graphs == (mean_kind == "causal_mean_on_device")
    assert lm.stepper.pipeline is False and lm.model.cache.has_mixer_state
    prompts = [random_tokens(300, n, seed=10 + n) for n in (23, 5, 40)]
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=9)
    for p, r in zip(prompts, got):
        assert r.tokens == toy_generate(toy_plain, W, TOY, p, 9)
    # the next turn of the last conversation: only the new tokens run, from the kept keys and the kept running sums
    turn2 = prompts[2] + got[2].tokens + random_tokens(300, 7, seed=99)
    r2 = lm.generate([turn2], temperature=0, repeat_penalty=1.0, max_tokens=9)[0]
    assert lm.stats.reused_tokens == len(prompts[2]) + len(got[2].tokens) - 1
    assert r2.tokens == toy_generate(toy_plain, W, TOY, turn2, 9)
    # a prompt that shares only a part of the kept sequence cannot go back there (the state belongs to its end)
    turn3 = turn2[:30] + random_tokens(300, 6, seed=98)
    r3 = lm.generate([turn3], temperature=0, repeat_penalty=1.0, max_tokens=5)[0]
    assert lm.stats.reused_tokens == 0 and r3.tokens == toy_generate(toy_plain, W, TOY, turn3, 5)
    lm.stepper.drop_retained()
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0


@pytest.mark.parametrize("pipeline", [True, False])
def test_toy_routed_architecture_generates_through_the_entry_point(pipeline):
    """The routed feed-forward says nothing about recording, so the model decodes step by step; greedy tokens of a
    batch of unequal prompts equal the plain model's (32-bit)."""
    from cima_b200.parts import register_feed_forward, register_position
    register_feed_forward("toy_top1_experts", Top1Experts)
    register_position("toy_scaled_rope", ScaledRope)
    register_architecture(ArchitectureEntry("ToyRoutedForCausalLM", "toyrouted", parse=lambda raw: raw, spec=toy2_spec))
    lm = cima_b200.load(config=TOY2, seed=9, dtype="float32", max_tokens=1024, verbose=False, pipeline=pipeline)
    assert not lm.stepper.use_graphs
    folder = tempfile.mkdtemp(prefix="cima_toy2_gen_")
    cima_b200.write_random_model(folder, TOY2, seed=9)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompts = [random_tokens(TOY2["vocab_size"], n, seed=30 + n) for n in (12, 1, 33)]
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=8)
    for p, r in zip(prompts, got):
        assert r.tokens == toy_generate(toy2_plain, W, TOY2, p, 8)
    assert lm.model.cache.slots.held == 0
