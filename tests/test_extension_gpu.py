"""Generality of the parts: a toy mixer with state of its own, defined here, is registered, built
into a toy architecture (also registered here) and stepped, without any change to the package.
The toy model also runs one layer twice (each run with storage of its own) and lets one attention
layer read another layer's keys and values."""
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
            mixer = MixerSpec("causal_mean", H, 0, 0, 0, False, False, 0, 0.0, PositionSpec("none", 0, 0, 1.0))
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
