"""Plain, slow implementation of the Qwen2 dense decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function for each part, float64 by
default. It shares no code with the ``cima_b200`` package: it reads
``config.json`` as a plain dict and ``model.safetensors`` through the
``safetensors`` Python package (an independent reader of the container).

It rests on the formulas of juliog922/cima's source (cited per function, paths
within that project); the reference's own model code is Rust and cannot be
compiled or imported here (no cargo/rustc on this machine), so no output of
the reference anchors it.  Independent cross-checks live in
``tests/test_plain.py`` (dense masked softmax, rotation as complex product).
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- parts

def plain_embed(table: torch.Tensor, ids) -> torch.Tensor:
    """x[t,:] = E[ids[t],:], no scaling (src/kernels.cu:10-21,
    src/models/transformer.rs:1324-1357)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = 1/sqrt(mean(x^2) + eps); y = x * inv * w, the weight being plain w
    (src/kernels.cu:37-50).  The +-65000 clamp of the reads there is an f16
    guard and has no counterpart here."""
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * w


def plain_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """C[m,n] = sum_k A[m,k] * B[n,k] (+ bias[n]): weights are [out, in]
    (src/kernels.cu:1410-1431, bias src/kernels.cu:390-393)."""
    y = x @ w.transpose(0, 1)
    if b is not None:
        y = y + b
    return y


def plain_rope(u: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotary (src/kernels.cu:397-414): for i < hd/2 pair (i, i+hd/2),
    f_i = theta^(-2i/hd), a = p * f_i,
    u_i' = u_i cos a - u_{i+hd/2} sin a,  u_{i+hd/2}' = u_i sin a + u_{i+hd/2} cos a.
    ``u`` is [T, heads, hd]; ``positions`` [T] absolute positions."""
    hd = u.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=u.dtype)
    freq = torch.pow(torch.tensor(theta, dtype=u.dtype), -2.0 * i / hd)
    ang = positions.to(u.dtype)[:, None] * freq[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = u[..., :half], u[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q [T, nh, hd], k/v [T, nkv, hd]. Head h reads group g = h / (nh / nkv);
    s_j = (q . k_j) / sqrt(hd); the query at p sees keys j <= p, and with a
    window > 0 only those with p - j < window; softmax over the visible keys;
    o = sum_j softmax_j v_j  (src/kernels.cu:458-491 for group, scale and the
    window's start ``seq - window``; src/kernels.cu:700-712 for the mask of
    prefill).  Written as a loop over queries with a plain softmax."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // rep
        for p in range(T):
            lo = max(0, p + 1 - window) if window > 0 else 0
            s = (k[lo:p + 1, g, :] @ q[p, h, :]) * scale
            w = torch.softmax(s, dim=0)
            out[p, h, :] = w @ v[lo:p + 1, g, :]
    return out


def plain_swiglu_mlp(h: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """g = h Wg^T, u = h Wu^T, a = g / (1 + exp(-g)) * u, out = a Wd^T; no biases
    (src/kernels.cu:81-84, src/models/transformer.rs:1273-1291)."""
    g = plain_linear(h, wg)
    u = plain_linear(h, wu)
    a = g / (1.0 + torch.exp(-g)) * u
    return plain_linear(a, wd)


def plain_layer_window(cfg: dict, layer: int) -> int:
    """Window of a layer's attention.  The reference hard-wires window = 0 for
    this architecture and does not read the keys (src/models/transformer.rs:
    1184-1199); its attention kernels take a per-call ``window``
    (src/kernels.cu:459).  This build reads config.json's own keys: with
    ``use_sliding_window`` true, layers from ``max_window_layers`` on look at the
    last ``sliding_window`` keys; otherwise every layer sees all keys.  A
    ``layer_types`` list, where given, names the windowed layers itself."""
    if cfg.get("layer_types") is not None:
        return int(cfg["sliding_window"]) if cfg["layer_types"][layer] == "sliding_attention" else 0
    if not cfg.get("use_sliding_window", False):
        return 0
    if layer >= int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return int(cfg["sliding_window"])
    return 0


def plain_block(x, W, cfg, layer, positions):
    """Pre-norm block: h = RMSNorm(x) -> attention -> residual; h = RMSNorm(x) ->
    MLP -> residual (src/models/transformer.rs:1024-1319, table of steps 1-11)."""
    p = f"model.layers.{layer}."
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim", cfg["hidden_size"] // nh)
    eps = cfg.get("rms_norm_eps", 1e-6)
    theta = cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta", 10000.0)
    T = x.shape[0]
    h = plain_rmsnorm(x, W[p + "input_layernorm.weight"], eps)
    q = plain_linear(h, W[p + "self_attn.q_proj.weight"], W[p + "self_attn.q_proj.bias"]).view(T, nh, hd)
    k = plain_linear(h, W[p + "self_attn.k_proj.weight"], W[p + "self_attn.k_proj.bias"]).view(T, nkv, hd)
    v = plain_linear(h, W[p + "self_attn.v_proj.weight"], W[p + "self_attn.v_proj.bias"]).view(T, nkv, hd)
    q = plain_rope(q, positions, theta)
    k = plain_rope(k, positions, theta)
    att = plain_attention(q, k, v, plain_layer_window(cfg, layer)).reshape(T, nh * hd)
    x = x + plain_linear(att, W[p + "self_attn.o_proj.weight"])
    h = plain_rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps)
    x = x + plain_swiglu_mlp(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                             W[p + "mlp.down_proj.weight"])
    return x


def plain_head(x, W, cfg):
    """Final RMSNorm with model.norm.weight, then logits = h W_head^T with
    W_head = lm_head.weight unless tied (or absent), no bias, no softcap
    (src/models/transformer.rs:837-846, 1361-1384, 1631-1652)."""
    h = plain_rmsnorm(x, W["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    tied = cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in W
    head = W["model.embed_tokens.weight"] if tied else W["lm_head.weight"]
    return plain_linear(h, head)


def plain_forward(W: dict, cfg: dict, tokens, dtype=torch.float64) -> torch.Tensor:
    """Logits [T, V] of one whole sequence, every position."""
    W = {k: v.to(dtype) for k, v in W.items()}
    T = len(tokens)
    positions = torch.arange(T)
    x = plain_embed(W["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        x = plain_block(x, W, cfg, layer, positions)
    return plain_head(x, W, cfg)


def plain_load(folder: str):
    """(config dict, {tensor name: tensor}) of a model folder."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- sampling

class PlainXorshift:
    """xorshift64* as in src/models/mod.rs:69-78; state = max(seed, 1)."""
    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = max(int(seed), 1) & self.MASK

    def next_f32(self) -> float:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & self.MASK
        x ^= x >> 27
        self.state = x
        return float(((x * 0x2545F4914F6CDD1D) & self.MASK) >> 40) / float(1 << 24)


def plain_sample(logits, history, opts: dict, rng: PlainXorshift) -> int:
    """The reference's chain (src/models/mod.rs:86-201) in float32 arithmetic:
    repeat penalty over the last 64 tokens of history, once per occurrence;
    temperature <= 0 -> argmax with ties to the higher index; top-k by
    (value desc, index desc); p = exp((l - max) / max(T, 1e-4)) normalised;
    top-p keeps the shortest prefix whose mass reaches top_p; draw
    r = u * sum(kept), walk until r <= 0."""
    import numpy as np
    l = np.array(logits, dtype=np.float32).copy()
    rp = np.float32(opts.get("repeat_penalty", 1.0))
    if rp != 1.0:
        for t in history[-64:]:
            if 0 <= t < len(l):
                l[t] = l[t] / rp if l[t] > 0 else l[t] * rp
    temp = float(opts.get("temperature", 0.0))
    if temp <= 0.0:
        best = 0
        for i in range(len(l)):
            if l[i] >= l[best]:
                best = i
        return int(best)
    k = int(opts.get("top_k", 0))
    k = len(l) if k == 0 else min(k, len(l))
    order = sorted(range(len(l)), key=lambda i: (-float(l[i]), -i))[:k]
    vals = l[order]
    inv_t = np.float32(1.0) / np.float32(max(temp, 1e-4))
    probs = np.exp((vals - vals[0]) * inv_t).astype(np.float32)
    total = np.float32(0.0)
    for p in probs:
        total = np.float32(total + p)
    probs = (probs / total).astype(np.float32)
    top_p = np.float32(opts.get("top_p", 1.0))
    cut, cum = len(probs), np.float32(0.0)
    for i, p in enumerate(probs):
        cum = np.float32(cum + p)
        if cum >= top_p:
            cut = i + 1
            break
    probs = probs[:cut]
    renorm = np.float32(0.0)
    for p in probs:
        renorm = np.float32(renorm + p)
    r = np.float32(np.float32(rng.next_f32()) * renorm)
    for i, p in enumerate(probs):
        r = np.float32(r - p)
        if r <= 0.0:
            return int(order[i])
    return int(order[cut - 1])
