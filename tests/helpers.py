"""Tiny configurations and helpers shared by the tests."""
from __future__ import annotations

import os
import tempfile

import numpy as np
import torch

import cima_b200
from cima_b200.engine import StepEntry, load_model

# Three tiny configurations that differ in every size and option.
TINY_A = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=128,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=256, vocab_size=512,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
              max_position_embeddings=128)
TINY_B = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=192,
              num_attention_heads=3, num_key_value_heads=1, head_dim=64, intermediate_size=448, vocab_size=1000,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, use_sliding_window=False,
              max_position_embeddings=256)
# hidden != heads * head_dim, a head size that is no power of two, a window on the later layers
TINY_C = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=4, hidden_size=200,
              num_attention_heads=6, num_key_value_heads=2, head_dim=48, intermediate_size=328, vocab_size=777,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, use_sliding_window=True,
              sliding_window=40, max_window_layers=2, max_position_embeddings=512)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}

_FOLDERS = {}


def model_folder(name: str, seed: int = 0) -> str:
    """A temporary model folder of a tiny configuration (made once per process)."""
    key = (name, seed)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"cima_tiny_{name}_")
        cima_b200.write_random_model(d, TINY[name], seed=seed)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def cpu_model(name: str, dtype="float32", max_tokens=1024, seed=0, **kw):
    from reference_kernels import ReferenceKernels
    return load_model(model_folder(name, seed), dtype=dtype, max_tokens=max_tokens, device="cpu",
                      kernels=ReferenceKernels(), **kw)


def gpu_model(name: str, dtype="float32", max_tokens=1024, seed=0, **kw):
    return load_model(model_folder(name, seed), dtype=dtype, max_tokens=max_tokens, device="cuda:0",
                      verbose=False, **kw)


def run_whole(model, tokens):
    """Logits at every position of one sequence fed whole; the slot is given back."""
    (slot,) = model.cache.open(1)
    try:
        return model.step([StepEntry(slot, tokens, list(range(len(tokens))))]).float().cpu()
    finally:
        model.cache.close([slot])


def run_tail_one_by_one(model, tokens, tail):
    """The same, the last ``tail`` tokens fed one by one."""
    (slot,) = model.cache.open(1)
    try:
        head = len(tokens) - tail
        outs = []
        if head > 0:
            outs.append(model.step([StepEntry(slot, tokens[:head], list(range(head)))]).float().cpu())
        for t in tokens[head:]:
            outs.append(model.step([StepEntry(slot, [t], [0])]).float().cpu())
        return torch.cat(outs)
    finally:
        model.cache.close([slot])


def run_in_pieces(model, seqs, cuts):
    """Sequences as one batch fed in pieces: step k brings tokens [cuts[i][k-1], cuts[i][k]) of sequence i (a
    sequence whose cuts are used up sits the step out).  All logits per sequence."""
    slots = model.cache.open(len(seqs))
    try:
        outs = [[] for _ in seqs]
        bounds = [[0] + list(c) + [len(q)] for q, c in zip(seqs, cuts)]
        for k in range(max(len(b) for b in bounds) - 1):
            live = [i for i, b in enumerate(bounds) if k + 1 < len(b) and b[k + 1] > b[k]]
            if not live:
                continue
            entries = [StepEntry(slots[i], seqs[i][bounds[i][k]:bounds[i][k + 1]], list(range(bounds[i][k + 1] - bounds[i][k])))
                       for i in live]
            lg = model.step(entries).float().cpu()
            r = 0
            for i in live:
                n = bounds[i][k + 1] - bounds[i][k]
                outs[i].append(lg[r:r + n]); r += n
        return [torch.cat(o) for o in outs]
    finally:
        model.cache.close(slots)


def run_batched(model, seqs, decode_from):
    """Sequences as one batch: tokens [0, decode_from[i]) as prompts in one step, then one token each
    per step until each sequence's own end; shorter ones end earlier.  Returns logits per sequence."""
    slots = model.cache.open(len(seqs))
    try:
        outs = [[] for _ in seqs]
        entries = [StepEntry(s, q[:d], list(range(d))) for s, q, d in zip(slots, seqs, decode_from)]
        lg = model.step(entries).float().cpu()
        r = 0
        for i, d in enumerate(decode_from):
            outs[i].append(lg[r:r + d]); r += d
        step = 0
        while True:
            live = [i for i, (q, d) in enumerate(zip(seqs, decode_from)) if d + step < len(q)]
            if not live:
                break
            lg = model.step([StepEntry(slots[i], [seqs[i][decode_from[i] + step]], [0]) for i in live]).float().cpu()
            for j, i in enumerate(live):
                outs[i].append(lg[j:j + 1])
            step += 1
        return [torch.cat(o) for o in outs]
    finally:
        model.cache.close(slots)
