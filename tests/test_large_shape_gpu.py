"""The Qwen2.5-7B layer shape (hidden 3584, 28/4 heads of 128, intermediate 18944) with two layers and a
smaller vocabulary: the kernels at the sizes the benchmark runs them, against the plain implementation
(float64, CPU) and against each other in every cutting."""
import tempfile

import pytest
import torch

import cima_b200
from cima_b200.engine import load_model
from helpers import random_tokens, run_batched, run_tail_one_by_one, run_whole
from qwen2_plain import plain_forward, plain_load

pytestmark = pytest.mark.gpu

# The tiny models' bfloat16 tolerance (2e-2 on logits whose standard deviation is 0.28) as a fraction of
# the logits' standard deviation; at this width the logits are about four times larger.
REL_BF16 = 2e-2 / 0.28

SHAPE = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584,
             num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
             vocab_size=20008, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
             use_sliding_window=False, max_position_embeddings=4096)


@pytest.fixture(scope="module")
def folder():
    d = tempfile.mkdtemp(prefix="cima_7bshape_")
    cima_b200.write_random_model(d, SHAPE, seed=11)
    return d


def test_7b_layer_shape_in_every_cutting(folder):
    cfg, W = plain_load(folder)
    toks = random_tokens(SHAPE["vocab_size"], 100, seed=1)
    want = plain_forward(W, cfg, toks).float()
    m32 = load_model(folder, dtype="float32", max_tokens=4096, verbose=False)
    whole32 = run_whole(m32, toks)
    # sums over 3584 to 18944 float32 terms, two layers, logits of magnitude about 1
    assert (whole32 - want).abs().max().item() <= 1e-4
    assert torch.equal(run_tail_one_by_one(m32, toks, 32), whole32)
    del m32
    torch.cuda.empty_cache()
    m16 = load_model(folder, dtype="bfloat16", max_tokens=4096, verbose=False)
    tol = REL_BF16 * want.std().item()
    whole16 = run_whole(m16, toks)
    assert (whole16 - want).abs().max().item() <= tol
    assert (run_tail_one_by_one(m16, toks, 32) - want).abs().max().item() <= tol
    seqs = [random_tokens(SHAPE["vocab_size"], n, seed=20 + n) for n in (70, 9, 130, 31)] + [toks]
    got = run_batched(m16, seqs, [60, 1, 100, 20, 68])
    assert (got[4] - want).abs().max().item() <= tol
    for q, g in zip(seqs[:2], got[:2]):
        assert (g - plain_forward(W, cfg, q).float()).abs().max().item() <= tol
    m16.cache.check()


def test_long_context_decode_against_whole_prompt(folder):
    """3,000 positions: the last 8 tokens one by one (split-KV decode attention over 47 pages) against the
    same positions of the whole prompt (flash prefill), bfloat16; both against float32 at the end."""
    toks = random_tokens(SHAPE["vocab_size"], 3000, seed=3)
    m16 = load_model(folder, dtype="bfloat16", max_tokens=4096, verbose=False)
    (slot,) = m16.cache.open(1)
    from cima_b200.engine import StepEntry
    try:
        whole = m16.step([StepEntry(slot, toks, list(range(2992, 3000)))]).float().cpu()
    finally:
        m16.cache.close([slot])
    (slot,) = m16.cache.open(1)
    try:
        m16.step([StepEntry(slot, toks[:2992], [])])
        tail = torch.cat([m16.step([StepEntry(slot, [t], [0])]).float().cpu() for t in toks[2992:]])
    finally:
        m16.cache.close([slot])
    tol = REL_BF16 * whole.std().item()
    assert (tail - whole).abs().max().item() <= tol
    del m16
    torch.cuda.empty_cache()
    m32 = load_model(folder, dtype="float32", max_tokens=4096, verbose=False)
    (slot,) = m32.cache.open(1)
    try:
        ref = m32.step([StepEntry(slot, toks, list(range(2992, 3000)))]).float().cpu()
    finally:
        m32.cache.close([slot])
    assert (whole - ref).abs().max().item() <= tol and (tail - ref).abs().max().item() <= tol


WIDER = {"14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824),
         "32b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648)}


@pytest.mark.parametrize("name", ["14b", "32b"])
def test_wider_layer_shapes(name, tmp_path):
    """One layer of the Qwen2.5-14B and -32B shapes (hidden 5120: 320 partial sums per row for the folded norm,
    more than the 256 a lane's registers take; 40/8 heads; intermediate 13,824 or 27,648): a prompt whole, its
    last 16 tokens one by one, and a 300-token prompt (the tcgen05 attention) in bfloat16 against float32."""
    shape = dict(SHAPE, num_hidden_layers=1, vocab_size=5000, **WIDER[name])
    folder = str(tmp_path / name)
    cima_b200.write_random_model(folder, shape, seed=13)
    cfg, W = plain_load(folder)
    toks = random_tokens(shape["vocab_size"], 72, seed=2)
    want = plain_forward(W, cfg, toks).float()
    long_toks = random_tokens(shape["vocab_size"], 300, seed=4)
    m32 = load_model(folder, dtype="float32", max_tokens=1024, verbose=False)
    assert (run_whole(m32, toks) - want).abs().max().item() <= 1e-4
    long32 = run_whole(m32, long_toks)
    del m32
    torch.cuda.empty_cache()
    m16 = load_model(folder, dtype="bfloat16", max_tokens=1024, verbose=False)
    tol = REL_BF16 * want.std().item()
    assert (run_whole(m16, toks) - want).abs().max().item() <= tol
    assert (run_tail_one_by_one(m16, toks, 16) - want).abs().max().item() <= tol
    assert (run_whole(m16, long_toks) - long32).abs().max().item() <= REL_BF16 * long32.std().item()
    m16.check_device()


def test_ragged_long_prompts_in_one_step(folder):
    """Five prompts of 1 to 700 tokens in one step (the longest decides that the tcgen05 attention runs: blocks
    of 128 query rows, sequences that end inside a block, one of a single token), bfloat16 against float32, at
    every sequence's last position and at a few inside."""
    from cima_b200.engine import StepEntry
    lens = [700, 130, 1, 257, 300]
    seqs = [random_tokens(SHAPE["vocab_size"], n, seed=40 + n) for n in lens]
    wants = [sorted({0, n // 2, max(0, n - 2), n - 1}) for n in lens]

    def run(dtype):
        m = load_model(folder, dtype=dtype, max_tokens=2048, verbose=False)
        slots = m.cache.open(len(seqs))
        try:
            out = m.step([StepEntry(s, t, w) for s, t, w in zip(slots, seqs, wants)]).float().cpu()
            m.check_device()
        finally:
            m.cache.close(slots)
        del m
        torch.cuda.empty_cache()
        return out

    got16, got32 = run("bfloat16"), run("float32")
    assert got16.shape == got32.shape == (sum(len(w) for w in wants), SHAPE["vocab_size"])
    assert (got16 - got32).abs().max().item() <= REL_BF16 * got32.std().item()
