"""The package's host logic (cache, block tables, step function) driven on the CPU through plain
statements of the kernels, compared with the plain implementation."""
import torch
import pytest

from helpers import TINY, cpu_model, model_folder, random_tokens, run_batched, run_tail_one_by_one, run_whole
from qwen2_plain import plain_forward, plain_load


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
