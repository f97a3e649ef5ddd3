"""Trace replay's bookkeeping (ids to slots, files, 'done' lines) on the CPU stand-in kernels."""
import io
import json
import os

import numpy as np
import torch

from helpers import model_folder, random_tokens
from qwen2_plain import plain_forward, plain_load
from reference_kernels import ReferenceKernels
from cima_b200.engine.trace import replay


def test_replay_writes_wanted_logits(tmp_path):
    folder = model_folder("A")
    cfg, W = plain_load(folder)
    a, b = random_tokens(512, 9, 1), random_tokens(512, 4, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:3], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [a[7]], "want": [0]}, {"id": "b", "tokens": [b[3]], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[8]], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [3]}], "end": ["c"]},
    ]
    out = io.StringIO()
    replay(folder, "float32", str(tmp_path), 256, [json.dumps(s) for s in steps], out=out, device="cpu",
           kernels=ReferenceKernels())
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(tmp_path)) == ["0.f32", "1.f32", "3.f32"]
    pa, pb = plain_forward(W, cfg, a).float(), plain_forward(W, cfg, b).float()
    s0 = torch.from_numpy(np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, 512))
    assert torch.allclose(s0, pa[[0, 6]], atol=2e-4)
    s1 = torch.from_numpy(np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(2, 512))
    assert torch.allclose(s1, torch.stack([pa[7], pb[3]]), atol=2e-4)
    s3 = torch.from_numpy(np.fromfile(tmp_path / "3.f32", dtype="<f4").reshape(1, 512))
    assert torch.allclose(s3[0], pb[3], atol=2e-4)


def test_replay_takes_a_request_that_goes_on_by_several_tokens(tmp_path):
    """A prompt cut into two steps beside a request that starts in the second: the same logits as whole."""
    folder = model_folder("A")
    cfg, W = plain_load(folder)
    a, b = random_tokens(512, 40, 3), random_tokens(512, 6, 4)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [24]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[25:], "want": [0, 14]}, {"id": "b", "tokens": b, "want": [5]}], "end": ["a", "b"]},
    ]
    out = io.StringIO()
    replay(folder, "float32", str(tmp_path), 256, [json.dumps(s) for s in steps], out=out, device="cpu",
           kernels=ReferenceKernels())
    assert out.getvalue().split() == ["done", "0", "done", "1"]
    pa, pb = plain_forward(W, cfg, a).float(), plain_forward(W, cfg, b).float()
    s1 = torch.from_numpy(np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(3, 512))
    assert torch.allclose(s1, torch.stack([pa[25], pa[39], pb[5]]), atol=2e-4)
