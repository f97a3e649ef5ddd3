"""Safetensors container, weights by name and their one error, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import cima_b200
from cima_b200.engine import build_plan
from cima_b200.config import Qwen2Config
from cima_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors, parse_header,
                               write_safetensors)
from helpers import TINY_A, TINY_B


def blob(header: dict, data: bytes = b"") -> bytes:
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


def test_header_validation_cases():
    """The cases of the reference's header tests (src/formats.rs:1598-1654) and a few more."""
    with pytest.raises(SafetensorsError, match="too short"):
        parse_header(b"\x00\x01", "f")
    with pytest.raises(SafetensorsError, match="exceeds"):
        parse_header(struct.pack("<Q", 1 << 40) + b"{}", "f")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        parse_header(struct.pack("<Q", 4) + b"nope", "f")
    with pytest.raises(SafetensorsError, match="not a JSON object"):
        parse_header(blob([1, 2]), "f")
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    assert parse_header(blob(ok, b"\0" * 8), "f")[0]["a"]["shape"] == (2,)
    with pytest.raises(SafetensorsError, match="outside the data"):
        parse_header(blob(ok, b"\0" * 4), "f")
    with pytest.raises(SafetensorsError, match="needs 8 bytes but spans 4"):
        parse_header(blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8), "f")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        parse_header(blob({"a": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 8), "f")
    with pytest.raises(SafetensorsError, match="overlap"):
        parse_header(blob({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]},
                           "b": {"dtype": "U8", "shape": [4], "data_offsets": [2, 6]}}, b"\0" * 8), "f")
    with pytest.raises(SafetensorsError, match="malformed shape"):
        parse_header(blob({"a": {"dtype": "U8", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 8), "f")


def test_round_trip_with_an_independent_reader_and_writer(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"w": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "i": torch.arange(6, dtype=torch.int64).view(2, 3),
         "h": torch.randn(4).to(torch.float16)}
    write_safetensors(str(tmp_path / "mine.safetensors"), t)
    theirs = load_file(str(tmp_path / "mine.safetensors"))
    assert all(torch.equal(theirs[k], v) for k, v in t.items())
    save_file(t, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(str(tmp_path / "theirs.safetensors"))
    assert all(torch.equal(f.read(k), v) for k, v in t.items())
    f.close()


def test_dtype_rule_of_the_loader(tmp_path):
    from cima_b200.weights import TensorSpec
    t = {"bf": torch.randn(2, 2).to(torch.bfloat16), "f32": torch.randn(2), "f16": torch.randn(2).to(torch.float16),
         "i64": torch.arange(3), "f64": torch.randn(2, dtype=torch.float64)}
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    got = load_tensors(str(tmp_path), {k: TensorSpec(tuple(v.shape)) for k, v in t.items()})
    assert got["bf"].dtype is torch.bfloat16 and got["f32"].dtype is torch.float32      # stored dtypes stay
    assert got["f16"].dtype is torch.float16 and got["f64"].dtype is torch.float32       # float16: the model's precision settles it
    from cima_b200.parts import Runtime
    assert Runtime(None, torch.bfloat16, "cpu").matrix(got["f16"].view(1, 2)).dtype is torch.bfloat16
    wide = Runtime(None, torch.float32, "cpu").matrix(got["f16"].view(1, 2))
    assert wide.dtype is torch.float32 and torch.equal(wide.view(2), t["f16"].float())   # exactly, not by way of bfloat16
    assert got["i64"].dtype is torch.int32 and got["i64"].tolist() == [0, 1, 2]          # integer tables as int32
    assert torch.equal(got["f32"], t["f32"])


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    cima_b200.write_random_model(str(tmp_path), TINY_A, seed=1)
    plan = build_plan(Qwen2Config.from_dict(TINY_A).model_spec())
    good = load_tensors(str(tmp_path), plan)
    assert set(good) == set(plan) and all(v.dtype is torch.bfloat16 for v in good.values())
    bad = dict(good)
    del bad["model.layers.1.self_attn.k_proj.bias"]                 # a missing q/k/v bias is an error here
    del bad["model.norm.weight"]
    bad["model.layers.0.mlp.down_proj.weight"] = torch.zeros(128, 255, dtype=torch.bfloat16)
    bad["model.layers.9.extra.weight"] = torch.zeros(3)
    write_safetensors(str(tmp_path / "model.safetensors"), bad)
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path), plan)
    msg = str(e.value)
    assert e.value.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.9.extra.weight"]
    assert e.value.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (128, 255), (128, 256))]
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "found [128, 255], expected [128, 256]"):
        assert needle in msg


def test_tied_model_may_hold_a_head_untied_must(tmp_path):
    plan_a = build_plan(Qwen2Config.from_dict(TINY_A).model_spec())
    assert "lm_head.weight" not in plan_a
    plan_b = build_plan(Qwen2Config.from_dict(TINY_B).model_spec())
    assert plan_b["lm_head.weight"].shape == (1000, 192)
    assert plan_b["model.layers.2.self_attn.q_proj.weight"].shape == (192, 192)
    assert plan_b["model.layers.2.self_attn.k_proj.bias"].shape == (64,)
    cima_b200.write_random_model(str(tmp_path), TINY_A, seed=1)
    t = load_tensors(str(tmp_path), plan_a)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    assert set(load_tensors(str(tmp_path), plan_a, ignore=["lm_head.weight"])) == set(plan_a)
    with pytest.raises(WeightError, match="unexpected"):
        load_tensors(str(tmp_path), plan_a)


def test_a_checkpoint_may_leave_out_the_model_prefix(tmp_path):
    """A bare backbone stores ``layers.0...``; the plan's names are served by it when the architecture allows
    the prefix to be absent, and the error still lists what is wrong under the stored names."""
    spec = Qwen2Config.from_dict(TINY_A).model_spec()
    plan = build_plan(spec)
    cima_b200.write_random_model(str(tmp_path), TINY_A, seed=1)
    t = load_tensors(str(tmp_path), plan)
    bare = {(n[len("model."):] if n.startswith("model.") else n): v for n, v in t.items()}
    write_safetensors(str(tmp_path / "model.safetensors"), bare)
    with pytest.raises(WeightError, match="missing"):
        load_tensors(str(tmp_path), plan)
    got = load_tensors(str(tmp_path), plan, optional_prefixes=spec.optional_prefixes)
    assert set(got) == set(plan) and all(torch.equal(got[n], t[n]) for n in plan)
    bare["layers.1.mlp.up_proj.weight"] = bare["layers.1.mlp.up_proj.weight"][:, :-1].contiguous()
    bare["extra.weight"] = torch.zeros(2)
    write_safetensors(str(tmp_path / "model.safetensors"), bare)
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path), plan, optional_prefixes=spec.optional_prefixes)
    assert e.value.unexpected == ["extra.weight"] and e.value.wrong_shape[0][0] == "layers.1.mlp.up_proj.weight"


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    cima_b200.write_random_model(str(tmp_path / "a"), TINY_A, seed=1)
    cima_b200.write_random_model(str(tmp_path / "b"), TINY_A, seed=1)
    cima_b200.write_random_model(str(tmp_path / "c"), TINY_A, seed=2)
    from safetensors.torch import load_file
    a, b, c = (load_file(str(tmp_path / d / "model.safetensors")) for d in "abc")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 2e-3 and abs(w.mean().item()) < 1e-3
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 1e-2
    # a tensor's values do not depend on what else the model holds
    cima_b200.write_random_model(str(tmp_path / "d"), dict(TINY_A, num_hidden_layers=1), seed=1)
    d = load_file(str(tmp_path / "d" / "model.safetensors"))
    assert torch.equal(d["model.layers.0.mlp.up_proj.weight"], a["model.layers.0.mlp.up_proj.weight"])


def test_shards_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "p1.safetensors"), {"a": torch.zeros(2)})
    write_safetensors(str(tmp_path / "p2.safetensors"), {"b": torch.ones(2)})
    json.dump({"weight_map": {"a": "p1.safetensors", "b": "p2.safetensors"}}, open(tmp_path / "model.safetensors.index.json", "w"))
    from cima_b200.weights import TensorSpec
    got = load_tensors(str(tmp_path), {"a": TensorSpec((2,)), "b": TensorSpec((2,))})
    assert got["b"].tolist() == [1.0, 1.0]
    write_safetensors(str(tmp_path / "p2.safetensors"), {"b": torch.ones(2), "a": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="appears in both"):
        load_tensors(str(tmp_path), {"a": TensorSpec((2,)), "b": TensorSpec((2,))})
    os.remove(tmp_path / "p1.safetensors")
    with pytest.raises(SafetensorsError, match="does not exist"):
        load_tensors(str(tmp_path), {"a": TensorSpec((2,))})


def test_source_hands_out_one_tensor_at_a_time(tmp_path):
    """``CheckpointTensors`` reads a tensor when it is asked for and counts what is alive: a consumer that drops
    each tensor before it asks for the next (as an upload to the device does) never holds more than the largest
    one; the whole plan is checked when the source opens, before anything is read."""
    from helpers import TINY, model_folder
    from cima_b200.weights import CheckpointTensors
    cfg = Qwen2Config.from_dict(TINY["B"])
    plan = build_plan(cfg.model_spec())
    size = {n: 2 * int(np.prod(s.shape)) for n, s in plan.items()}
    with CheckpointTensors(model_folder("B"), plan) as src:
        assert sorted(src.names()) == sorted(plan) and src.live_bytes == 0
        for n in plan:
            t = src[n]
            assert tuple(t.shape) == tuple(plan[n].shape) and src.live_bytes == size[n]
            del t
            assert src.live_bytes == 0
        assert src.peak_bytes == max(size.values()) and src.fetched == list(plan)
    bad = dict(plan)
    bad["model.layers.9.mlp.up_proj.weight"] = plan["model.layers.0.mlp.up_proj.weight"]
    with pytest.raises(WeightError, match="missing"):
        CheckpointTensors(model_folder("B"), bad)


def test_state_dict_of_a_seeded_model_is_the_random_weights_mode(tmp_path):
    """A model made from a configuration and a seed in memory holds exactly ``random_tensors(plan, seed)``, and a
    slab-wise draw gives the values of a draw in one piece."""
    import cima_b200.weights.random_init as R
    from helpers import TINY
    from reference_kernels import ReferenceKernels
    from cima_b200.engine import build_plan, load_model
    from cima_b200.weights import TensorSpec, random_tensor, random_tensors
    m = load_model(config=TINY["A"], seed=12, dtype="bfloat16", max_tokens=256, device="cpu", kernels=ReferenceKernels())
    want = random_tensors(build_plan(m.spec), 12)
    sd = m.state_dict()
    assert sorted(sd) == sorted(want)
    for n, t in want.items():
        assert torch.equal(sd[n].float(), t.float()), n
    spec = TensorSpec((1000, 77))
    whole = random_tensor(spec, 3, "x")
    slab = R._SLAB
    try:
        R._SLAB = 1600
        assert torch.equal(random_tensor(spec, 3, "x"), whole)
    finally:
        R._SLAB = slab
    g = torch.Generator()
    g.manual_seed(R._tensor_seed(3, "x"))
    assert torch.equal(torch.empty(1000, 77).normal_(0.0, 0.02, generator=g).to(torch.bfloat16), whole)
    with pytest.raises(ValueError, match="one of the two"):
        load_model(device="cpu", kernels=ReferenceKernels())
