#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen2.5-7B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--prompt 2048] [--layers L]
    python bench.py --impl reference ...      # the reference arm (unavailable here: a Rust crate)

One JSON line on standard output.  ``value`` is decoded tokens per second of a batch of ``--batch``
sequences after ``--prompt``-token prompts, timed on the device over exactly K decode steps (tokens
fed forward on the device).  ``e2e`` is the same through ``cima_b200.LM.generate``: host token ids
in, host token ids out, one host-to-device copy of the step's inputs and one device-to-host read of
its tokens per step.  ``prefill`` is one 2,048-token prompt; ``points`` are decode at batch 1 and 64;
``roofline`` is the decode step's necessary bytes (every weight once, the live requests' keys and
values) over its time, against the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=28, hidden_size=3584,
                 num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
                 vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                 use_sliding_window=False, max_position_embeddings=32768)
SLOT_TOKENS = 4096          # context per sequence slot of the benchmark configuration
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "juliog922/cima is a Rust crate (Cargo.toml, no Python packaging); pip cannot install it and "
                      "this image has no cargo/rustc to build it"}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration's 28 (named in config)")
    ap.add_argument("--shape", default="qwen2.5-7b", help="another shape of cima_b200.config.shapes.SHAPES (the metric is "
                    "defined on the default, Qwen2.5-7B)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--per-kernel", action="store_true", help="instead of the metric line: every launch of one decode step "
                    "(--batch) and of one prompt step (--prompt tokens) with its time inside the step, bytes and flops "
                    "over time against the measured peaks; use few layers (--layers 2)")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py measures one GPU only (this library does no multi-GPU work); --gpus {a.gpus} is not run")
        return 2
    a.warmup = max(a.warmup, 3)

    import numpy as np
    import torch
    import cima_b200
    from cima_b200.engine import StepEntry
    from cima_b200.sampling import GenOptions

    pk = peaks()
    raw = dict(QWEN25_7B)
    if a.shape != "qwen2.5-7b":
        from cima_b200.config.shapes import SHAPES
        raw = dict(SHAPES[a.shape])
    layers_full = raw["num_hidden_layers"]
    if a.layers:
        raw["num_hidden_layers"] = a.layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    max_batch = max(a.batch, 1 if a.no_points else 64)
    per_seq = a.prompt + a.steps + a.warmup + 64
    # Random weights drawn on the device, tensor by tensor (seeded by name, as the random-weights mode); a cache with
    # room for the batches of the decode runs and for the one 2,048-token prompt of the prefill figure.
    # e2e below is measured with every step's input tokens copied from pinned host memory (pipeline off);
    # "pipelined" is the default mode of the library, where the next step is queued before the host has
    # read the current one's tokens and its inputs never leave the device
    lm = cima_b200.load(config=raw, seed=0, draw="device", dtype="bfloat16", device=dev, max_seqs=max_batch,
                        max_tokens=max(max_batch * (-(-per_seq // 64) * 64), 2048 + 64), max_batch=max_batch,
                        pipeline=False, verbose=True)
    model, cfg = lm.model, lm.config
    K = model.rt.kernels
    st = lm.stepper
    greedy = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=a.steps, ignore_eos=True)
    rng = np.random.default_rng(0)
    V = cfg.vocab_size
    kv_bytes_per_token = sum(g.storage.element_size() * len(g.layers) * 2 * g.request.n_kv_heads * g.request.head_dim
                             for g in model.cache.groups)
    weight_bytes = model.weight_bytes()

    if a.per_kernel:
        from cima_b200.engine.profile import profile_decode, profile_prompt, table
        prompts = [rng.integers(0, V, size=a.prompt).tolist() for _ in range(a.batch)]
        slots = st.open(a.batch)
        try:
            opts = [greedy] * a.batch
            first = st.prefill(slots, prompts, opts)
            rows = profile_decode(st, slots, first, opts)
        finally:
            st.close(slots)
        print(f"decode step, batch {a.batch}, context {a.prompt}, {cfg.num_hidden_layers} of {layers_full} layers "
              f"(time of each launch inside the recorded step; peaks {pk['source']}):")
        print(table(rows, pk["hbm_gbs"], pk["bf16_tflops"], tokens=a.batch))
        rows = profile_prompt(model, [a.prompt])
        print(f"\nprompt step, one prompt of {a.prompt} tokens:")
        print(table(rows, pk["hbm_gbs"], pk["bf16_tflops"]))
        return 0

    def timed(fn, reps=1):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3

    def decode_run(batch, steps, warmup):
        """(seconds for `steps` decode steps on the device, launches per step, mean context)."""
        prompts = [rng.integers(0, V, size=a.prompt).tolist() for _ in range(batch)]
        slots = st.open(batch)
        try:
            opts = [greedy] * batch
            first = st.prefill(slots, prompts, opts)          # the model runs a step of many rows in parts of 16,384
            last = st.decode(slots, first, opts)                  # arms and captures the graph
            st.decode_on_device(slots, last, opts, warmup, reach=warmup + steps)
            before = K.launches
            secs = timed(lambda: st.decode_on_device(slots, None, opts, steps))
            ctx = a.prompt + 1 + warmup + steps / 2.0
            assert K.launches == before                           # everything ran from the graph
            return secs, st.recorded_launches(batch), ctx
        finally:
            st.close(slots)

    out = {}
    with ClockSampler() as clocks:
        secs, lps, ctx = decode_run(a.batch, a.steps, a.warmup)
    clk = clocks.summary()
    value = a.batch * a.steps / secs
    step_bytes = weight_bytes + a.batch * ctx * kv_bytes_per_token
    achieved = step_bytes / (secs / a.steps) / 1e9

    # prefill of one 2,048-token prompt
    T = 2048
    prompt = rng.integers(0, V, size=T).tolist()
    tok = torch.empty(1, dtype=torch.int32, device=dev)

    def prefill_once():
        (slot,) = model.cache.open(1)
        try:
            logits = model.step([StepEntry(slot, prompt, [T - 1])])
            K.argmax(logits, tok)
        finally:
            model.cache.close([slot])
    for _ in range(3):
        prefill_once()
    reps = 3
    psecs = timed(prefill_once, reps) / reps
    lin_params = (weight_bytes - 0) / 2                          # bf16 bytes -> parameters of the matrices (norms negligible)
    L, nh, hd = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim
    flops = 2.0 * T * (lin_params - V * cfg.hidden_size) + 2.0 * V * cfg.hidden_size + L * 2.0 * nh * T * T * hd
    # frac: of the burst figure of the library product (a kernel alone); frac_sustained: of what the same product
    # holds back to back under the power cap, which is how the layers of a prefill run
    prefill = {"value": T / psecs, "tokens": T, "ms": psecs * 1e3, "frac": flops / psecs / (pk["bf16_tflops"] * 1e12),
               "frac_sustained": flops / psecs / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12)}

    points = {}
    if not a.no_points:
        for b in (1, 64):
            s, _, _ = decode_run(b, a.steps, a.warmup)
            points[f"decode_b{b}"] = b * a.steps / s

    e2e = None
    if not a.no_e2e:
        prompts = [rng.integers(0, V, size=a.prompt).tolist() for _ in range(a.batch)]
        lm.generate(prompts, GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=a.warmup, ignore_eos=True))
        # bytes that cross per decode step: counted over the decode steps of the timed call (the stepper
        # counts what it copies; the prefill's share is taken out by a second call that only prefills)
        st.h2d_bytes = st.d2h_bytes = 0
        lm.generate(prompts, GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=1, ignore_eos=True))
        pre_h2d, pre_d2h = st.h2d_bytes, st.d2h_bytes
        st.h2d_bytes = st.d2h_bytes = 0
        res = lm.generate(prompts, greedy)
        stats = lm.stats
        assert all(len(r.tokens) == a.steps for r in res)
        # the first token of each sequence comes from the prefill; the decode steps made the rest
        e2e = {"value": a.batch * stats.decode_steps / stats.decode_s, "unit": "tokens/s",
               "h2d_bytes_per_step": (st.h2d_bytes - pre_h2d) / max(stats.decode_steps, 1),
               "d2h_bytes_per_step": (st.d2h_bytes - pre_d2h) / max(stats.decode_steps, 1)}
        # The same call with 48 more tokens, its last K steps timed on the host as their tokens arrive: after the
        # 16k-token prefill has run at the power cap, the SM clock stays near 1.3 GHz for some 25 decode steps (a
        # step then takes 3.8 ms instead of 3.15), which is most of what this dictionary's "value" sees at a small K.
        stamps = []
        lm.generate(prompts, GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=a.steps + 48, ignore_eos=True),
                    on_token=lambda i, t: stamps.append(time.perf_counter()) if i == 0 else None)
        e2e["after_48_steps"] = a.batch * a.steps / (stamps[-1] - stamps[-1 - a.steps])
        st.pipeline = True
        lm.generate(prompts, GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=a.warmup, ignore_eos=True))
        res = lm.generate(prompts, greedy)
        e2e["pipelined"] = a.batch * lm.stats.decode_steps / lm.stats.decode_s
        st.pipeline = False

    # the first token of one short prompt through the entry point (host ids in, the token out), wall clock
    first_token = {}
    if not a.no_e2e:
        one = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=1, ignore_eos=True)
        for n in (16, 128, 300):
            p = rng.integers(0, V, size=n).tolist()
            for _ in range(3):
                lm.generate([p], one)
            ts = []
            for _ in range(7):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                lm.generate([p], one)
                ts.append(time.perf_counter() - t0)
            first_token[f"prompt_{n}"] = statistics.median(ts) * 1e3

    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B bf16)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": secs / a.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 0, uniform random token ids",
        "config": {"model": "Qwen2.5-7B shape" if a.shape == "qwen2.5-7b" else a.shape + " shape", "global_batch": a.batch, "seq_len": SLOT_TOKENS, "parallelism": "single GPU",
                   "prompt_tokens": a.prompt, "layers": cfg.num_hidden_layers, "layers_of_config": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "tied_head": cfg.tie_word_embeddings,
                   "kv_dtype": "bf16", "sampling": "greedy on device", "l2": "inputs (weights) exceed L2"},
        "e2e": e2e, "gpu_launches": lps * a.steps, "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]},
        "points": points, "first_token_ms": first_token, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
