"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it opens slots in the
model's cache, calls the model's step function and gives slots back, exactly as generation does.
Steps come as JSON lines on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

The requests of a step usually either all start or all go on by one token; any other mix is taken too (a
request may go on by several tokens), through the general rows-from-the-cache path of the step function.
For a step that wants logits, ``<out>/<step>.f32`` holds them as little-endian float32
[wanted, vocab] in the order of the entries and of their ``want``.  After every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict


from .batch import StepEntry
from .model import load_model


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines, out=sys.stdout, device="cuda:0",
           kernels=None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    model = load_model(model_dir, dtype=dtype, max_tokens=max_tokens, device=device, kernels=kernels)
    slots: Dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries = []
        new = [e["id"] for e in msg.get("entries", []) if e["id"] not in slots]
        if new:
            for rid, slot in zip(new, model.cache.open(len(new))):
                slots[rid] = slot
        for e in msg.get("entries", []):
            entries.append(StepEntry(slots[e["id"]], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = model.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
                model.check_device()                    # before the file appears: a reader never sees invalid logits
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
            elif device != "cpu":
                import torch
                torch.cuda.synchronize()
        ended = [rid for rid in msg.get("end", []) if rid in slots]
        if ended:
            model.cache.close([slots.pop(rid) for rid in ended])
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens, sys.stdin)


if __name__ == "__main__":
    sys.exit(main())
