"""Command line in the manner of the reference's ``cima`` (src/main.rs:19-70, :220-270):

    cima run <MODEL_DIR> [TOKEN_ID ...] [--prompts FILE] [--dtype D] [--max-seq N] [--PARAM VALUE]...
    cima run --random-shape NAME [--weights-seed S] [TOKEN_ID ...] ...
    cima bench <MODEL_DIR> [-n TOKENS] [--iters N] [--batch B] [--prompt-len P]
    cima profile <MODEL_DIR> | --random-shape NAME [--batch B] [--prompt-len P]
    cima random <OUT_DIR> --shape NAME | --config FILE [--seed S]
    cima show <MODEL_DIR>
    cima selftest
    cima help

``run`` takes the prompt as token ids (this library has no tokenizer): words or comma-separated
numbers on the command line, or one prompt per line in ``--prompts FILE``; several prompts run as
batches.  Every generation parameter goes through the option table (``--temp 0``, ``--top-k 40``,
``--max-tokens 64``, ``--stop 151645``, ``--ignore-eos true`` ...), as ``GenOptions::set`` does in the
reference.  The generated ids go to standard output, one line per prompt; a summary in the
reference's form ``[N prompt tok | M gen tok | ttft T ms | R tok/s]`` goes to standard error.
"""
from __future__ import annotations

import json
import sys
import time
from typing import List

from .sampling.options import GenOptions, OptionError, render_help

USAGE = """\
cima_b200 — generation library for the Qwen2 dense decoder on one B200

Usage:
  cima run <MODEL_DIR> [TOKEN_ID ...]   Generate from a prompt of token ids (--prompts FILE: one per line)
       --random-shape NAME                instead of MODEL_DIR: a known shape with random weights in memory
       --weights-seed S                   seed of those weights (default 0)
       --stream                           print every token as its step is read ("<prompt>:<token>" a line)
       --dtype bfloat16|float32           precision of the whole model (default bfloat16)
       --max-seq N                        positions the cache holds in all (default 8192)
       --PARAM VALUE                      generation parameters (see `cima run --help`)
  cima bench <MODEL_DIR> [-n TOKENS] [--iters N] [--batch B] [--prompt-len P]
                                        Greedy decode rate, stop tokens ignored, one discarded warm-up
  cima profile <MODEL_DIR> | --random-shape NAME [--batch B] [--prompt-len P]
                                        Every launch of a decode step and of a prompt step with its time inside the step
  cima random <OUT_DIR> --shape NAME | --config FILE [--seed S]
                                        Write a model folder with seeded random weights
  cima show <MODEL_DIR>                 Show the model's configuration and layers
  cima selftest                         A tiny random model: both precisions, twice, must agree
  cima help                             Show this help
"""


def _ids(words: List[str]) -> List[int]:
    out: List[int] = []
    for w in words:
        for part in w.replace(",", " ").split():
            try:
                out.append(int(part))
            except ValueError:
                raise SystemExit(f"'{part}' is not a token id: prompts are given as token ids")
    return out


def _flag(args: List[str], name: str, default=None):
    if name in args:
        i = args.index(name)
        if i + 1 >= len(args):
            raise SystemExit(f"{name} expects a value")
        v = args[i + 1]
        del args[i:i + 2]
        return v
    return default


def cmd_run(args: List[str]) -> int:
    if "--help" in args or "-h" in args:
        print("usage: cima run <MODEL_DIR> [TOKEN_ID ...] [--prompts FILE] [--dtype D] [--max-seq N] [--PARAM VALUE]...\n")
        print(render_help(), end="")
        return 0
    rest = list(args)
    shape = _flag(rest, "--random-shape")
    weights_seed = int(_flag(rest, "--weights-seed", "0"))
    model_dir = None
    if shape is None:
        if not rest or rest[0].startswith("--"):
            raise SystemExit("cima run: a model folder (or --random-shape NAME) is needed")
        model_dir = rest.pop(0)
    else:
        from .config.shapes import SHAPES
        if shape not in SHAPES:
            raise SystemExit(f"cima run: unknown shape '{shape}' (known: {', '.join(sorted(SHAPES))})")
    dtype = _flag(rest, "--dtype", "bfloat16")
    max_seq = int(_flag(rest, "--max-seq", "8192"))
    prompts_file = _flag(rest, "--prompts")
    stream = "--stream" in rest
    if stream:
        rest.remove("--stream")
    opts = GenOptions()
    words: List[str] = []
    i = 0
    while i < len(rest):
        if rest[i].startswith("--") and i + 1 < len(rest):
            try:
                opts = opts.set(rest[i], rest[i + 1])
            except OptionError as e:
                raise SystemExit(f"cima run: {e}")
            i += 2
        else:
            words.append(rest[i])
            i += 1
    prompts: List[List[int]] = []
    if prompts_file:
        with open(prompts_file) as f:
            prompts = [_ids([line]) for line in f if line.strip()]
    if words:
        prompts.append(_ids(words))
    if not prompts:
        raise SystemExit("cima run: no prompt (token ids on the command line or --prompts FILE)")
    import cima_b200
    if model_dir is not None:
        print(f"loading {model_dir} …", file=sys.stderr)
        lm = cima_b200.load(model_dir, dtype=dtype, max_tokens=max_seq)
    else:
        print(f"random weights of shape {shape}, seed {weights_seed} …", file=sys.stderr)
        lm = cima_b200.load(config=SHAPES[shape], seed=weights_seed, dtype=dtype, max_tokens=max_seq)
    t0 = time.perf_counter()
    on_token = (lambda i, t: print(f"{i}:{t}", flush=True)) if stream else None
    results = lm.generate(prompts, opts, on_token=on_token)
    total = time.perf_counter() - t0
    if not stream:
        for r in results:
            print(" ".join(str(t) for t in r.tokens))
    s = lm.stats
    rate = s.gen_tokens / total if total > 0 else 0.0
    print(f"[{s.prompt_tokens} prompt tok | {s.gen_tokens} gen tok | ttft {s.prefill_s * 1e3:.0f} ms | {rate:.1f} tok/s]",
          file=sys.stderr)
    return 0


def cmd_bench(args: List[str]) -> int:
    if not args:
        raise SystemExit("cima bench: a model folder is needed")
    model_dir, rest = args[0], list(args[1:])
    n = int(_flag(rest, "-n", "128"))
    iters = int(_flag(rest, "--iters", "3"))
    batch = int(_flag(rest, "--batch", "1"))
    plen = int(_flag(rest, "--prompt-len", "128"))
    dtype = _flag(rest, "--dtype", "bfloat16")
    import numpy as np
    import cima_b200
    lm = cima_b200.load(model_dir, dtype=dtype, max_tokens=batch * (plen + n + 64), max_batch=batch)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, lm.spec.vocab, size=plen).tolist() for _ in range(batch)]
    o = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=n, ignore_eos=True)
    lm.generate(prompts, o)                                  # discarded warm-up
    rates = []
    for _ in range(iters):
        lm.generate(prompts, o)
        s = lm.stats
        rates.append(batch * s.decode_steps / s.decode_s)
    rates.sort()
    print(json.dumps({"model": model_dir, "batch": batch, "prompt_tokens": plen, "gen_tokens": n, "iters": iters,
                      "decode_tok_per_s_p50": rates[len(rates) // 2], "decode_tok_per_s_min": rates[0],
                      "ttft_ms": lm.stats.prefill_s * 1e3}))
    return 0


def cmd_profile(args: List[str]) -> int:
    """Where a step's time goes, launch by launch, without a profiler (the reference's ``cima profile`` prints
    microseconds per launch, launches per token and the weight-streaming floor, src/selftest.rs:1201-1331)."""
    rest = list(args)
    shape = _flag(rest, "--random-shape")
    batch = int(_flag(rest, "--batch", "1"))
    plen = int(_flag(rest, "--prompt-len", "128"))
    dtype = _flag(rest, "--dtype", "bfloat16")
    hbm = float(_flag(rest, "--hbm-gbs", "6650"))
    tflops = float(_flag(rest, "--tflops", "1590"))
    if shape is None and not rest:
        raise SystemExit("cima profile: a model folder (or --random-shape NAME) is needed")
    import numpy as np
    import cima_b200
    from .engine.profile import profile_decode, profile_prompt, table
    kw = dict(dtype=dtype, max_tokens=batch * (plen + 1024), max_batch=batch, pipeline=False)
    if shape is not None:
        from .config.shapes import SHAPES
        if shape not in SHAPES:
            raise SystemExit(f"cima profile: unknown shape '{shape}' (known: {', '.join(sorted(SHAPES))})")
        lm = cima_b200.load(config=SHAPES[shape], seed=0, draw="device", **kw)
    else:
        lm = cima_b200.load(rest[0], **kw)
    st = lm.stepper
    if not st.use_graphs:
        raise SystemExit("cima profile: this model's steps cannot be recorded (a part is not fit for it, or no GPU)")
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, lm.spec.vocab, size=plen).tolist() for _ in range(batch)]
    o = [GenOptions(temperature=0.0, repeat_penalty=1.0, ignore_eos=True)] * batch
    slots = st.open(batch)
    try:
        first = st.prefill(slots, prompts, o)
        rows = profile_decode(st, slots, first, o)
    finally:
        st.close(slots)
    print(f"decode step, batch {batch}, context {plen} (peaks given: {hbm:.0f} GB/s, {tflops:.0f} TFLOP/s):")
    print(table(rows, hbm, tflops, tokens=batch))
    print(f"\nprompt step, one prompt of {plen} tokens:")
    print(table(profile_prompt(lm.model, [plen]), hbm, tflops))
    return 0


def cmd_random(args: List[str]) -> int:
    if not args:
        raise SystemExit("cima random: an output folder is needed")
    out, rest = args[0], list(args[1:])
    shape, cfg_file, seed = _flag(rest, "--shape"), _flag(rest, "--config"), int(_flag(rest, "--seed", "0"))
    from .config.shapes import SHAPES
    if cfg_file:
        with open(cfg_file) as f:
            raw = json.load(f)
    elif shape:
        if shape not in SHAPES:
            raise SystemExit(f"cima random: unknown shape '{shape}' (known: {', '.join(sorted(SHAPES))})")
        raw = SHAPES[shape]
    else:
        raise SystemExit("cima random: --shape NAME or --config FILE is needed")
    import cima_b200
    cima_b200.write_random_model(out, raw, seed=seed)
    print(f"wrote {out} (seed {seed})")
    return 0


def cmd_show(args: List[str]) -> int:
    if not args:
        raise SystemExit("cima show: a model folder is needed")
    import cima_b200
    from .engine import build_plan
    raw = cima_b200.read_config_json(args[0])
    entry = cima_b200.lookup_architecture(raw)
    spec = entry.spec(entry.parse(raw))
    plan = build_plan(spec)
    params = sum(int(__import__("math").prod(s.shape)) for s in plan.values())
    print(spec.describe())
    print(f"{len(plan)} tensors, {params / 1e6:.2f} M parameters")
    return 0


def cmd_selftest(args: List[str]) -> int:
    """A tiny model with random weights in memory, on the GPU: the same prompts generate the same tokens twice
    (greedy and sampled, with graphs and run-ahead), in 32-bit and in bfloat16; a step's bfloat16 logits stay
    within rounding of the 32-bit ones; the cache ends empty.  (The reference's selftest drives its real
    generation path over stand-in weights the same way, src/selftest.rs:184-337.)"""
    import cima_b200
    from .config.shapes import SHAPES
    from .engine import StepEntry
    prompts = [[5, 17, 3, 200, 411, 9, 1], [42], [7, 7, 7, 300, 2, 1, 0, 99, 100, 101, 511, 250, 3]]
    chains = (dict(temperature=0.0, repeat_penalty=1.0), dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=3))
    logits = {}
    for dtype in ("float32", "bfloat16"):
        lm = cima_b200.load(config=SHAPES["tiny-a"], seed=7, dtype=dtype, max_tokens=512, verbose=False)
        for opts in chains:
            first = [r.tokens for r in lm.generate(prompts, max_tokens=12, **opts)]
            again = [r.tokens for r in lm.generate(prompts, max_tokens=12, **opts)]
            if first != again or any(len(t) != 12 for t in first):
                print(f"selftest FAILED ({dtype}, {opts}): {first} then {again}", file=sys.stderr)
                return 1
        (slot,) = lm.model.cache.open(1)
        try:
            logits[dtype] = lm.step([StepEntry(slot, prompts[2], list(range(len(prompts[2]))))]).float().cpu()
        finally:
            lm.model.cache.close([slot])
        lm.model.cache.check()
        if lm.model.cache.slots.held:
            print(f"selftest FAILED ({dtype}): {lm.model.cache.slots.held} slots still held", file=sys.stderr)
            return 1
        print(f"selftest {dtype}: ok ({lm.model.rt.kernels.launches} kernel launches)")
    worst = (logits["float32"] - logits["bfloat16"]).abs().max().item()
    if not worst <= 2e-2:
        print(f"selftest FAILED: bfloat16 logits are {worst:.3g} from the 32-bit ones", file=sys.stderr)
        return 1
    print(f"selftest: bfloat16 within {worst:.2g} of 32-bit")
    return 0


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args or args[0] in ("help", "--help", "-h"):
        print(USAGE, end="")
        return 0
    cmd, rest = args[0], args[1:]
    if cmd == "run":
        return cmd_run(rest)
    if cmd == "bench":
        return cmd_bench(rest)
    if cmd == "profile":
        return cmd_profile(rest)
    if cmd == "random":
        return cmd_random(rest)
    if cmd == "show":
        return cmd_show(rest)
    if cmd == "selftest":
        return cmd_selftest(rest)
    print(USAGE, end="")
    print(f"unknown command '{cmd}'", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
