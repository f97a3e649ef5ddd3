"""Generation options under the reference's names, aliases, ranges and defaults.

One table drives the command line, the Python entry point and the help text, as
``GenOptions::TABLE`` / ``GenOptions::set`` do (src/traits.rs:389-570): temperature (alias temp;
0..=10, 0 = greedy; default 0.8), top_k (0 = unlimited; 40), top_p (0..=1; 0.9), repeat_penalty
(> 0, 1.0 = off; 1.1), seed (u64; 0xC0FFEE), max_tokens (aliases num_predict, n; 1024), stop
(repeatable; the reference stops on strings, this library works on token ids and stops on ids),
ignore_eos (false).  A failed ``set`` leaves the options untouched.
"""
from __future__ import annotations

from dataclasses import dataclass, replace



class OptionError(ValueError):
    pass


OPTION_TABLE = [
    # name, aliases, range, default, description
    ("temperature", "temp", "0..=10 (0 = greedy)", "0.8", "softmax temperature; 0 selects greedy decoding"),
    ("top_k", "", "0 = unlimited", "40", "keep only the k most likely tokens before top_p"),
    ("top_p", "", "0..=1", "0.9", "nucleus truncation over the top_k survivors"),
    ("repeat_penalty", "", "> 0 (1.0 = off)", "1.1", "penalize tokens seen in the last 64 (once per occurrence, sign-aware)"),
    ("seed", "", "u64", str(0xC0FFEE), "rng seed; same seed + options reproduces a sampled run"),
    ("max_tokens", "num_predict, n", "u32", "1024", "generation cap (a stop token may end earlier)"),
    ("stop", "", "token id, repeatable", "none", "stop token id; generation halts before emitting it"),
    ("ignore_eos", "", "true|false", "false", "keep generating past stop tokens (benchmarks)"),
]


@dataclass(frozen=True)
class GenOptions:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    repeat_penalty: float = 1.1
    seed: int = 0xC0FFEE
    max_tokens: int = 1024
    stop: tuple = ()
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        """The reference's test for its argmax-only path (src/models/mod.rs:1083-1085)."""
        return (self.temperature <= 0.0 or self.top_k == 1) and self.repeat_penalty == 1.0

    def set(self, key: str, value) -> "GenOptions":
        """A copy with one option set from its command-line or JSON spelling."""
        k = str(key).lstrip("-").replace("-", "_")

        def num(cast):
            try:
                return cast(value)
            except (TypeError, ValueError):
                raise OptionError(f"'{k}' expects a number, got '{value}'") from None

        if k in ("temp", "temperature"):
            v = num(float)
            if not (0.0 <= v <= 10.0):
                raise OptionError(f"temperature out of range [0,10]: {v}")
            return replace(self, temperature=v)
        if k == "top_p":
            v = num(float)
            if not (0.0 <= v <= 1.0):
                raise OptionError(f"top_p out of range [0,1]: {v}")
            return replace(self, top_p=v)
        if k == "top_k":
            v = num(int)
            if v < 0:
                raise OptionError(f"top_k must not be negative: {v}")
            return replace(self, top_k=v)
        if k in ("max_tokens", "num_predict", "n"):
            v = num(int)
            if v < 0:
                raise OptionError(f"max_tokens must not be negative: {v}")
            return replace(self, max_tokens=v)
        if k == "seed":
            v = num(int)
            if not (0 <= v < 1 << 64):
                raise OptionError(f"seed must fit 64 unsigned bits: {v}")
            return replace(self, seed=v)
        if k == "repeat_penalty":
            v = num(float)
            if v <= 0.0:
                raise OptionError(f"repeat_penalty must be > 0: {v}")
            return replace(self, repeat_penalty=v)
        if k == "stop":
            v = num(int)
            return replace(self, stop=tuple(self.stop) + (v,))
        if k == "ignore_eos":
            if isinstance(value, bool):
                return replace(self, ignore_eos=value)
            if str(value).lower() in ("true", "false"):
                return replace(self, ignore_eos=str(value).lower() == "true")
            raise OptionError("ignore_eos expects true/false")
        raise OptionError(f"unknown option '{key}'")


def render_help() -> str:
    out = ["generation parameters (--PARAM VALUE):"]
    for name, aliases, rng, default, desc in OPTION_TABLE:
        alias = f" (alias: {aliases})" if aliases else ""
        out.append(f"  --{name.replace('_', '-'):<16}{alias}")
        out.append(f"      {desc}  [range: {rng}; default: {default}]")
    return "\n".join(out) + "\n"
