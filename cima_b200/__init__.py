"""cima_b200: a small generation library for one GPU (NVIDIA B200, sm_100a).

    import cima_b200
    lm = cima_b200.load("model_dir", dtype="bfloat16", max_tokens=8192)
    results = lm.generate([[1, 2, 3], [4, 5]], temperature=0, max_tokens=32)
    lm = cima_b200.load(config={...config.json keys...}, seed=0)     # random weights, no folder
    weights = lm.state_dict()                                         # tensors by their checkpoint names

A model folder holds ``config.json`` and ``model.safetensors``; the model class is chosen by
config.json through the architecture registry.  ``cima_b200.write_random_model`` makes such a folder
from a configuration and a seed.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from .config import (ArchitectureEntry, ConfigError, Qwen2Config, lookup_architecture, read_config_json,
                     register_architecture, registered_architectures)
from .sampling import GenOptions, OptionError

register_architecture(ArchitectureEntry(name=Qwen2Config.ARCHITECTURE, model_type="qwen2",
                                        parse=Qwen2Config.from_dict, spec=Qwen2Config.model_spec))

__version__ = "0.1.0"


class LM:
    """A loaded model with its cache, stepper and generation loop."""

    def __init__(self, model, eos_ids: Sequence[int] = (), max_batch: int = 64, pipeline: bool = True, retain: int = 0,
                 use_graphs: bool = True):
        from .engine import GenerationLoop, ModelStepper
        self.model = model
        self.stepper = ModelStepper(model, max_batch=max_batch, use_graphs=use_graphs, pipeline=pipeline, retain=retain)
        self.loop = GenerationLoop(self.stepper, eos_ids)

    def state_dict(self):
        """The model's tensors by their checkpoint names, as kept on the device (``Model.state_dict``)."""
        return self.model.state_dict()

    @property
    def spec(self):
        return self.model.spec

    @property
    def config(self):
        """The typed configuration that config.json was parsed into."""
        return self.model.config

    def step(self, entries):
        """The model's step function (``cima_b200.engine.StepEntry`` per sequence): float32 logits at the wanted
        places.  The caller opens and closes the slots (``lm.model.cache``)."""
        return self.model.step(entries)

    def generate(self, prompts: Sequence[Sequence[int]], options: Union[GenOptions, Sequence[GenOptions], None] = None,
                 on_token=None, **named):
        """Token ids in, ``GenResult`` per prompt out.  Options by the reference's names
        (temperature, top_k, top_p, repeat_penalty, seed, max_tokens, stop, ignore_eos), either as a
        ``GenOptions`` (one for all prompts or one per prompt) or as keyword arguments.  ``on_token(i, token)`` is
        called for every token of prompt ``i`` as soon as its step is read."""
        if named:
            if options is not None and not isinstance(options, GenOptions):
                raise ValueError("keyword options go with at most one GenOptions")
            o = options or GenOptions()
            for k, v in named.items():
                if k == "stop" and not isinstance(v, (int, str)):
                    for s in v:
                        o = o.set("stop", s)
                else:
                    o = o.set(k, v)
            options = o
        return self.loop.generate(prompts, options, on_token=on_token)

    @property
    def stats(self):
        return self.loop.stats


def eos_ids_of(folder: str) -> List[int]:
    """Stop ids a model folder declares (generation_config.json, then config.json), as the reference
    gathers them (src/tokenizer.rs:704-749)."""
    import json, os
    out: List[int] = []
    for name in ("generation_config.json", "config.json"):
        p = os.path.join(folder, name)
        if os.path.exists(p):
            try:
                with open(p) as f:
                    v = json.load(f).get("eos_token_id")
            except (OSError, ValueError):
                continue
            for t in (v if isinstance(v, list) else [v]):
                if isinstance(t, int) and not isinstance(t, bool) and t not in out:
                    out.append(t)
    return out


def _eos_ids_of_config(raw) -> List[int]:
    v = raw.get("eos_token_id") if isinstance(raw, dict) else None
    return [t for t in (v if isinstance(v, list) else [v]) if isinstance(t, int) and not isinstance(t, bool)]


def load(folder: Optional[str] = None, dtype: str = "bfloat16", max_tokens: int = 8192, max_seqs: Optional[int] = None,
         max_batch: int = 64, device: str = "cuda:0", verbose: bool = True, pipeline: bool = True,
         retain: int = 0, use_graphs: bool = True, config=None, seed: int = 0, draw: str = "cpu") -> LM:
    """A model from ``folder`` (config.json, model.safetensors), or from ``config`` (a config.json dict or a typed
    configuration) and ``seed`` with random weights in memory (``draw``: see ``engine.load_model``).
    ``pipeline``: queue the next decode step before the host has read the current one's tokens
    (the tokens are fed forward on the device).  ``retain``: how many finished sequences stay in the cache for
    later prompts that begin with the same tokens (the next turn of a conversation runs only what is new; the
    reference keeps its one sequence so, src/models/mod.rs:1022-1058); they give way when a batch needs the room.
    ``use_graphs``: record decode steps as CUDA graphs (a model with a part that is unfit for it decodes step by
    step whatever is asked)."""
    from .engine import load_model
    model = load_model(folder, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs, device=device, verbose=verbose,
                       config=config, seed=seed, draw=draw)
    if folder is not None:
        eos = eos_ids_of(folder)
    else:
        eos = _eos_ids_of_config(config.to_dict() if hasattr(config, "to_dict") else config)
    return LM(model, eos, max_batch=max_batch, pipeline=pipeline, retain=retain, use_graphs=use_graphs)


def write_random_model(folder: str, config: Union[dict, Qwen2Config], seed: int = 0) -> None:
    """A model folder (config.json, model.safetensors in bfloat16) from a configuration and a seed."""
    from .engine import build_plan
    from .weights import write_random_model as _write
    raw = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    entry = lookup_architecture(raw)
    typed = entry.parse(raw)
    out = typed.to_dict() if hasattr(typed, "to_dict") else raw
    for k, v in raw.items():
        out.setdefault(k, v)
    _write(folder, out, build_plan(entry.spec(typed)), seed)


__all__ = ["LM", "load", "write_random_model", "eos_ids_of", "GenOptions", "OptionError", "ConfigError",
           "Qwen2Config", "register_architecture", "registered_architectures", "lookup_architecture",
           "read_config_json", "ArchitectureEntry"]
