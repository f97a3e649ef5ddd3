"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Parity with the reference's ``ModelConfig::load`` (src/models/transformer.rs:81-277):
required keys and the error that names the missing key (:69-77), defaults of the
optional keys (:162-163, :184, :264-267), the geometry checks (:170-182), and
q/k/v bias following from ``model_type`` starting with "qwen2" (:257).

Beyond the reference, which does not read them (its window is hard-wired 0,
src/models/transformer.rs:1184-1199): ``use_sliding_window``, ``sliding_window``
and ``max_window_layers`` select a windowed attention for the layers from
``max_window_layers`` on, or for the layers that ``layer_types`` calls
"sliding_attention" where that list is given; ``rope_parameters`` (the newer
spelling: ``{"rope_theta": ..., "rope_type": "default"}``) gives the base when
``rope_theta`` is absent; ``hidden_act`` other than "silu" and a rotary
scaling of any type but "default" are refused rather than ignored.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec)


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


def _req_int(cfg: Dict[str, Any], key: str) -> int:
    v = cfg.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: required integer attribute '{key}' is missing or not a number")
    return int(v)


def _opt_int(cfg: Dict[str, Any], key: str, default: int) -> int:
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: attribute '{key}' is not an integer: {v!r}")
    return int(v)


def _opt_float(cfg: Dict[str, Any], key: str, default: float) -> float:
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: attribute '{key}' is not a number: {v!r}")
    return float(v)


def _opt_bool(cfg: Dict[str, Any], key: str, default: bool) -> bool:
    v = cfg.get(key)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: attribute '{key}' is not true/false: {v!r}")
    return v


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    use_sliding_window: bool
    sliding_window: int
    max_window_layers: int
    hidden_act: str = "silu"
    model_type: str = "qwen2"
    layer_types: Optional[Tuple[str, ...]] = None      # per layer "full_attention" | "sliding_attention", if given

    ARCHITECTURE = "Qwen2ForCausalLM"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "Qwen2Config":
        model_type = cfg.get("model_type")
        if not isinstance(model_type, str):
            raise ConfigError("config.json: 'model_type' missing — cannot select an architecture")
        if model_type != "qwen2":
            raise ConfigError(f"config.json: model_type '{model_type}' is not 'qwen2'")
        hidden = _req_int(cfg, "hidden_size")
        layers = _req_int(cfg, "num_hidden_layers")
        heads = _req_int(cfg, "num_attention_heads")
        inter = _req_int(cfg, "intermediate_size")
        vocab = _req_int(cfg, "vocab_size")
        kv_heads = _opt_int(cfg, "num_key_value_heads", heads)
        head_dim = _opt_int(cfg, "head_dim", hidden // max(heads, 1))
        if min(hidden, layers, inter, vocab) <= 0:
            raise ConfigError(f"config.json: sizes must be positive (hidden_size={hidden}, "
                              f"num_hidden_layers={layers}, intermediate_size={inter}, vocab_size={vocab})")
        if heads <= 0 or kv_heads <= 0 or head_dim <= 0:
            raise ConfigError(f"config.json: zero attention geometry (num_attention_heads={heads}, "
                              f"num_key_value_heads={kv_heads}, head_dim={head_dim})")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) is not a multiple of "
                              f"num_key_value_heads ({kv_heads}) — invalid GQA geometry")
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({head_dim}) must be even for rotary embeddings")
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        for key in ("rope_scaling", "rope_parameters"):
            rope = cfg.get(key)
            if rope is None:
                continue
            if not isinstance(rope, dict):
                raise ConfigError(f"config.json: attribute '{key}' is not an object: {rope!r}")
            kind = rope.get("rope_type", rope.get("type", "default"))
            if kind != "default":
                raise ConfigError(f"config.json: {key} asks for '{kind}' rotary embeddings; only 'default' is supported")
        eps = _opt_float(cfg, "rms_norm_eps", 1e-6)
        if cfg.get("rope_theta") is None and isinstance(cfg.get("rope_parameters"), dict):
            theta = _opt_float(cfg["rope_parameters"], "rope_theta", 10000.0)
        else:
            theta = _opt_float(cfg, "rope_theta", 10000.0)
        if eps <= 0 or theta <= 0:
            raise ConfigError(f"config.json: rms_norm_eps ({eps}) and rope_theta ({theta}) must be positive")
        max_pos = _opt_int(cfg, "max_position_embeddings", 4096)
        if max_pos <= 0:
            raise ConfigError(f"config.json: max_position_embeddings ({max_pos}) must be positive")
        use_win = _opt_bool(cfg, "use_sliding_window", False)
        window = _opt_int(cfg, "sliding_window", 0) if cfg.get("sliding_window") is not None else 0
        max_win_layers = _opt_int(cfg, "max_window_layers", layers)
        if use_win and window <= 0:
            raise ConfigError("config.json: use_sliding_window is true but sliding_window is missing or not positive")
        if max_win_layers < 0:
            raise ConfigError(f"config.json: max_window_layers ({max_win_layers}) is negative")
        layer_types = cfg.get("layer_types")
        if layer_types is not None:
            kinds = ("full_attention", "sliding_attention")
            if not isinstance(layer_types, list) or len(layer_types) != layers or any(t not in kinds for t in layer_types):
                raise ConfigError(f"config.json: layer_types must name one of {kinds} for each of the {layers} layers")
            if "sliding_attention" in layer_types and window <= 0:
                raise ConfigError("config.json: layer_types has sliding_attention but sliding_window is missing or not positive")
            layer_types = tuple(layer_types)
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                   num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim,
                   max_position_embeddings=max_pos, rms_norm_eps=eps, rope_theta=theta,
                   tie_word_embeddings=_opt_bool(cfg, "tie_word_embeddings", False),
                   use_sliding_window=use_win, sliding_window=window,
                   max_window_layers=max_win_layers, hidden_act=act, model_type=model_type,
                   layer_types=layer_types)

    @classmethod
    def load(cls, folder: str) -> "Qwen2Config":
        path = os.path.join(folder, "config.json")
        try:
            with open(path) as f:
                raw = json.load(f)
        except OSError as e:
            raise ConfigError(f"cannot read {path}: {e}") from e
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from e
        if not isinstance(raw, dict):
            raise ConfigError(f"{path} does not hold a JSON object")
        return cls.from_dict(raw)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        if self.layer_types is None:
            del d["layer_types"]
        else:
            d["layer_types"] = list(self.layer_types)
        d["architectures"] = [self.ARCHITECTURE]
        d["torch_dtype"] = "bfloat16"
        return d

    # ------------------------------------------------------------------ layers
    def layer_window(self, layer: int) -> int:
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else 0
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    def model_spec(self) -> ModelSpec:
        qd = self.num_attention_heads * self.head_dim
        position = PositionSpec(kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
                                theta=self.rope_theta)
        names = {
            "q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj",
            "o": "self_attn.o_proj", "gate": "mlp.gate_proj", "up": "mlp.up_proj",
            "down": "mlp.down_proj", "mixer_norm": "input_layernorm",
            "ffn_norm": "post_attention_layernorm",
        }
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = MixerSpec(kind="attention", hidden=self.hidden_size,
                              n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
                              head_dim=self.head_dim, qkv_bias=True, out_bias=False,
                              window=self.layer_window(i), scale=1.0 / math.sqrt(self.head_dim),
                              position=position)
            ffn = FeedForwardSpec(kind="gated_mlp", hidden=self.hidden_size,
                                  intermediate=self.intermediate_size, activation=self.hidden_act)
            norm = NormSpec(kind="rmsnorm", size=self.hidden_size, eps=self.rms_norm_eps)
            layers.append(BlockSpec(kind="prenorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    ffn_norm=norm, prefix=f"model.layers.{i}.", names=names))
        assert qd > 0
        return ModelSpec(architecture=self.ARCHITECTURE, vocab=self.vocab_size, hidden=self.hidden_size,
                         max_position=self.max_position_embeddings, layers=layers,
                         schedule=list(range(self.num_hidden_layers)),
                         final_norm=NormSpec(kind="rmsnorm", size=self.hidden_size, eps=self.rms_norm_eps),
                         tie_head=self.tie_word_embeddings, embed_name="model.embed_tokens.weight",
                         final_norm_name="model.norm.weight", head_name="lm_head.weight",
                         head_may_be_absent=True, optional_prefixes=("model.",))
