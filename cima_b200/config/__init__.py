from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)
from .registry import (ArchitectureEntry, UnknownArchitecture, lookup_architecture,
                       read_config_json, register_architecture, registered_architectures)
from .qwen2 import ConfigError, Qwen2Config
from . import shapes

__all__ = ["BlockSpec", "FeedForwardSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "ArchitectureEntry", "UnknownArchitecture", "lookup_architecture", "read_config_json",
           "register_architecture", "registered_architectures", "ConfigError", "Qwen2Config"]
