"""Typed configurations and the architecture registry."""

from .specs import (AttentionSpec, BlockSpec, ConfigError, DeltaRuleSpec, DenseMLPSpec,
                    GatedMLPSpec, LayerCall, LogDistanceAttentionSpec, ModelSpec, NormSpec,
                    RotarySpec, StreamBlockSpec)
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       known_architectures, register_architecture)
from .qwen2 import Qwen2Config
from .tebonex import TebonexConfig

__all__ = ["AttentionSpec", "BlockSpec", "ConfigError", "DeltaRuleSpec", "DenseMLPSpec",
           "GatedMLPSpec", "LayerCall", "LogDistanceAttentionSpec", "ModelSpec", "NormSpec",
           "RotarySpec", "StreamBlockSpec", "Qwen2Config", "TebonexConfig", "architecture_name", "config_from_dict",
           "config_from_folder", "known_architectures", "register_architecture"]
