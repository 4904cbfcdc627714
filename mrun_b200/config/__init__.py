from .base import ConfigError, UnsupportedArchitecture
from .qwen3 import Qwen3Config
from .spec import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec,
                   ScheduleEntry, TensorSpec)

__all__ = ["ConfigError", "UnsupportedArchitecture", "Qwen3Config", "AttentionSpec",
           "GatedMLPSpec", "LayerSpec", "ModelSpec", "RMSNormSpec", "RotarySpec",
           "ScheduleEntry", "TensorSpec"]
