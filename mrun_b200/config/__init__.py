from .base import ConfigError, UnsupportedArchitecture
from .qwen3 import Qwen3Config
from .spec import (AttentionSpec, GatedMLPSpec, LatentAttentionSpec, LayerSpec, ModelSpec, RMSNormSpec,
                   RotarySpec, RoutedMLPSpec, ScaledRotarySpec, ScheduleEntry, SoftCapSpec, TensorSpec)
from .zasesun import ZasesunConfig

__all__ = ["ConfigError", "UnsupportedArchitecture", "Qwen3Config", "ZasesunConfig", "AttentionSpec",
           "GatedMLPSpec", "LatentAttentionSpec", "LayerSpec", "ModelSpec", "RMSNormSpec", "RotarySpec",
           "RoutedMLPSpec", "ScaledRotarySpec", "ScheduleEntry", "SoftCapSpec", "TensorSpec"]
