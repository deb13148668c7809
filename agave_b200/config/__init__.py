from .base import (AttentionSpec, BlockSpec, ConfigError, DenseFeedForwardSpec, DistanceBiasSpec,
                   GatedFeedForwardSpec, IdentityNormSpec, LatentAttentionSpec, LayerCall,
                   LayerNormSpec, ModelSpec, NormSpec, QueryTemperatureSpec,
                   RoutedFeedForwardSpec, RotarySpec, WavelengthScalingSpec, default_schedule)
from .registry import (load_config, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture)
from .gemma3 import Gemma3Config
from .ramilorn import RamilornConfig
from .zazerax import ZazeraxConfig
from .bovozen import BovozenConfig
from .kadavik import KadavikConfig

__all__ = [
    "AttentionSpec", "BlockSpec", "ConfigError", "GatedFeedForwardSpec", "LayerCall",
    "LayerNormSpec", "ModelSpec", "NormSpec", "QueryTemperatureSpec", "RoutedFeedForwardSpec",
    "RotarySpec", "RamilornConfig", "default_schedule", "load_config",
    "read_config_json", "register_architecture", "registered_architectures",
    "resolve_architecture", "Gemma3Config", "ZazeraxConfig", "DenseFeedForwardSpec",
    "DistanceBiasSpec", "IdentityNormSpec", "LatentAttentionSpec", "WavelengthScalingSpec",
    "BovozenConfig", "KadavikConfig",
]
