"""Typed configurations, part specifications and the architecture registry."""

from .errors import ConfigError, UnknownArchitectureError
from .lfm2 import Lfm2Config
from .plan import (
    AttentionSpec,
    BlockSpec,
    DenseMLPSpec,
    FeedForwardSpec,
    GatedDeltaSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    LinearAttentionSpec,
    MixerSpec,
    ModelPlan,
    NormSpec,
    OutputNormBlockSpec,
    ParallelMixerSpec,
    PooledWindowAttentionSpec,
    PositionSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedMLPSpec,
    SandwichBlockSpec,
    ScheduleEntry,
    ShortConvSpec,
    StreamMixSpec,
    YarnScaling,
)
from .tudulix import TudulixConfig
from .vivulorn import VivulornConfig
from .vuvulorn import VuvulornConfig
from .zozenex import ZozenexConfig
from .registry import architectures, config_from_dict, load_config, register_architecture

register_architecture("Lfm2ForCausalLM", Lfm2Config)
register_architecture("Vuvulorn", VuvulornConfig)
register_architecture("Tudulix", TudulixConfig)
register_architecture("Vivulorn", VivulornConfig)
register_architecture("Zozenex", ZozenexConfig)

__all__ = [
    "AttentionSpec",
    "BlockSpec",
    "ConfigError",
    "DenseMLPSpec",
    "FeedForwardSpec",
    "GatedDeltaSpec",
    "GatedMLPSpec",
    "LatentAttentionSpec",
    "LayerNormSpec",
    "Lfm2Config",
    "LinearAttentionSpec",
    "MixerSpec",
    "ModelPlan",
    "NormSpec",
    "OutputNormBlockSpec",
    "ParallelMixerSpec",
    "PooledWindowAttentionSpec",
    "PositionSpec",
    "RMSNormSpec",
    "RopeSpec",
    "RoutedMLPSpec",
    "SandwichBlockSpec",
    "ScheduleEntry",
    "ShortConvSpec",
    "StreamMixSpec",
    "TudulixConfig",
    "UnknownArchitectureError",
    "VivulornConfig",
    "VuvulornConfig",
    "YarnScaling",
    "ZozenexConfig",
    "architectures",
    "config_from_dict",
    "load_config",
    "register_architecture",
]
