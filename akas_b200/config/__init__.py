"""Typed configurations and the architecture registry."""

from .engine import EngineConfig
from .lfm2 import ARCHITECTURE as LFM2_ARCHITECTURE
from .lfm2 import ConfigError, Lfm2Config
from .registry import (
    architecture_of,
    architectures,
    config_from_dict,
    load_config,
    register_architecture,
)
from .specs import (
    AttentionSpec,
    LayerSpec,
    ModelSpec,
    PartSpec,
    RMSNormSpec,
    RopeSpec,
    ScheduleEntry,
    ShortConvSpec,
    SwiGLUSpec,
)

register_architecture(LFM2_ARCHITECTURE, Lfm2Config, model_type="lfm2")

__all__ = [
    "AttentionSpec", "ConfigError", "EngineConfig", "LayerSpec", "Lfm2Config", "ModelSpec", "PartSpec",
    "RMSNormSpec", "RopeSpec", "ScheduleEntry", "ShortConvSpec", "SwiGLUSpec", "architecture_of",
    "architectures", "config_from_dict", "load_config", "register_architecture",
]
