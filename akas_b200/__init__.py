"""A single-GPU inference engine for the dense LFM2 decoder on NVIDIA B200 (sm_100a)."""

from .config import EngineConfig, Lfm2Config, load_config, register_architecture

__version__ = "0.1.0"
__all__ = ["EngineConfig", "Lfm2Config", "load_config", "register_architecture", "__version__"]
