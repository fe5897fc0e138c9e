"""A single-GPU inference engine for the dense LFM2 decoder on NVIDIA B200 (sm_100a).

    from akas_b200 import Engine, EngineConfig
    engine = Engine("model_folder", config=EngineConfig(dtype="bfloat16"))
    out = engine.generate([[1, 2, 3]], max_tokens=16)[0]["generated_tokens"]

As in kreasof-ai/akas (src/akas/__init__.py:3-6) the package exports ``Engine``, ``EngineConfig`` and
``Request``.
"""

from .config import EngineConfig, Lfm2Config, load_config, register_architecture
from .engine import Engine, ModelRunner, Request, StepEntry

__version__ = "0.1.0"
__all__ = ["Engine", "EngineConfig", "Lfm2Config", "ModelRunner", "Request", "StepEntry", "load_config",
           "register_architecture", "__version__"]
