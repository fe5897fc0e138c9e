"""Budgets and sizes of the engine; the model's own sizes stay in its configuration.

The first four fields carry the names and meanings of kreasof-ai/akas's
``EngineConfig`` (src/akas/config.py:6-24) as its scheduler uses them
(src/akas/scheduling/scheduler.py:149-161): each turn, at most
``prefill_requests`` requests get a portion of their prompt, none more than
``prefill_chunk`` tokens, all together at most ``prefill_token_budget`` (default:
chunk x requests), and at most ``decode_prefill_token_budget`` while any request
decodes. The defaults are larger than the reference's 32/32, which fit its
precompiled launch shapes; here any portion length runs.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


def _positive(name, value, optional=False):
    if value is None and optional:
        return
    if type(value) is not int or value < 1:
        raise ValueError(f"{name} must be a positive integer, got {value!r}")


@dataclass(frozen=True)
class EngineConfig:
    prefill_chunk: int = 2048
    prefill_requests: int = 32
    prefill_token_budget: Optional[int] = 8192
    decode_prefill_token_budget: Optional[int] = None
    max_requests: int = 64  # requests that hold cache at a time (the reference's max_requests / capacity)
    context: int = 4096  # most tokens one request may hold (prompt + generated)
    max_tokens: Optional[int] = None  # tokens the page pool holds; None: max_requests x context
    page_size: int = 64  # tokens per page of keys and values
    dtype: str = "bfloat16"  # "bfloat16" or "float32"
    device: str = "cuda:0"
    cuda_graphs: bool = True  # replay captured graphs for steps that only decode
    run_ahead: bool = True  # launch the next decode step before the tokens of the one in flight are read
    sampling: str = "device"  # "host": the logits are read back and NumPy picks the argmax, a check of the device's
                              # choice as in the reference (src/akas/generation/greedy.py:82-93); greedy requests only

    def __post_init__(self):
        for name in ("prefill_chunk", "prefill_requests", "max_requests", "context", "page_size"):
            _positive(name, getattr(self, name))
        for name in ("prefill_token_budget", "decode_prefill_token_budget", "max_tokens"):
            _positive(name, getattr(self, name), optional=True)
        if self.sampling not in ("device", "host"):
            raise ValueError(f"sampling must be 'device' or 'host', got {self.sampling!r}")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")

    @property
    def pool_tokens(self) -> int:
        return self.max_tokens if self.max_tokens is not None else self.max_requests * self.context
