"""One generation request as the scheduler sees it.

The first fields are those of kreasof-ai/akas's ``Request`` (src/akas/requests.py:7-16): prompt, limit
(``max_tokens``), cancelled, slot, offset, output, published. Sampling options and the reason a request
finished are added here.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from threading import Event
from typing import List, Optional

import numpy as np

_ids = itertools.count()


@dataclass(eq=False)  # a request is itself, not its field values: lists of requests are searched by identity
class Request:
    prompt: List[int]
    limit: int  # most tokens to generate
    channel: object = None
    cancelled: Event = field(default_factory=Event)
    slot: Optional[int] = None
    offset: int = 0  # tokens of prompt + output whose keys, values and state are in the cache
    output: List[int] = field(default_factory=list)
    published: int = 0
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    softcap: float = 0.0  # 0: none
    repetition_penalty: float = 1.0  # 1: none
    repetition_window: int = 96  # how many of the last generated tokens the penalty looks at
    seed: Optional[int] = None
    eos_token_id: Optional[int] = None
    finish_reason: Optional[str] = None  # "length", "stop" (end-of-sequence token) or "cancelled"
    preemptions: int = 0
    inflight: int = 0  # tokens sampled by steps that were launched and not read back yet
    id: int = field(default_factory=lambda: next(_ids))
    _uniforms: Optional[np.ndarray] = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def tokens(self) -> List[int]:
        """Everything the cache must hold before the next token can be sampled: prompt, then output."""
        return self.prompt + self.output

    def pending_tokens(self) -> int:
        """Tokens the cache does not hold yet; a token that is still in flight counts as the last of them."""
        return len(self.prompt) + len(self.output) + self.inflight - self.offset

    @property
    def adjusts_logits(self) -> bool:
        return self.softcap > 0 or self.repetition_penalty != 1.0

    def recent(self) -> List[int]:
        """The generated tokens that the repetition penalty looks at."""
        return self.output[-self.repetition_window:] if self.repetition_window > 0 else []

    def uniform(self) -> float:
        """The uniform number for the next generated token: a function of (seed, index of that token) only,
        so what a request samples does not depend on the batches it ran in, nor on a preemption."""
        if self._uniforms is None:
            seed = self.seed if self.seed is not None else np.random.SeedSequence().entropy
            self._uniforms = np.random.default_rng(seed).random(self.limit, dtype=np.float32)
        return float(self._uniforms[len(self.output) + self.inflight])
