"""Architecture-neutral descriptions of a decoder: what the engine builds from.

An architecture's typed configuration (for instance ``Lfm2Config``) turns itself
into a ``ModelSpec``. The model builder, the cache manager and the weight loader
read only the spec: every size and constant that a part needs is a field here,
chosen layer by layer, so one model may hold different mixers and feed-forwards
in different layers. The order in which layers run is data too (``ModelSpec.schedule``).

A spec of a part is a frozen dataclass with a ``kind`` string; the registries in
``akas_b200.parts.registry`` map that string to the class that implements it.
Parts defined outside this package use ``PartSpec`` directly (kind + free-form
``options``) or their own dataclass with a ``kind`` attribute.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part that this package does not know: its kind and whatever it needs."""

    kind: str
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (w, or 1 + w when zero_centered)."""

    size: int
    eps: float
    zero_centered: bool = False
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding of the first ``rotary_dim`` channels of each head."""

    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None  # None: the whole head
    kind: str = "rope"

    @property
    def rotary(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: Optional[Any] = None  # a norm spec of size head_dim, applied per head before the position encoding
    position: Optional[Any] = None  # a position-encoding spec, or None
    window: Optional[int] = None  # None: every earlier key; w: the last w keys, the query's own included
    scale: Optional[float] = None  # None: head_dim ** -0.5
    kind: str = "attention"
    names: Mapping[str, str] = field(default_factory=dict)  # local parameter name -> name in the checkpoint


@dataclass(frozen=True)
class ShortConvSpec:
    """LFM2's gated causal depthwise convolution with a state of kernel_size-1 rows."""

    hidden_size: int
    kernel_size: int
    bias: bool = False
    kind: str = "short_conv"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class SwiGLUSpec:
    """silu(x W1^T) * (x W3^T), then W2."""

    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts it holds, how they are arranged, and where its weights are.

    ``mixer_prefix`` and ``ffn_prefix`` are prepended to the parts' local parameter
    names (``"model.layers.3.self_attn."``); the two norms name their weight whole.
    """

    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    mixer_prefix: str
    ffn_prefix: str
    mixer_norm_name: str
    ffn_norm_name: str
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One call in the run order: layer ``layer`` runs with cache ``cache``.

    ``cache`` names a cache by the index of the schedule entry that owns it; by
    default an entry owns its own cache. An entry whose ``cache`` is another
    entry's index reads that entry's cache and writes nothing into it (the mixer
    is told ``write=False``). Naming a layer in two entries runs its weights twice,
    each time with the cache of its own entry.
    """

    layer: int
    cache: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    final_norm: Any
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]  # None: the head is always the embedding
    head_optional: bool = False  # the head tensor may be absent; the embedding is the head then
    schedule: Tuple[ScheduleEntry, ...] = ()
    max_context: int = 128000
    # What some architectures do at the decoder's two ends (LFM2 does none of it): the embedding's rows times a
    # constant; the logits times a constant; then cap * tanh(logits / cap).
    embedding_multiplier: Optional[float] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))
