"""What every part is, and the registries that map a spec's ``kind`` to a part.

A part is a mixer, a feed-forward, a norm or a position encoding. It is built
from its spec alone (``Part(spec, runtime)``), says which tensors it wants
(``params()``), takes them (``load()``), and computes (``forward()``). No part
knows which model it is in: names of checkpoint tensors reach it through the
prefix that the block passes, and sizes through its spec.

Interfaces (duck-typed; these base classes only document and give defaults):

* Norm: ``params()``, ``load(get)``, ``forward(x, out_dtype=None, rows=None)``; optionally
  ``lazy(h, rows=None)`` -> ``Normed`` so that a following product may absorb it.
* PositionEncoding: ``prepare(ctx)`` once per step, ``tables(ctx)`` -> (cos, sin)
  for the fused rotary kernel, or ``apply(q, k, ctx)`` for any other encoding.
* Mixer: ``params()``, ``load(get)``, ``cache()`` -> the cache it needs (a
  ``PagedKVSpec``, a ``StateSpec`` or ``None``), ``forward(x, ctx, cache, residual,
  write)``.
* FeedForward: ``params()``, ``load(get)``, ``forward(x, ctx, residual)``.

``forward`` of a mixer or feed-forward gets the normed activations ``x`` ``[N, C]``
in the compute dtype and, when ``residual`` is given (float32 ``[N, C]``), returns
``residual + result`` in float32 (it may add in place; the fused kernels do).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class Param:
    """A tensor a part wants from the checkpoint.

    ``role`` decides the dtype it is held in: a ``"matrix"`` is an operand of a
    matrix product and takes the compute dtype; a ``"vector"`` (norm weights,
    convolution taps, biases) is held in float32; ``"table"`` is an integer table
    held in int32. ``optional`` tensors may be absent from the checkpoint. ``mean``
    is the mean that the random-weights mode draws the tensor around (1 for norm
    weights).
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    mean: float = 0.0


class PagedSpec:
    """What a mixer with per-token storage asks of the cache manager; a mixer returns an instance from ``cache()``.

    ``pools(page_size)`` names its pools and gives the shape of ONE page of each (``{"k": (kv_heads, page, head_dim),
    ...}``); the manager allocates ``[pages, *shape]`` per pool and hands them over as attributes of the view the
    mixer gets (``cache.k``). ``window``: how many of the latest tokens are ever read (None: all); pages behind the
    window are given back while the request runs. ``page_size``: tokens per page if the mixer needs a size of its own
    (None: the engine's). ``dtype``: None for the compute dtype. Layers whose specs agree in ``paging()`` share page
    numbers, a free list and a block table; everything else (what a page holds) is the layer's own."""

    window: Optional[int] = None
    page_size: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def pools(self, page_size: int) -> Dict[str, Tuple[int, ...]]:
        raise NotImplementedError

    def paging(self) -> tuple:
        return (self.window, self.page_size)


@dataclass(frozen=True)
class PagedKVSpec(PagedSpec):
    """Keys and values of every position (or of the last ``window``), in pages ``[kv_heads, page, head_dim]``."""

    num_kv_heads: int = 1
    head_dim: int = 16
    window: Optional[int] = None
    page_size: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def pools(self, page_size: int) -> Dict[str, Tuple[int, ...]]:
        shape = (self.num_kv_heads, page_size, self.head_dim)
        return {"k": shape, "v": shape}


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one row of ``shape`` per request slot, zero at admission."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What a part needs to know about where it runs: compute dtype, device, kernels."""

    dtype: torch.dtype
    device: torch.device
    ops: Any


class Normed:
    """The output of a norm that has not run yet: ``norm(h[rows])``.

    A block hands it to parts that set ``takes_normed``; they pass it to ``project`` /
    ``project_swiglu`` for their first matrix product, where the kernels may compute the norm inside
    the product instead of in a pass of its own. ``tensor()`` runs the norm and gives the plain result.
    """

    def __init__(self, norm, h, rows=None):
        self.norm, self.h, self.rows = norm, h, rows
        self._tensor = None

    def tensor(self):
        if self._tensor is None:
            self._tensor = self.norm.forward(self.h, rows=self.rows)
        return self._tensor


def project(rt: "Runtime", x, w, out_dtype=None, residual=None):
    """``x . w^T`` for a tensor or a ``Normed``; with ``residual`` the product is added into it."""
    if isinstance(x, Normed):
        spec = x.norm.spec
        if residual is None and getattr(spec, "kind", None) == "rmsnorm" and hasattr(rt.ops, "norm_linear"):
            return rt.ops.norm_linear(x.h, x.norm.weight, spec.eps, spec.zero_centered, w, out_dtype, x.rows)
        x = x.tensor()
    return rt.ops.linear(x, w, out_dtype=out_dtype, residual=residual)


def project_swiglu(rt: "Runtime", x, w_gate_up):
    """``silu(x . w1^T) * (x . w3^T)`` for the stacked ``[w1; w3]``, for a tensor or a ``Normed``."""
    if isinstance(x, Normed):
        spec = x.norm.spec
        if getattr(spec, "kind", None) == "rmsnorm" and hasattr(rt.ops, "norm_linear"):
            return rt.ops.norm_linear(x.h, x.norm.weight, spec.eps, spec.zero_centered, w_gate_up, None, x.rows, True)
        x = x.tensor()
    if hasattr(rt.ops, "linear_swiglu"):
        return rt.ops.linear_swiglu(x, w_gate_up)
    return rt.ops.swiglu(rt.ops.linear(x, w_gate_up))


class Part:
    takes_normed = False  # True: forward accepts a ``Normed`` in place of the normed tensor
    # True: the part reads and writes device tensors through ``runtime.ops`` functions only, so an operations module
    # that defers launches (a decode step run as one chain) may keep deferring across it. A part that computes with
    # torch directly leaves this False, and the decoder makes everything pending run before the part does.
    chain_safe = False

    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime

    def params(self) -> Dict[str, Param]:
        return {}

    def load(self, get: Callable[[str], torch.Tensor]) -> None:
        pass


class Mixer(Part):
    # True: another entry of the run order may read this mixer's cache (``write=False``) after the owner has run in
    # the same step, and sees the same past however the tokens were cut into steps: attention does, since every
    # earlier token's keys and values lie in the cache by then. A mixer whose cache is a summary of the past leaves
    # this False: once the owner has run, the summary has moved past the step's tokens, so a reader would see another
    # past in a step of one token than in a step of many. The decoder refuses a run order that shares such a cache.
    shares_cache = False

    def cache(self):
        return None

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx, residual=None):
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "ffn": {}, "norm": {}, "position": {}}


def _register(family: str, kind: str, cls: type) -> None:
    _REGISTRIES[family][kind] = cls


def register_mixer(kind: str, cls: type) -> None:
    _register("mixer", kind, cls)


def register_ffn(kind: str, cls: type) -> None:
    _register("ffn", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    _register("norm", kind, cls)


def register_position(kind: str, cls: type) -> None:
    _register("position", kind, cls)


def build_part(family: str, spec, runtime: Runtime):
    """The part that ``spec.kind`` names in the registry of ``family``; ``None`` for a ``None`` spec."""
    if spec is None:
        return None
    table = _REGISTRIES[family]
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise KeyError(f"no {family} registered for kind {kind!r}; registered: {sorted(table)}")
    return table[kind](spec, runtime)


def renamed(spec, local: str) -> str:
    """The checkpoint's name for a part's local parameter name (``spec.names`` overrides)."""
    names = getattr(spec, "names", None) or {}
    return names.get(local, local)
