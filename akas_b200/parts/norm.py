"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, computed in float32.

kreasof-ai/akas: src/akas/ops/normalization/kernel.py:440-444; the weight is used
as it stands (its ``zero_centered`` flag, 1 + w, belongs to other contracts:
src/akas/ops/normalization/definition.py:285-348) and is offered here as an option.
"""

from __future__ import annotations

import torch

from .base import Normed, Param, Part, register_norm


class RMSNorm(Part):
    chain_safe = True

    def __init__(self, spec, runtime, name: str = "weight"):
        super().__init__(spec, runtime)
        self.name = name
        self.weight = None

    def params(self):
        return {self.name: Param((self.spec.size,), role="vector", mean=0.0 if self.spec.zero_centered else 1.0)}

    def load(self, get):
        self.weight = get(self.name)

    def forward(self, x, out_dtype=None, rows=None):
        """x: [N, size] (or [N, heads, size] flattened by the caller); rows: optional int32 row indices."""
        return self.rt.ops.rmsnorm(
            x, self.weight, self.spec.eps, self.spec.zero_centered, out_dtype or self.rt.dtype, rows
        )


    def lazy(self, h, rows=None) -> Normed:
        return Normed(self, h, rows)


register_norm("rmsnorm", RMSNorm)
