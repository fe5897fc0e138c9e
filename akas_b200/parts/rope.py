"""Rotary position encoding, rotate-half pairing (i, i + rotary/2).

theta_i = position * base^(-2i/rotary). kreasof-ai/akas forms this product with a
hi/lo split of the frequency and a two-term reduction by 2 pi so that float32 stays
accurate at long positions (src/akas/ops/attention/kernel.py:788-851, 927-939). Here
the frequencies are float64 constants made once on the host, and the kernel
multiplies, reduces and rounds to float32 last; the tables of a step are made once
and shared by every layer with the same encoding.
"""

from __future__ import annotations

import torch

from .base import Part, register_position


class Rope(Part):
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        rotary = spec.rotary
        if rotary % 2 or rotary > spec.head_dim or rotary <= 0:
            raise ValueError(f"rotary_dim {rotary} must be even and at most head_dim {spec.head_dim}")
        i = torch.arange(rotary // 2, dtype=torch.float64)
        self.inv_freq = (torch.tensor(float(spec.theta), dtype=torch.float64) ** (-2.0 * i / rotary)).to(runtime.device)
        self.key = ("rope", rotary, float(spec.theta))

    def tables(self, ctx):
        """(cos, sin), float32 [N, rotary/2], for the tokens of this step."""
        cached = ctx.memo.get(self.key)
        if cached is None:
            cached = self.rt.ops.rope_tables(ctx.positions, self.inv_freq)
            ctx.memo[self.key] = cached
        return cached


register_position("rope", Rope)
