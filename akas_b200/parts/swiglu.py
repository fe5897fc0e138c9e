"""SwiGLU feed-forward: (silu(x W1^T) * (x W3^T)) W2^T.

W1 (gate) and W3 (up) are stacked at load so that one product feeds the
activation. kreasof-ai/akas: src/akas/models/lfm2/_composition.py:349-355 and
src/akas/ops/activation/kernel.py:86-90; it fuses the two products at graph level
(src/akas/ops/linear/definition.py:652-727).
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, project, project_swiglu, register_ffn, renamed


class SwiGLU(FeedForward):
    takes_normed = True
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.w_gate_up = self.w_down = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        c, f = self.spec.hidden_size, self.spec.intermediate_size
        return {
            self._n("w1.weight"): Param((f, c)),
            self._n("w3.weight"): Param((f, c)),
            self._n("w2.weight"): Param((c, f)),
        }

    def load(self, get):
        self.w_gate_up = torch.cat([get(self._n("w1.weight")), get(self._n("w3.weight"))], dim=0).contiguous()
        self.w_down = get(self._n("w2.weight"))

    def forward(self, x, ctx, residual=None):
        act = project_swiglu(self.rt, x, self.w_gate_up)
        return project(self.rt, act, self.w_down, residual=residual)


register_ffn("swiglu", SwiGLU)
