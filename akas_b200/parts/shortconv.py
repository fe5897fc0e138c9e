"""LFM2's short-convolution mixer.

BCx = x W_in^T gives, per token, three parts in the order B, C, x. u = B * x;
s[t] = sum_j hist[j] * w[:, j] + u[t] * w[:, L-1] (+ bias), hist being the previous
L-1 values of u of this request, oldest first, zero where the request began;
y = C * s; out = y W_out^T. The state of a request is its last L-1 values of u, in
float32. kreasof-ai/akas: src/akas/ops/convolution/kernel.py:43-91, and :318-333
for where a bias is added; the checkpoint's taps are [C, 1, L]
(src/akas/models/lfm2/weights.py:405-407).

``bias`` (LFM2's ``conv_bias``) switches on three biases together: ``in_proj.bias`` [3C] on BCx,
``conv.bias`` [C] on s, ``out_proj.bias`` [C] on the output. kreasof-ai/akas refuses the option
(src/akas/models/lfm2/config.py:87), so this reading is the architecture's, not the reference's: a
checkpoint with ``conv_bias: true`` carries all three tensors, and one that lacks any is refused.
The two projection biases are added in float32, before the product's one rounding.
"""

from __future__ import annotations

import torch

from .base import Mixer, Normed, Param, StateSpec, project, register_mixer, renamed


class ShortConv(Mixer):
    takes_normed = True
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if not 2 <= spec.kernel_size <= 16:
            raise ValueError(f"short-conv kernel_size {spec.kernel_size} must be from 2 to 16")
        self.w_in = self.w_out = self.taps = self.bias = self.bias_in = self.bias_out = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        c, l = self.spec.hidden_size, self.spec.kernel_size
        p = {
            self._n("in_proj.weight"): Param((3 * c, c)),
            self._n("conv.weight"): Param((c, 1, l), role="vector"),
            self._n("out_proj.weight"): Param((c, c)),
        }
        if self.spec.bias:
            p[self._n("in_proj.bias")] = Param((3 * c,), role="vector")
            p[self._n("conv.bias")] = Param((c,), role="vector")
            p[self._n("out_proj.bias")] = Param((c,), role="vector")
        return p

    def load(self, get):
        c, l = self.spec.hidden_size, self.spec.kernel_size
        self.w_in = get(self._n("in_proj.weight"))
        self.taps = get(self._n("conv.weight")).reshape(c, l).contiguous()
        self.w_out = get(self._n("out_proj.weight"))
        if self.spec.bias:
            self.bias_in = get(self._n("in_proj.bias"))
            self.bias = get(self._n("conv.bias"))
            self.bias_out = get(self._n("out_proj.bias"))

    def cache(self):
        return StateSpec((self.spec.kernel_size - 1, self.spec.hidden_size), torch.float32)

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        ops = self.rt.ops
        y = None
        if (self.bias_in is None and ctx.decode_only and isinstance(x, Normed) and x.rows is None
                and getattr(x.norm.spec, "kind", None) == "rmsnorm" and hasattr(ops, "norm_linear_short_conv")):
            # a decode step: norm, in projection and convolution as one kernel, where the kernels have one
            y = ops.norm_linear_short_conv(x.h, x.norm.weight, x.norm.spec.eps, x.norm.spec.zero_centered, self.w_in,
                                           self.taps, self.bias, cache.state, ctx.seq_of_token, ctx.slots, write=write)
        if y is None:
            if self.bias_in is None:
                bcx = project(self.rt, x, self.w_in)
            else:  # the product stays float32 until its bias is in, then rounds once
                bcx = ops.add_bias(project(self.rt, x, self.w_in, out_dtype=torch.float32), self.bias_in, self.rt.dtype)
            y = ops.short_conv(bcx, self.taps, self.bias, cache.state, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots,
                               decode_only=ctx.decode_only, write=write)
        if self.bias_out is None:
            return project(self.rt, y, self.w_out, residual=residual)
        if residual is None:
            return ops.add_bias(project(self.rt, y, self.w_out, out_dtype=torch.float32), self.bias_out, self.rt.dtype)
        return project(self.rt, y, self.w_out, residual=ops.add_bias(residual, self.bias_out))


register_mixer("short_conv", ShortConv)
