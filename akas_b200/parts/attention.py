"""Grouped-query attention over the paged cache.

In order (src/akas/models/lfm2/_composition.py:234-307 in kreasof-ai/akas): one
product for q, k and v (their three matrices are stacked at load); RMSNorm of each
head of q and k over head_dim, then the position encoding of q and k, and the
write of k and v into the pages at each token's absolute position (one kernel);
attention of every query over the keys of its own request up to its own position,
read from the pages, so a portion of a prompt attends to what earlier steps left
and to itself; the output product, added to the residual.
"""

from __future__ import annotations

import torch

from .base import Mixer, PagedKVSpec, Param, build_part, project, register_mixer, renamed


class Attention(Mixer):
    takes_normed = True
    chain_safe = True
    shares_cache = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} heads are not a multiple of {s.num_kv_heads} key/value heads")
        if s.head_dim % 16 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim} must be a multiple of 16, at most 256")
        self.q_norm = build_part("norm", s.qk_norm, runtime)
        self.k_norm = build_part("norm", s.qk_norm, runtime)
        self.position = build_part("position", s.position, runtime)
        self.scale = s.scale if s.scale is not None else s.head_dim ** -0.5
        self.w_qkv = None
        self.w_out = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        p = {
            self._n("q_proj.weight"): Param((s.num_heads * s.head_dim, s.hidden_size)),
            self._n("k_proj.weight"): Param((s.num_kv_heads * s.head_dim, s.hidden_size)),
            self._n("v_proj.weight"): Param((s.num_kv_heads * s.head_dim, s.hidden_size)),
            self._n("out_proj.weight"): Param((s.hidden_size, s.num_heads * s.head_dim)),
        }
        if self.q_norm is not None:
            (norm_param,) = self.q_norm.params().values()
            p[self._n("q_norm.weight")] = norm_param
            p[self._n("k_norm.weight")] = norm_param
        return p

    def load(self, get):
        self.w_qkv = torch.cat(
            [get(self._n("q_proj.weight")), get(self._n("k_proj.weight")), get(self._n("v_proj.weight"))], dim=0
        ).contiguous()
        self.w_out = get(self._n("out_proj.weight"))
        if self.q_norm is not None:
            self.q_norm.weight = get(self._n("q_norm.weight"))
            self.k_norm.weight = get(self._n("k_norm.weight"))

    def cache(self):
        return PagedKVSpec(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        s, ops = self.spec, self.rt.ops
        qkv = project(self.rt, x, self.w_qkv)
        fused = self.position is None or hasattr(self.position, "tables")
        cos = sin = None
        if self.position is not None and fused:
            cos, sin = self.position.tables(ctx)
        norm = self.q_norm.spec if self.q_norm is not None else None
        if fused and ctx.decode_only and hasattr(ops, "qkv_decode_attention"):
            # a decode step: everything between the qkv product and the output product as one kernel, where there is one
            out = ops.qkv_decode_attention(
                qkv, s.num_heads, s.num_kv_heads, s.head_dim,
                self.q_norm.weight if norm else None, self.k_norm.weight if norm else None,
                norm.eps if norm else 0.0, bool(norm and norm.zero_centered), cos, sin, cache.k, cache.v,
                ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions, self.scale, s.window, cache.page_size,
                ctx, write=write,
            )
            if out is not None:
                return project(self.rt, out, self.w_out, residual=residual)
        store = write and fused
        q = ops.qk_norm_rope_store(
            qkv, s.num_heads, s.num_kv_heads, s.head_dim,
            self.q_norm.weight if norm else None, self.k_norm.weight if norm else None,
            norm.eps if norm else 0.0, bool(norm and norm.zero_centered), cos, sin,
            cache.k if store else None, cache.v if store else None,
            ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions, cache.page_size,
        )
        if not fused:
            # A position encoding without rotary tables rewrites q and k itself; k and v go to the pages after it.
            k = qkv[:, s.num_heads * s.head_dim : (s.num_heads + s.num_kv_heads) * s.head_dim]
            q, k = self.position.apply(q, k, ctx)
            if write:
                v = qkv[:, (s.num_heads + s.num_kv_heads) * s.head_dim :]
                ops.kv_store(k, v, cache.k, cache.v, ctx.block_table(cache.group), ctx.seq_of_token,
                             ctx.positions, cache.page_size)
        out = ops.paged_attention(
            q, cache.k, cache.v, ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions,
            self.scale, s.window, cache.page_size, ctx,
        )
        return project(self.rt, out, self.w_out, residual=residual)


register_mixer("attention", Attention)
