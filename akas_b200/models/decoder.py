"""The generic decoder that every registered architecture is built as.

Embedding (times ``ModelSpec.embedding_multiplier`` if the architecture has one), the blocks of
``ModelSpec.layers`` in the order of ``ModelSpec.schedule`` (a list that may name a layer twice or let an
entry read another entry's cache), the final norm on the rows whose logits are wanted, the head, and the
architecture's ``logit_scale`` and ``logit_softcap`` if it has them. The head is the checkpoint's
head tensor when it has one, else the embedding:
src/akas/models/lfm2/weights.py:399-402 and _composition.py:363-380 in kreasof-ai/akas).
It holds weights and computes; caches belong to the cache manager and reach the
blocks through ``caches[entry]``.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from ..config.specs import ModelSpec
from ..parts.base import Param, Runtime, build_part, project
from ..parts.block import Block


class Decoder:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.blocks: List[Block] = [Block(layer, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.schedule = spec.run_order()
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}; there are {len(self.blocks)}")
            if entry.cache is not None:
                owner = self.schedule[entry.cache] if 0 <= entry.cache < i else None
                if owner is None or owner.cache is not None:
                    raise ValueError(f"schedule entry {i} reads cache {entry.cache}, which is no earlier owning entry")
                for which in (owner.layer, entry.layer):
                    mixer = self.blocks[which].mixer
                    if not mixer.shares_cache:
                        raise ValueError(f"schedule entry {i} reads the cache of entry {entry.cache}, but the mixer of layer "
                                         f"{which} ({type(mixer).__name__}) keeps a summary of the past that has moved on "
                                         "when a reader runs: give the entry a cache of its own")
        self.embedding = None
        self.head = None

    # ------------------------------------------------------------------ weights

    def params(self) -> Dict[str, Param]:
        s = self.spec
        out = {s.embedding_name: Param((s.vocab_size, s.hidden_size))}
        (norm_param,) = self.final_norm.params().values()
        out[s.final_norm_name] = norm_param
        if s.head_name is not None:
            out[s.head_name] = Param((s.vocab_size, s.hidden_size), optional=s.head_optional)
        for block in self.blocks:
            out.update(block.params())
        return out

    def load(self, get: Callable[[str], torch.Tensor], has: Callable[[str], bool] = lambda name: True) -> None:
        s = self.spec
        self.embedding = get(s.embedding_name)
        self.final_norm.load(lambda _name: get(s.final_norm_name))
        self.head = get(s.head_name) if s.head_name is not None and has(s.head_name) else self.embedding
        for block in self.blocks:
            block.load(get)

    # ------------------------------------------------------------------ compute

    def cache_specs(self):
        """For each schedule entry that owns a cache: what its mixer needs (or None)."""
        return [self.blocks[e.layer].mixer.cache() if e.cache is None else None for e in self.schedule]

    def forward(self, ctx, caches) -> torch.Tensor:
        """Runs the tokens of ``ctx`` and returns float32 logits ``[len(ctx.logit_rows), vocab]``."""
        ops = self.rt.ops
        # A decode step is a chain of small operations; kernels that can run such a chain as one launch are told
        # where it begins and ends, and it is cut before any block that has not declared itself safe inside one.
        chained = ctx.decode_only and hasattr(ops, "chain_begin") and ops.chain_begin(ctx.num_tokens)
        try:
            return self._forward(ctx, caches, chained)
        finally:
            if chained:
                ops.chain_end()

    def _forward(self, ctx, caches, chained: bool) -> torch.Tensor:
        ops = self.rt.ops
        spec = self.spec
        h = ops.embedding(ctx.token_ids, self.embedding)
        if spec.embedding_multiplier is not None:
            h = ops.scale_cap(h, scale=spec.embedding_multiplier)
        for i, entry in enumerate(self.schedule):
            owner = i if entry.cache is None else entry.cache
            block = self.blocks[entry.layer]
            if chained and not block.chain_safe:
                ops.chain_flush()
            h = block.forward(h, ctx, caches[owner], write=entry.cache is None)
        if chained and not getattr(self.final_norm, "chain_safe", False):
            ops.chain_flush()
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        if hasattr(self.final_norm, "lazy"):
            x = self.final_norm.lazy(h, rows=ctx.logit_rows)
        else:
            x = self.final_norm.forward(h, rows=ctx.logit_rows)
        logits = project(self.rt, x, self.head, out_dtype=torch.float32)
        if spec.logit_scale is not None or spec.logit_softcap is not None:
            logits = ops.scale_cap(logits, scale=1.0 if spec.logit_scale is None else spec.logit_scale,
                                   cap=spec.logit_softcap or 0.0)
        return logits
