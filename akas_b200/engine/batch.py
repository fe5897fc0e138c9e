"""One step's batch: flat arrays that every kernel reads, built on the host and uploaded in one copy.

kreasof-ai/akas uploads a padded rectangle ``rows x chunk`` of one phase with
``mapping``, ``positions`` and ``lengths`` per row (src/akas/execution/batch.py:21-48)
and expands per-token positions on the device (src/akas/ops/sequence/kernel.py:289-312).
Here a step is a flat run of tokens: portions of prompts of some requests beside
single decoded tokens of others, cut anywhere.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # For a single token that is not known on the host yet: its place among the tokens sampled by the step before
    # (the step function then takes it from the device; ``tokens`` holds any valid id). -1: ``tokens`` is the token.
    source: int = -1


@dataclass
class StepContext:
    """Device views of the batch plus a few host-known sizes; parts read it, none writes it.

    ``seq_of_token`` is ``-1`` and ``slots`` is ``-1`` for padding (a captured decode
    step is padded up to its bucket); kernels touch no cache for those.
    """

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # int32 [N]
    positions: torch.Tensor  # int32 [N] absolute position of each token in its request
    seq_of_token: torch.Tensor  # int32 [N] row of the request in slots / block tables
    cu_seqlens: torch.Tensor  # int32 [R + 1]
    slots: torch.Tensor  # int32 [R] state slot of each request
    logit_rows: torch.Tensor  # int32 [M] flat token index of each wanted row
    num_logit_rows: int
    block_tables: List[torch.Tensor]  # per page group: int32 [R, that group's max_blocks]
    max_query_len: int
    max_context: int  # largest position + 1 in the batch
    decode_only: bool  # every request brings exactly one token
    query_lens: Tuple[int, ...] = ()  # how many tokens each request brings, known on the host (a kernel sizes its grid from it)
    memo: Dict = field(default_factory=dict)  # per-step results shared between layers (rotary tables)

    def block_table(self, group: int) -> torch.Tensor:
        return self.block_tables[group]


class BatchLayout:
    """Offsets (in int32 elements) of each array inside the staging buffer for a batch of N tokens, R requests."""

    def __init__(self, n: int, r: int, m: int, table_widths: Sequence[int]):
        """``table_widths``: for each page group the columns of its block table (``CacheManager.table_widths``)."""
        self.n, self.r, self.m = n, r, m
        off = 0

        def take(count):
            nonlocal off
            start = off
            off += (count + 3) // 4 * 4  # keep every array 16-byte aligned
            return start

        self.token_ids = take(n)
        self.token_src = take(n)
        self.positions = take(n)
        self.seq_of_token = take(n)
        self.cu_seqlens = take(r + 1)
        self.slots = take(r)
        self.logit_rows = take(max(m, 1))
        self.table_widths = tuple(table_widths)
        self.tables = [take(r * width) for width in self.table_widths]
        self.size = off


def fill_batch(host: np.ndarray, layout: BatchLayout, entries: Sequence[StepEntry], cache, pad_to: int = 0, tokens=None):
    """Writes the arrays of ``entries`` into ``host`` (int32) at ``layout``'s offsets.

    ``pad_to``: for a decode-only step, the bucket size; padding tokens get request -1.
    ``tokens``: the entries' token ids as arrays, if the caller has them already.
    Returns (max_query_len, max_context).
    """
    n, r = layout.n, layout.r
    tok = host[layout.token_ids : layout.token_ids + n]
    src = host[layout.token_src : layout.token_src + n]
    pos = host[layout.positions : layout.positions + n]
    seq = host[layout.seq_of_token : layout.seq_of_token + n]
    cu = host[layout.cu_seqlens : layout.cu_seqlens + r + 1]
    slots = host[layout.slots : layout.slots + r]
    rows = host[layout.logit_rows : layout.logit_rows + max(layout.m, 1)]
    live = len(entries)
    max_q = max_ctx = at = 0
    if live:
        # whole arrays at once: a step may hold hundreds of requests, and a statement per request adds up
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=live)
        starts = np.fromiter((cache.length(e.request) for e in entries), dtype=np.int64, count=live)
        first = np.zeros(live + 1, dtype=np.int64)
        np.cumsum(counts, out=first[1:])
        at = int(first[live])
        if tokens is None:
            tokens = [np.asarray(e.tokens, dtype=np.int64) for e in entries]
        tok[:at] = np.concatenate(tokens) if live > 1 else tokens[0]
        owner = np.repeat(np.arange(live, dtype=np.int64), counts)
        seq[:at] = owner
        pos[:at] = np.arange(at, dtype=np.int64) + (starts - first[:live])[owner]
        cu[:live] = first[:live]
        slots[:live] = np.fromiter((cache.slot(e.request) for e in entries), dtype=np.int64, count=live)
        src[:at] = -1
        for i, e in enumerate(entries):
            if e.source >= 0:
                if counts[i] != 1:
                    raise ValueError("only a single token can come from the step before")
                src[first[i]] = e.source
        wanted = [int(first[i]) + w for i, e in enumerate(entries) for w in e.want]
        rows[: len(wanted)] = wanted
        for g, (offset, max_blocks) in enumerate(zip(layout.tables, layout.table_widths)):
            table = host[offset : offset + live * max_blocks].reshape(live, max_blocks)
            table[:] = -1
            for i, e in enumerate(entries):
                blocks = cache.blocks(e.request, g)
                table[i, : len(blocks)] = blocks
        max_q = int(counts.max())
        max_ctx = int((starts + counts).max())
    cu[len(entries)] = at
    if pad_to:
        tok[at:n] = 0
        src[at:n] = -1
        pos[at:n] = 0
        seq[at:n] = -1
        cu[live + 1 : r + 1] = at
        slots[live:r] = -1
        for offset, max_blocks in zip(layout.tables, layout.table_widths):
            host[offset + live * max_blocks : offset + r * max_blocks] = -1
    return max_q, max_ctx
