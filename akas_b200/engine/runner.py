"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

``ModelRunner`` owns the model, the cache manager and the staging of a step's
arrays. ``step`` runs only the tokens it is given, as one batch, from what earlier
steps left in the cache; it is the only writer of pages and state slots. Generation,
the scheduler and trace replay all go through it.

kreasof-ai/akas's counterpart is ``Executor`` with ``Batch.prepare/run``
(src/akas/execution/executor.py:360-374, src/akas/execution/batch.py:21-134): one
captured CUDA graph per compiled ``rows x chunk`` geometry, prefill and decode in
separate launches. Here any mix runs eagerly, and steps that only decode replay a
CUDA graph captured per batch-size bucket (the reference's device for decode
latency too: src/akas/execution/forward.py:41-45).
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.engine import EngineConfig
from ..config.registry import load_config
from ..models.decoder import Decoder
from ..parts.base import Runtime
from ..weights.loader import load_weights
from .batch import BatchLayout, StepContext, StepEntry, fill_batch

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
_GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
_TOKEN_ROUNDING = 256
_SHAPE_REPEATS, _SHAPE_GRAPHS = 3, 4  # a step shape is captured when it comes the third time; at most four are kept


def default_ops(device: torch.device, dtype: torch.dtype):
    """The compiled sm_100a kernels. There is no other product path: anything else fails here."""
    if device.type != "cuda":
        raise RuntimeError(
            f"akas_b200 runs on CUDA devices only (got {device}); pass ops=akas_b200.ops.reference "
            "explicitly to exercise host logic without kernels"
        )
    from ..ops import cuda as cuda_ops

    cuda_ops.require(cuda_ops.libraries_for(dtype))
    return cuda_ops


class ModelRunner:
    def __init__(self, model_dir, config: Optional[EngineConfig] = None, ops=None, model_config=None):
        self.config = config or EngineConfig()
        self.device = torch.device(self.config.device)
        self.dtype = _DTYPES[self.config.dtype]
        self.ops = ops if ops is not None else default_ops(self.device, self.dtype)
        self.model_config = model_config if model_config is not None else load_config(model_dir)
        spec = self.model_config.model_spec()
        self.runtime = Runtime(self.dtype, self.device, self.ops)
        self.model = Decoder(spec, self.runtime)
        self.weight_bytes = load_weights(self.model, model_dir)
        self.vocab_size = spec.vocab_size
        self.cache = CacheManager(
            self.model.cache_specs(), self.config.page_size, self.config.pool_tokens, self.config.max_requests,
            self.config.context, dtype=self.dtype, device=self.device,
        )
        self._host = None  # pinned int32 staging
        self._dev = None
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._shape_graphs: Dict[tuple, "_DecodeGraph"] = {}
        self._shape_counts: Dict[tuple, int] = {}
        self.steps = 0
        self.kernels_per_decode_step: Dict[int, int] = {}  # bucket -> kernels inside its captured graph

    # ------------------------------------------------------------------ requests

    def admit(self, request: Hashable) -> int:
        return self.cache.admit(request, zero=getattr(self.ops, "zero_rows", None))

    def release(self, request: Hashable) -> None:
        self.cache.release(request)

    # ------------------------------------------------------------------ staging

    def _staging(self, size: int):
        """A pinned host buffer and a device buffer for one step's arrays. The copy between them is asynchronous
        and nothing makes the host wait for a step, so host buffers are taken in turn from a small ring, and one is
        reused only after the copy that last read it has run (``_Pinned.take`` waits for that copy's event)."""
        if self._dev is None or self._dev.numel() < size:
            cap = max(size, 1 << 14)
            cap = 1 << (cap - 1).bit_length()
            self._host = _Pinned(cap, self.device)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._host, self._dev

    def _context(self, dev: torch.Tensor, lay: BatchLayout, max_q: int, max_ctx: int, decode_only: bool, query_lens=()):
        return StepContext(
            num_tokens=lay.n,
            num_seqs=lay.r,
            token_ids=dev[lay.token_ids : lay.token_ids + lay.n],
            positions=dev[lay.positions : lay.positions + lay.n],
            seq_of_token=dev[lay.seq_of_token : lay.seq_of_token + lay.n],
            cu_seqlens=dev[lay.cu_seqlens : lay.cu_seqlens + lay.r + 1],
            slots=dev[lay.slots : lay.slots + lay.r],
            logit_rows=dev[lay.logit_rows : lay.logit_rows + lay.m],
            num_logit_rows=lay.m,
            block_tables=[dev[o : o + lay.r * mb].view(lay.r, mb) for o, mb in zip(lay.tables, lay.table_widths)],
            max_query_len=max_q,
            max_context=max_ctx,
            decode_only=decode_only,
            query_lens=tuple(query_lens),
        )

    # ------------------------------------------------------------------ the step

    def step(self, entries: Sequence[StepEntry], previous: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one batch. Returns float32 logits ``[sum(len(e.want)), vocab]`` on the device, in the
        order of the entries and of their ``want``. The result is valid until the next call of ``step``: a step that
        replays a captured graph returns the graph's own output buffer, which the next replay overwrites (and which
        the sampler may adjust in place); clone it to keep it longer. Unknown requests are admitted; pages are taken
        first. When a request cannot be admitted or ``OutOfPages`` is raised, nothing has run, the requests that
        this call admitted are released again, and pages already reserved for known requests stay with them.
        ``previous``: the int32 device tensor of tokens that the step before sampled, for entries that name a
        ``source`` in it."""
        entries = [e for e in entries if len(e.tokens)]
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        arrays = [np.asarray(e.tokens, dtype=np.int64) for e in entries]  # converted once, checked and copied as arrays
        if previous is None and any(e.source >= 0 for e in entries):
            raise ValueError("an entry takes its token from the step before, but no such tokens were given")
        if len({e.request for e in entries}) != len(entries):
            twice = [e.request for e in entries if sum(1 for o in entries if o.request == e.request) > 1]
            raise ValueError(f"request {twice[0]!r} appears twice in one step")
        flat = np.concatenate(arrays) if len(arrays) > 1 else arrays[0]
        if flat.ndim != 1 or any(ids.ndim != 1 for ids in arrays):
            raise ValueError("tokens must be flat sequences of ids")
        if int(flat.min()) < 0 or int(flat.max()) >= self.vocab_size:  # one check for the step; the culprit only then
            for e, ids in zip(entries, arrays):
                bad = ids[(ids < 0) | (ids >= self.vocab_size)]
                if bad.size:
                    raise ValueError(f"request {e.request!r}: token ids {bad[:4].tolist()} outside [0, {self.vocab_size})")
        for e in entries:  # every entry is checked before any request is admitted or any page is taken
            if any(not 0 <= w < len(e.tokens) for w in e.want):
                raise ValueError(f"request {e.request!r}: wanted places {list(e.want)} outside its {len(e.tokens)} tokens")
        newcomers = []
        try:
            for e in entries:
                if e.request not in self.cache:
                    self.admit(e.request)
                    newcomers.append(e.request)
            for e in entries:
                self.cache.reserve(e.request, len(e.tokens))
        except Exception:
            for request in newcomers:  # a step that cannot run leaves no request behind that it brought in itself
                self.release(request)
            raise

        decode_only = all(len(e.tokens) == 1 for e in entries)
        all_wanted = all(list(e.want) == [0] for e in entries)
        graphs = self.config.cuda_graphs and self.device.type == "cuda"
        repeated = self._repeated_shape(entries) if graphs and not (decode_only and all_wanted) else None
        if decode_only and all_wanted and graphs:
            logits = self._decode_graph_step(entries, arrays, previous)
        elif repeated is not None:
            logits = repeated.run(entries, arrays, previous)
        else:
            n = sum(len(e.tokens) for e in entries)
            m = sum(len(e.want) for e in entries)
            # A serving step brings any number of tokens. Beyond 256 the step is padded to a multiple of 256 with
            # tokens of no request, which every kernel skips: the products' tiles hold 256 token rows (a pair of SMs),
            # so the rounding costs them nothing, and what is set up per number of rows (the library's plans, when
            # the library is selected for the products: about 45 us of host time each) is set up for a few sizes only.
            padded = -(-n // _TOKEN_ROUNDING) * _TOKEN_ROUNDING if n > _TOKEN_ROUNDING and self.dtype == torch.bfloat16 else n
            lay = BatchLayout(padded, len(entries), m, self.cache.table_widths)
            ring, dev = self._staging(lay.size)
            host = ring.take()
            max_q, max_ctx = fill_batch(host.numpy(), lay, entries, self.cache, pad_to=padded if padded > n else 0,
                                        tokens=arrays)
            dev[: lay.size].copy_(host[: lay.size], non_blocking=True)
            ring.copied()
            ctx = self._context(dev, lay, max_q, max_ctx, decode_only, [len(e.tokens) for e in entries])
            if previous is not None:
                self.ops.take_tokens(ctx.token_ids, dev[lay.token_src : lay.token_src + lay.n], previous)
            logits = self.model.forward(ctx, self.cache.views)
        for e in entries:
            self.cache.advance(e.request, len(e.tokens))
        self.steps += 1
        return logits

    # ------------------------------------------------------------------ captured steps

    def capture_decode_graphs(self, most: Optional[int] = None) -> List[int]:
        """Captures the decode graphs for every batch-size bucket up to ``most`` requests (default: the engine's
        ``max_requests``) now, rather than when a batch of that size first comes; returns the buckets."""
        if not (self.config.cuda_graphs and self.device.type == "cuda"):
            return []
        most = self.config.max_requests if most is None else most
        top = next((b for b in _GRAPH_BUCKETS if b >= most), -(-most // 64) * 64)
        done = []
        for bucket in [b for b in _GRAPH_BUCKETS if b < top] + [top]:
            if bucket not in self._graphs:
                self._graphs[bucket] = _DecodeGraph(self, bucket)
            self._graphs[bucket].capture()
            done.append(bucket)
        return done

    def prepare_steps(self, most_tokens: int) -> List[int]:
        """Runs a step of padding only for every number of tokens that an eager bfloat16 step can be padded to, up
        to ``most_tokens``: whatever the kernels and the library behind the larger products set up per size (plans,
        heuristics, tensor maps, workspaces) is then in place before the first request. Pages and state are left
        alone. Returns the sizes."""
        if self.device.type != "cuda" or self.dtype != torch.bfloat16:
            return []
        sizes = list(range(2 * _TOKEN_ROUNDING, -(-most_tokens // _TOKEN_ROUNDING) * _TOKEN_ROUNDING + 1, _TOKEN_ROUNDING))
        for n in sizes:
            lay = BatchLayout(n, 1, 1, self.cache.table_widths)
            ring, dev = self._staging(lay.size)
            host = ring.take()
            fill_batch(host.numpy(), lay, [], self.cache, pad_to=n)
            host.numpy()[lay.logit_rows] = 0
            dev[: lay.size].copy_(host[: lay.size], non_blocking=True)
            ring.copied()
            ctx = self._context(dev, lay, n, self.config.context, False, [n])
            self.model.forward(ctx, self.cache.views)
        torch.cuda.synchronize(self.device)
        return sizes

    def _repeated_shape(self, entries):
        """A captured graph for steps whose requests bring exactly these numbers of tokens, once that shape has come
        _SHAPE_REPEATS times (the equal portions of a long prompt, a batch of prompts of one length); else None.
        At most _SHAPE_GRAPHS shapes are kept: each holds the activations of its step."""
        key = (tuple(len(e.tokens) for e in entries), sum(len(e.want) for e in entries))
        graph = self._shape_graphs.get(key)
        if graph is not None:
            return graph
        seen = self._shape_counts.get(key, 0) + 1
        self._shape_counts[key] = seen
        if len(self._shape_counts) > 4096:
            self._shape_counts.clear()
        if seen < _SHAPE_REPEATS or len(self._shape_graphs) >= _SHAPE_GRAPHS:
            return None
        graph = self._shape_graphs[key] = _DecodeGraph(self, 0, lengths=key[0], wanted=key[1])
        return graph

    def decode_capacity(self, count: int) -> int:
        """The number of rows that a step of ``count`` decoded tokens runs at: the bucket of its captured graph."""
        if not (self.config.cuda_graphs and self.device.type == "cuda"):
            return count
        return next((b for b in _GRAPH_BUCKETS if b >= count), -(-count // 64) * 64)

    def _decode_graph_step(self, entries, arrays=None, previous=None):
        count = len(entries)
        bucket = next((b for b in _GRAPH_BUCKETS if b >= count), -(-count // 64) * 64)
        graph = self._graphs.get(bucket)
        if graph is None:
            graph = self._graphs[bucket] = _DecodeGraph(self, bucket)
            # A batch shrinks as requests end: the smaller buckets are captured now, together, rather than each
            # in the middle of serving when it is first needed (a capture holds the device for tens of ms).
            for smaller in _GRAPH_BUCKETS:
                if smaller < bucket and smaller not in self._graphs:
                    self._graphs[smaller] = _DecodeGraph(self, smaller)
                    self._graphs[smaller].capture()
        return graph.run(entries, arrays, previous)


class _Pinned:
    """A ring of pinned int32 host buffers, each with the event of the last copy that read it."""

    def __init__(self, size: int, device, count: int = 4):
        self.cuda = device.type == "cuda"
        self.buffers = [torch.empty(size, dtype=torch.int32, pin_memory=self.cuda) for _ in range(count)]
        self.events = [None] * count
        self.at = -1

    def take(self) -> torch.Tensor:
        """The next buffer, once the copy that last read it has run."""
        self.at = (self.at + 1) % len(self.buffers)
        if self.events[self.at] is not None:
            self.events[self.at].synchronize()
        return self.buffers[self.at]

    def copied(self) -> None:
        """Call after enqueueing the copy out of the buffer that ``take`` gave last."""
        if self.cuda:
            event = self.events[self.at] or torch.cuda.Event()
            event.record()
            self.events[self.at] = event


class _DecodeGraph:
    """One captured step: a decode step for ``bucket`` requests of one token each, or (``lengths`` given) a step
    of requests that bring exactly these numbers of tokens, ``wanted`` logits rows in all.

    The batch arrays live at fixed addresses; a replay copies the step's arrays in
    and launches the graph. Requests short of the bucket are padding (request -1).
    Launch shapes inside depend on the bucket (or the lengths) only; positions, pages and slots are read on the device.
    """

    def __init__(self, runner: ModelRunner, bucket: int, lengths=None, wanted: int = 0):
        self.runner = runner
        self.bucket = bucket
        self.lengths = lengths
        cache = runner.cache
        if lengths is None:
            self.layout = BatchLayout(bucket, bucket, bucket, cache.table_widths)
        else:
            self.layout = BatchLayout(sum(lengths), len(lengths), wanted, cache.table_widths)
        self.ring = _Pinned(self.layout.size, runner.device)
        self.dev = torch.zeros(self.layout.size, dtype=torch.int32, device=runner.device)
        self.graph = None
        self.logits = None

    def _fill(self, entries, arrays=None):
        host = self.ring.take()
        lay = self.layout
        if self.lengths is None:
            fill_batch(host.numpy(), lay, entries, self.runner.cache, pad_to=self.bucket, tokens=arrays)
            host.numpy()[lay.logit_rows : lay.logit_rows + self.bucket] = np.arange(self.bucket, dtype=np.int32)
        elif entries:
            fill_batch(host.numpy(), lay, entries, self.runner.cache, tokens=arrays)
        else:  # all padding, for warm-up and capture
            fill_batch(host.numpy(), lay, [], self.runner.cache, pad_to=lay.n)
            host.numpy()[lay.logit_rows : lay.logit_rows + max(lay.m, 1)] = 0
        self.dev.copy_(host, non_blocking=True)
        self.ring.copied()

    def capture(self) -> None:
        runner = self.runner
        if self.graph is None:
            # Warm-up and capture run on a batch of padding only: they must leave pages and state alone.
            # The context's host-side sizes are upper bounds so that the captured launches fit every replay.
            self._fill([])
            if self.lengths is None:
                ctx = runner._context(self.dev, self.layout, 1, runner.config.context, True, [1] * self.bucket)
            else:
                ctx = runner._context(self.dev, self.layout, max(self.lengths), runner.config.context,
                                      all(n == 1 for n in self.lengths), self.lengths)
            ctx.memo["captured"] = True
            stream = torch.cuda.Stream(device=runner.device)
            stream.wait_stream(torch.cuda.current_stream(runner.device))
            with torch.cuda.stream(stream):
                for _ in range(2):  # warm up: library handles, heuristics and workspaces before capture
                    ctx.memo = {"captured": True}
                    runner.model.forward(ctx, runner.cache.views)
            torch.cuda.current_stream(runner.device).wait_stream(stream)
            torch.cuda.synchronize(runner.device)
            graph = torch.cuda.CUDAGraph()
            ctx.memo = {"captured": True}
            before = getattr(runner.ops, "launch_count", 0)
            with torch.cuda.graph(graph):
                self.logits = runner.model.forward(ctx, runner.cache.views)
            if self.lengths is None:
                runner.kernels_per_decode_step[self.bucket] = getattr(runner.ops, "launch_count", 0) - before
            self.graph = graph

    def run(self, entries, arrays=None, previous=None):
        runner = self.runner
        self.capture()
        self._fill(entries, arrays)
        if previous is not None:
            lay = self.layout
            runner.ops.take_tokens(self.dev[lay.token_ids : lay.token_ids + lay.n],
                                   self.dev[lay.token_src : lay.token_src + lay.n], previous)
        self.graph.replay()
        return self.logits[: len(entries)] if self.lengths is None else self.logits
