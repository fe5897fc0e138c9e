"""Device time per kind of operation: a stand-in for an ops module that brackets every call with CUDA events.

kreasof-ai/akas attributes kernels to phases with CUDA events in a tool of its own (tools/cuda_profile.py:1-40).
Here the step function takes the module of its operations as an argument, so the attribution is a wrapper around
that module: ``ModelRunner(folder, config, ops=TimedOps(cuda_ops))`` runs the same kernels, and ``table()`` says
where the time of the steps since ``clear()`` went. Events serialise nothing, but a step that replays a captured
graph makes no calls to time: use ``cuda_graphs=False``.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Dict, List

import torch


class TimedOps:
    def __init__(self, ops):
        self._ops = ops
        self._events: Dict[str, List] = defaultdict(list)

    def __getattr__(self, name):
        value = getattr(self._ops, name)
        if not callable(value) or name.startswith("_") or name.endswith("_status") or name in ("require", "libraries_for"):
            return value

        def timed(*args, **kwargs):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                return value(*args, **kwargs)
            finally:
                end.record()
                self._events[name].append((start, end))

        return timed

    def chain_begin(self, num_tokens: int) -> bool:
        """Operations that join a chain launch together, later: there would be nothing to time per call."""
        return False

    def clear(self) -> None:
        torch.cuda.synchronize()
        self._events.clear()

    def table(self) -> List[dict]:
        """One row per operation, longest first: calls, milliseconds on the device, share of the total."""
        torch.cuda.synchronize()
        rows = [dict(op=name, calls=len(pairs), ms=sum(a.elapsed_time(b) for a, b in pairs))
                for name, pairs in self._events.items()]
        total = sum(row["ms"] for row in rows) or 1.0
        for row in rows:
            row["share"] = row["ms"] / total
        return sorted(rows, key=lambda row: -row["ms"])
