"""From the logits of a step to one token per request: greedy, or temperature with top-k and top-p.

kreasof-ai/akas samples LFM2 greedily on the device, ties to the lowest id
(src/akas/ops/vocabulary/kernel.py:112-153). Softcap, repetition penalty, top-k, temperature and top-p follow the
stages of its one stochastic sampler, in its order (src/akas/ops/vocabulary/kernel.py:515-671): the uniform number
comes from the host, one per (request, generated index), so results do not depend on batch composition.
"""

from __future__ import annotations

from typing import List, Sequence

import torch


class Sampler:
    def __init__(self, ops, device, where: str = "device"):
        self.ops = ops
        self.device = device
        self.where = where  # "host": greedy choices are made by NumPy on logits read back from the device

    def sample(self, logits: torch.Tensor, requests: Sequence) -> List[int]:
        """``logits``: float32 [M, vocab], one row per request in order. Returns M token ids (host ints)."""
        if logits.shape[0] == 0:
            return []
        return self.launch(logits, requests).tolist()

    def launch(self, logits: torch.Tensor, requests: Sequence) -> torch.Tensor:
        """The same without waiting for the device: the M token ids as an int32 device tensor. The uniform number
        of a request is the one of the token it is about to generate, counting tokens that are still in flight."""
        if any(r.adjusts_logits for r in requests):
            window = max(1, max(len(r.recent()) for r in requests))
            history = torch.full((len(requests), window), -1, dtype=torch.int32)
            for row, r in enumerate(requests):
                recent = r.recent() if r.repetition_penalty != 1.0 else []
                if recent:
                    history[row, : len(recent)] = torch.tensor(recent, dtype=torch.int32)
            knobs = torch.tensor([[r.softcap, r.repetition_penalty] for r in requests], dtype=torch.float32).t().contiguous()
            knobs = knobs.to(self.device, non_blocking=True)
            logits = self.ops.adjust_logits(logits, knobs[0], knobs[1], history.to(self.device, non_blocking=True))
        if self.where == "host":
            if any(r.temperature > 0 for r in requests):
                raise ValueError("host sampling is greedy: a request asks for a temperature")
            import numpy as np

            picks = np.argmax(logits.detach().to("cpu", torch.float32).numpy(), axis=1).astype(np.int32)
            return torch.from_numpy(picks).to(self.device)
        if all(r.temperature <= 0 for r in requests):
            return self.ops.argmax(logits)
        params = torch.tensor(
            [[r.temperature, float(r.top_k), r.top_p, r.uniform() if r.temperature > 0 else 0.0] for r in requests],
            dtype=torch.float32,
        ).t().contiguous().to(self.device, non_blocking=True)
        top_k = params[1].to(torch.int32)
        return self.ops.sample(logits, params[0], top_k, params[2], params[3])
