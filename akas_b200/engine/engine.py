"""The request API: submit token ids, step the engine, read what it generated.

``Engine`` has the surface of kreasof-ai/akas's engine (src/akas/engine.py:10-110): ``submit(prompt,
max_tokens=)`` returns a ``Request`` whose ``output`` grows, ``step()`` runs one scheduler turn and says
whether work is left, ``cancel``, ``run``, ``close``; requests are validated at submission; the engine
runs on the thread that made it. ``generate`` is the Python entry point for whole batches of prompts:
host token ids in, host token ids out.
"""

from __future__ import annotations

from collections import deque
from dataclasses import replace
from threading import get_ident
from typing import List, Optional, Sequence

import torch

from ..config.engine import EngineConfig
from ..sampling.sampler import Sampler
from .request import Request
from .runner import ModelRunner
from .scheduler import Scheduler


class _Sampled:
    """The tokens a launched step sampled: on the device (the next step may take its inputs from there), and on
    their way to pinned host memory by a copy on a stream of its own. A copy on the step's stream would queue
    behind whatever was launched after the step, and reading it would wait for that too."""

    def __init__(self, tokens: torch.Tensor, copy_stream, host: Optional[torch.Tensor] = None):
        self.tokens = tokens
        if tokens.device.type != "cuda":
            self.host, self.done = tokens, None
            return
        self.host = host[: tokens.numel()] if host is not None else torch.empty(tokens.shape, dtype=tokens.dtype, pin_memory=True)
        ready = torch.cuda.Event()
        ready.record()
        copy_stream.wait_event(ready)
        with torch.cuda.stream(copy_stream):
            self.host.copy_(tokens, non_blocking=True)
            self.done = torch.cuda.Event()
            self.done.record()
        tokens.record_stream(copy_stream)

    def read(self) -> List[int]:
        if self.done is not None:
            self.done.synchronize()
        return self.host.tolist()


def _check_sampling(temperature, top_k, top_p, softcap, repetition_penalty, repetition_window, greedy_only=False):
    """Refuses sampling options outside their ranges, naming each one that is."""
    faults = []
    if temperature < 0:
        faults.append(f"temperature = {temperature} is negative (0 is greedy)")
    if top_k < 0:
        faults.append(f"top_k = {top_k} is negative (0 keeps every token)")
    if not 0.0 < top_p <= 1.0:
        faults.append(f"top_p = {top_p} is outside (0, 1]")
    if softcap < 0:
        faults.append(f"softcap = {softcap} is negative (0 is none)")
    if repetition_penalty <= 0:
        faults.append(f"repetition_penalty = {repetition_penalty} is not positive (1 is none)")
    if repetition_window < 0:
        faults.append(f"repetition_window = {repetition_window} is negative")
    if greedy_only and temperature > 0:
        faults.append("host sampling is greedy, and the request asks for a temperature")
    if faults:
        raise ValueError("; ".join(faults))


class Engine:
    def __init__(self, model, *, config: Optional[EngineConfig] = None, publish=None, ops=None):
        """``model``: a model folder (config.json + model.safetensors), or a ready ``ModelRunner``."""
        self.thread = get_ident()
        if isinstance(model, ModelRunner):
            self.runner = model
            self.config = model.config
        else:
            self.config = config or EngineConfig()
            self.runner = ModelRunner(model, self.config, ops=ops)
        self.sampler = Sampler(self.runner.ops, self.runner.device, self.config.sampling)
        on_gpu = self.runner.device.type == "cuda"
        self._copy_stream = torch.cuda.Stream(self.runner.device) if on_gpu else None
        self._token_buffers = [torch.empty(max(self.config.max_requests, 1), dtype=torch.int32, pin_memory=True)
                               for _ in range(4)] if on_gpu else []
        self._token_turn = 0
        self.events = deque()
        self.closed = False
        self.scheduler = Scheduler(
            self.runner.cache,
            self._execute,
            publish if publish is not None else self.events.extend,
            prefill_chunk=self.config.prefill_chunk,
            prefill_requests=self.config.prefill_requests,
            prefill_token_budget=self.config.prefill_token_budget,
            decode_prefill_token_budget=self.config.decode_prefill_token_budget,
            admit=self.runner.admit,
            launch=self._launch if self.config.run_ahead else None,
            collect=self._collect if self.config.run_ahead else None,
            capacity=self.runner.decode_capacity,
        )

    @classmethod
    def from_checkpoint(cls, checkpoint, *, config: Optional[EngineConfig] = None, publish=None, **options):
        """Loads the model folder ``checkpoint``; ``options`` override fields of ``config``."""
        config = replace(config or EngineConfig(), **options)
        return cls(checkpoint, config=config, publish=publish)

    # ------------------------------------------------------------------ properties of the model

    @property
    def context(self) -> int:
        return min(self.config.context, self.runner.cache.capacity_tokens())

    @property
    def capacity(self) -> int:
        return self.config.max_requests

    @property
    def stats(self) -> dict:
        return self.scheduler.stats

    # ------------------------------------------------------------------ requests

    def submit(self, prompt, *, max_tokens, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
               seed: Optional[int] = None, eos_token_id: Optional[int] = None, softcap: float = 0.0,
               repetition_penalty: float = 1.0, repetition_window: int = 96) -> Request:
        """Queues a request for the next turn (any thread may). Everything that could make a later step fail is refused here, with
        the place of the fault in the message: the step function trusts what the scheduler hands it."""
        tokens = list(prompt)
        if not tokens:
            raise ValueError("an empty prompt: a request needs at least one token id")
        vocab = self.runner.vocab_size
        for place, token in enumerate(tokens):
            if type(token) is not int or not 0 <= token < vocab:
                raise ValueError(f"prompt[{place}] = {token!r} is not a token id (an int in [0, {vocab}))")
        if type(max_tokens) is not int or max_tokens <= 0:
            raise ValueError(f"max_tokens = {max_tokens!r}: a request generates a whole number of tokens, at least one")
        room = self.context - len(tokens)
        if max_tokens > room:
            raise ValueError(f"{len(tokens)} prompt tokens and {max_tokens} to generate do not fit the context "
                             f"of {self.context} tokens (room for {max(room, 0)})")
        _check_sampling(temperature, top_k, top_p, softcap, repetition_penalty, repetition_window,
                        greedy_only=self.config.sampling == "host")
        request = Request(tokens, max_tokens, temperature=float(temperature), top_k=int(top_k), top_p=float(top_p),
                          seed=seed, eos_token_id=eos_token_id, softcap=float(softcap),
                          repetition_penalty=float(repetition_penalty), repetition_window=int(repetition_window))
        self.scheduler.submit(request)
        return request

    def warm_up(self, most: Optional[int] = None, tokens: Optional[int] = None) -> None:
        """Compiles, loads and captures what serving will need, so that the first requests do not pay for it: the
        decode graphs of every batch size up to ``most`` requests (default ``max_requests``), and a step of padding
        for every size a step of prompt portions can have, up to ``tokens`` (default: the prefill token budget plus
        one decoded token per request)."""
        self._owner_only("warm_up")
        self.runner.capture_decode_graphs(most)
        if tokens is None:
            budget = self.config.prefill_token_budget or self.config.prefill_chunk * self.config.prefill_requests
            tokens = budget + self.config.max_requests
        self.runner.prepare_steps(tokens)

    def _execute(self, entries, requests) -> List[int]:
        logits = self.runner.step(entries)
        return self.sampler.sample(logits, requests)

    def _launch(self, entries, requests, previous=None):
        """A step without waiting for it: the sampled tokens stay on the device (``_collect`` reads them).
        ``previous``: what ``_launch`` returned for the step before, for entries that take their token from it."""
        logits = self.runner.step(entries, previous=None if previous is None else previous.tokens)
        if not len(requests):
            return None
        # pinned buffers are taken in turn; at most two steps' tokens are unread at any time
        self._token_turn = (self._token_turn + 1) % len(self._token_buffers) if self._token_buffers else 0
        host = self._token_buffers[self._token_turn] if self._token_buffers else None
        if host is not None and host.numel() < len(requests):
            host = None
        return _Sampled(self.sampler.launch(logits, requests), self._copy_stream, host)

    @staticmethod
    def _collect(handle) -> List[int]:
        return [] if handle is None else handle.read()

    def _owner_only(self, what: str) -> None:
        """The cache manager, the staging ring and the captured graphs are not locked: one thread drives them."""
        if get_ident() != self.thread:
            raise RuntimeError(f"Engine.{what}() was called from another thread than the one that built the engine")

    def step(self) -> bool:
        """One scheduler turn; whether anything is still waiting, running or in flight."""
        self._owner_only("step")
        if self.closed:
            raise RuntimeError("Engine.step() after close()")
        return self.scheduler.turn()

    def cancel(self, request: Request) -> None:
        """Marks ``request`` (any thread may); the next turn gives back what it holds."""
        request.cancelled.set()

    def run(self) -> None:
        """Serves until ``scheduler.stopped`` is set (from any thread), then closes."""
        self._owner_only("run")
        with self:
            self.scheduler.run()

    def close(self) -> None:
        """Stops the scheduler, waits for the step in flight and frees every request's pages and slot. Idempotent."""
        self._owner_only("close")
        if not self.closed:
            self.closed = True
            self.scheduler.stopped.set()
            self.scheduler.shutdown()

    def __enter__(self):
        return self

    def __exit__(self, kind, error, trace):
        self.close()

    # ------------------------------------------------------------------ whole batches

    def generate(self, prompts: Sequence[Sequence[int]], *, max_tokens: int = 128, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None,
                 eos_token_id: Optional[int] = None, softcap: float = 0.0, repetition_penalty: float = 1.0,
                 repetition_window: int = 96) -> List[dict]:
        """Generates for every prompt (token ids) and returns, per prompt, what the reference's
        ``generate`` returns (src/akas/generation/greedy.py:110-114): ``prompt_tokens``,
        ``generated_tokens`` and ``text`` (``None``: this engine holds no tokenizer), plus ``finish_reason``.
        A single prompt may be given as a flat list of ids."""
        single = bool(prompts) and isinstance(prompts[0], int)
        batch = [prompts] if single else list(prompts)
        requests = [
            self.submit(p, max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                        seed=None if seed is None else seed + i, eos_token_id=eos_token_id, softcap=softcap,
                        repetition_penalty=repetition_penalty, repetition_window=repetition_window)
            for i, p in enumerate(batch)
        ]
        while self.step():
            pass
        self.events.clear()
        results = [
            dict(prompt_tokens=list(r.prompt), generated_tokens=list(r.output), text=None,
                 finish_reason=r.finish_reason)
            for r in requests
        ]
        return results[0] if single else results
