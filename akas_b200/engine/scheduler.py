"""Continuous admission, portions of prompts under a token budget, decoding, finishing and freeing.

The budgets carry the names and meanings of kreasof-ai/akas's scheduler
(src/akas/scheduling/scheduler.py:15-52, 112-194): each turn every decoding request gets one token,
and at most ``prefill_requests`` requests get a portion of their prompt, none more than
``prefill_chunk`` tokens, all together at most ``prefill_token_budget`` (default chunk x requests)
and at most ``decode_prefill_token_budget`` while any request decodes. Two things differ.
The reference launches decode and prefill separately in one turn; here both are one batch of one
step. And the reference reserves a whole context per slot, so it cannot run out of cache; here pages
are taken as tokens are written, so they can run out, and what happens then is decided:

* a request is admitted only while a slot is free and the free pages cover its first portion;
* a portion is shortened to the pages that are free (a request that can get none waits);
* when a decoding request needs a page and none is free, the most recently admitted request that
  holds cache is preempted: its pages and slot are given back, and it returns to the front of the
  waiting queue, to be recomputed from its prompt and the tokens it has generated so far. The
  oldest request is never preempted, so the engine always makes progress; a request that could not
  fit in the pool even alone is refused when it is submitted.

The scheduler never touches the device: it plans with the cache manager's host-side counts and
hands the batch to ``execute(entries, requests) -> tokens``.

One step ahead. Given ``launch(entries, requests, previous) -> handle`` and ``collect(handle) -> tokens`` instead,
a turn leaves its step in flight and the next turn reads it. While every running request decodes, the next turn
goes further: it launches the following decode step *before* it reads the tokens of the one in flight (each
entry names the place of its input token among those, and the step function takes it from the device), so the
host's work for a step (planning, batch arrays, bookkeeping of the tokens read) runs while the device computes.
What the host cannot know yet is only whether a request has just produced its end-of-sequence token; such a
request runs one step too many, whose result is dropped when it lands. Everything else (admission, portions of
prompts, preemption, a request that reaches its limit) is decided as before, after the step in flight has landed.
"""

from __future__ import annotations

from collections import deque
from queue import Empty, Queue
from threading import Event
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

from ..cache.manager import CacheManager, OutOfPages
from .batch import StepEntry
from .request import Request


# A request's first token and its last are published at once; in between, every fourth (the reference's rhythm).
_PUBLISH_EVERY = 4


class _Flight:
    """A step that was launched and whose sampled tokens have not been read: the requests it samples for, in
    order, what ``launch`` returned, and whether it was a step of single decoded tokens only."""

    __slots__ = ("requests", "handle", "decode_only")

    def __init__(self, requests, handle, decode_only):
        self.requests, self.handle, self.decode_only = requests, handle, decode_only


@dataclass(frozen=True)
class Budgets:
    """How much prompt work a turn may hold, under kreasof-ai/akas's option names: at most ``prefill_requests``
    requests get a portion, none longer than ``prefill_chunk``, ``prefill_token_budget`` tokens in all (default:
    chunk x requests), and no more than ``decode_prefill_token_budget`` beside decoding requests."""

    prefill_chunk: int = 2048
    prefill_requests: int = 32
    prefill_token_budget: Optional[int] = None
    decode_prefill_token_budget: Optional[int] = None

    def __post_init__(self):
        for field in ("prefill_chunk", "prefill_requests"):
            value = getattr(self, field)
            if type(value) is not int or value < 1:
                raise ValueError(f"{field} = {value!r}: a whole number of at least 1 is needed")
        for field in ("prefill_token_budget", "decode_prefill_token_budget"):
            value = getattr(self, field)
            if value is not None and (type(value) is not int or value < 1):
                raise ValueError(f"{field} = {value!r}: None (no limit of its own) or a whole number of at least 1")

    def prompt_tokens(self, beside_decoding: bool) -> int:
        """The prompt tokens one turn may run."""
        most = self.prefill_token_budget if self.prefill_token_budget is not None else self.prefill_chunk * self.prefill_requests
        if beside_decoding and self.decode_prefill_token_budget is not None:
            most = min(most, self.decode_prefill_token_budget)
        return most


_COUNTERS = ("tokens", "completed", "cancelled", "steps", "decode_rounds", "prefill_rounds", "decode_rows",
             "padded_decode_rows", "max_active", "prefill_tokens", "max_prefill_tokens_per_turn",
             "max_prefill_tokens_with_decoding", "max_tokens_per_step", "preemptions", "pages_in_use_max", "steps_ahead")


class Scheduler:
    def __init__(self, cache: CacheManager, execute: Callable, publish: Callable, *, prefill_chunk=2048,
                 prefill_requests=32, prefill_token_budget=None, decode_prefill_token_budget=None,
                 admit: Optional[Callable] = None, launch: Optional[Callable] = None,
                 collect: Optional[Callable] = None, capacity: Optional[Callable] = None):
        self.budgets = Budgets(prefill_chunk, prefill_requests, prefill_token_budget, decode_prefill_token_budget)
        if (launch is None) != (collect is None):
            raise ValueError("launch and collect come as a pair")
        self.cache = cache
        self.execute, self.launch, self.collect = execute, launch, collect
        self.publish = publish
        self.admit_request = admit or cache.admit
        self.capacity = capacity  # rows that a step of only decoded tokens runs at, for the statistics
        self.flight: Optional[_Flight] = None
        self.incoming: Queue = Queue()  # filled by submit() from any thread, emptied at the start of a turn
        self.pending: deque = deque()  # waiting for a slot and pages
        self.running: List[Request] = []  # hold cache, in order of admission
        self.stopped = Event()
        self.stats = {name: 0 for name in _COUNTERS}
        self.stats["capacity_counts"] = {}

    prefill_chunk = property(lambda self: self.budgets.prefill_chunk)
    prefill_requests = property(lambda self: self.budgets.prefill_requests)
    prefill_token_budget = property(lambda self: self.budgets.prefill_token_budget)
    decode_prefill_token_budget = property(lambda self: self.budgets.decode_prefill_token_budget)

    # ------------------------------------------------------------------ requests in and out

    def submit(self, request: Request) -> None:
        """Hands a request over (from any thread); the next turn sees it."""
        if self.stopped.is_set():
            raise RuntimeError("the scheduler has been stopped and takes no more requests")
        self.incoming.put(request)

    def _drain_inbox(self, wait: float = 0.0) -> None:
        """Moves what ``submit`` queued to the waiting line; with ``wait``, blocks that long for a first arrival."""
        try:
            if wait:
                self.pending.append(self.incoming.get(timeout=wait))
            while True:
                self.pending.append(self.incoming.get_nowait())
        except Empty:
            pass

    @property
    def prefilling(self) -> List[Request]:
        return [r for r in self.running if r.pending_tokens() > 1]

    @property
    def decoding(self) -> List[Request]:
        return [r for r in self.running if r.pending_tokens() == 1]

    def _release(self, request: Request) -> None:
        if request.slot is not None:
            self.cache.release(request.id)
            request.slot = None

    def _finish(self, request: Request, reason: str) -> None:
        self._release(request)
        request.finish_reason = reason
        self.stats["cancelled" if reason == "cancelled" else "completed"] += 1

    def _preempt(self, request: Request) -> None:
        """Gives back everything ``request`` holds; it will be recomputed from prompt + output."""
        self._release(request)
        request.offset = 0
        request.preemptions += 1
        self.running.remove(request)
        self.pending.appendleft(request)
        self.stats["preemptions"] += 1

    @staticmethod
    def _event(request: Request) -> tuple:
        """What ``publish`` gets for a request: the record layout of kreasof-ai/akas's stream events."""
        end = {"type": request.finish_reason, "length": request.limit} if request.finished else None
        counts = {"prompt_tokens": len(request.prompt), "completion_tokens": len(request.output), "finish_reason": end}
        return request, {"output_ids": list(request.output), "meta_info": counts}

    # ------------------------------------------------------------------ one turn

    def plan(self) -> List[tuple]:
        """Decides this turn's batch: [(request, number of tokens)], decoding requests first.

        Takes the pages the batch needs (so the step cannot run out), preempting if a decoding request
        would otherwise stall, and admits waiting requests into free slots.
        """
        cache = self.cache
        batch: List[tuple] = []
        # 1. every decoding request gets its token; make room by preempting the youngest if need be
        for request in list(self.decoding):
            if request not in self.running:
                continue  # preempted a moment ago
            while True:
                try:
                    cache.reserve(request.id, 1)
                    batch.append((request, 1))
                    break
                except OutOfPages as error:
                    victim = self.running[-1]
                    if victim is request and len(self.running) == 1:
                        raise RuntimeError("the page pool cannot hold a single request") from error
                    if victim is request:
                        # the youngest itself is the one that stalls: it waits, recomputed later
                        self._preempt(request)
                        break
                    batch = [(r, n) for r, n in batch if r is not victim]
                    self._preempt(victim)
        decoding_now = bool(batch)
        remaining = self.budgets.prompt_tokens(beside_decoding=decoding_now)
        selected = 0

        def portion(request) -> None:
            """Gives ``request`` the next portion of its prompt, shortened to the budget and the free pages."""
            nonlocal remaining, selected
            if selected >= self.prefill_requests or remaining <= 0:
                return
            count = min(self.prefill_chunk, remaining, request.pending_tokens(), cache.room(request.id))
            if count <= 0:
                return
            cache.reserve(request.id, count)
            batch.append((request, count))
            remaining -= count
            selected += 1

        # 2. portions of the prompts that are under way, oldest first
        for request in self.prefilling:
            portion(request)
        # 3. admission: a free slot, and free pages for a first portion; the admitted request starts at once
        while self.pending and cache.free_slots() > 0:
            request = self.pending[0]
            if request.cancelled.is_set():
                self.pending.popleft()
                self._finish(request, "cancelled")
                continue
            first = min(self.prefill_chunk, request.pending_tokens())
            if not cache.fits(first) and self.running:
                break  # wait until running requests finish and give pages back
            self.pending.popleft()
            request.slot = self.admit_request(request.id)
            self.running.append(request)
            portion(request)
        return batch

    def turn(self) -> bool:
        """One step of the engine. Returns whether anything is still waiting, running or in flight."""
        self._drain_inbox()
        for request in list(self.running):
            if request.cancelled.is_set():
                self.running.remove(request)
                self._finish(request, "cancelled")

        if self.flight is not None:
            ahead = self._plan_ahead()
            if ahead is not None:
                following = self._launch_ahead(ahead)
                self._land(self.flight)
                self.flight = following
                return True
            self._land(self.flight)
            self.flight = None

        batch = self.plan()
        self.stats["max_active"] = max(self.stats["max_active"], len(self.running))
        self.stats["pages_in_use_max"] = max(self.stats["pages_in_use_max"], self.cache.peak_pages)
        if not batch:
            if self.running and not self.pending:
                raise RuntimeError("running requests can make no progress: the page pool is too small")
            return bool(self.pending or self.running)

        entries, sampled = [], []
        for request, count in batch:
            tokens = request.tokens()[request.offset:request.offset + count]
            last = request.offset + count == len(request.prompt) + len(request.output)
            entries.append(StepEntry(request.id, tokens, (count - 1,) if last else ()))
            if last:
                sampled.append(request)
        decode_only = all(count == 1 for _, count in batch) and len(sampled) == len(batch)
        self._account(batch)
        if self.launch is not None:
            handle = self.launch(entries, sampled, None)
            for request, count in batch:
                request.offset += count
            for request in sampled:
                request.inflight += 1
            self.flight = _Flight(sampled, handle, decode_only)
            return True
        new_tokens = self.execute(entries, sampled)
        if len(new_tokens) != len(sampled):
            raise ValueError("missing generated request result")
        for request, count in batch:
            request.offset += count
        for request in sampled:
            request.inflight += 1
        self._take(sampled, new_tokens)
        return bool(self.pending or self.running)

    def _account(self, batch) -> None:
        decode_rows = sum(1 for r, n in batch if n == 1 and r.pending_tokens() == 1)
        prefill_tokens = sum(n for r, n in batch) - decode_rows
        st = self.stats
        st["steps"] += 1
        st["max_tokens_per_step"] = max(st["max_tokens_per_step"], decode_rows + prefill_tokens)
        if decode_rows:
            st["decode_rounds"] += 1
            st["decode_rows"] += decode_rows
            if not prefill_tokens and self.capacity is not None:
                capacity = self.capacity(decode_rows)
                st["padded_decode_rows"] += capacity - decode_rows
                st["capacity_counts"][str(capacity)] = st["capacity_counts"].get(str(capacity), 0) + 1
        if prefill_tokens:
            st["prefill_rounds"] += 1
            st["prefill_tokens"] += prefill_tokens
            st["max_prefill_tokens_per_turn"] = max(st["max_prefill_tokens_per_turn"], prefill_tokens)
            if decode_rows:
                st["max_prefill_tokens_with_decoding"] = max(st["max_prefill_tokens_with_decoding"], prefill_tokens)

    def _take(self, sampled: Sequence[Request], new_tokens: Sequence[int]) -> None:
        """Gives each request the token a step sampled for it; finishes and publishes."""
        st = self.stats
        events = []
        for request, token in zip(sampled, new_tokens):
            if request.finished:
                continue  # ended while the step was in flight: this token comes after its last
            request.inflight -= 1
            request.output.append(int(token))
            st["tokens"] += 1
            if request.eos_token_id is not None and int(token) == request.eos_token_id:
                reason = "stop"
            elif len(request.output) >= request.limit:
                reason = "length"
            else:
                reason = None
            if reason:
                self.running.remove(request)
                self._finish(request, reason)
            unpublished = len(request.output) - request.published
            if reason or request.published == 0 or unpublished >= _PUBLISH_EVERY:
                events.append(self._event(request))
                request.published = len(request.output)
        if events:
            self.publish(events)

    # ------------------------------------------------------------------ one step ahead

    def _land(self, flight: _Flight) -> None:
        new_tokens = self.collect(flight.handle)
        if len(new_tokens) != len(flight.requests):
            raise ValueError("missing generated request result")
        self._take(flight.requests, new_tokens)

    def _plan_ahead(self) -> Optional[List[Request]]:
        """The requests of the next decode step, if it can be launched before the step in flight has been read:
        the one in flight decodes only, nobody waits who could be admitted, every running request is in it with
        nothing but its coming token outstanding and no repetition penalty, and pages are free for all without
        preempting. Requests that
        reach their limit with the token in flight are left out. ``None``: plan in full after landing."""
        flight, cache = self.flight, self.cache
        if not flight.decode_only or (self.pending and cache.free_slots() > 0):
            return None
        members = {id(r) for r in flight.requests}
        ahead = []
        for request in self.running:
            if id(request) not in members or request.inflight != 1 or request.pending_tokens() != 1:
                return None
            if getattr(request, "repetition_penalty", 1.0) != 1.0:
                return None  # its penalty needs the token in flight on the host before the next one is sampled
            if len(request.output) + request.inflight < request.limit:
                ahead.append(request)
        if not ahead:
            return None
        need = [0] * len(cache.groups)
        for request in ahead:
            for group, pages in enumerate(cache.pages_needed(request.id, 1)):
                need[group] += pages
        if any(pages > cache.free_pages(group) for group, pages in enumerate(need)):
            return None
        return ahead

    def _launch_ahead(self, ahead: List[Request]) -> _Flight:
        place = {id(r): i for i, r in enumerate(self.flight.requests)}
        entries = []
        for request in ahead:
            self.cache.reserve(request.id, 1)
            entries.append(StepEntry(request.id, (0,), (0,), source=place[id(request)]))
        self._account([(request, 1) for request in ahead])
        handle = self.launch(entries, ahead, self.flight.handle)
        self.stats["steps_ahead"] += 1
        for request in ahead:
            request.offset += 1
            request.inflight += 1
        return _Flight(ahead, handle, True)

    def run(self) -> None:
        try:
            while not self.stopped.is_set():
                if not self.turn() and self.flight is None:
                    self._drain_inbox(wait=0.01)  # idle: sleep until something arrives
        finally:
            self.shutdown()

    def shutdown(self) -> None:
        if self.flight is not None:
            self.collect(self.flight.handle)  # wait for the step in flight; its tokens are dropped
            self.flight = None
        for request in list(self.running):
            self._finish(request, "cancelled")
        self.running.clear()
        self.pending.clear()
