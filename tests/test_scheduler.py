"""The scheduler's decisions, with a fake step function (no device).

The fake keeps, per request, a rolling hash of every token it was fed, in order; the token it "generates"
is a function of that hash. Outputs are therefore sensitive to order, to lost or repeated tokens and to a
wrong recomputation after a preemption, as the reference's FakeEngine is (tests/test_dense_scheduler.py:7-37).

Every test runs twice: with the plain ``execute`` callback, and with the ``launch`` / ``collect`` pair, where
the scheduler leaves a step in flight and, while all requests decode, launches the next one before it has read
the tokens of the last (the fake then takes those tokens from the handle of the step before, as the device does).
"""

import pytest

from akas_b200.cache import CacheManager
from akas_b200.engine.request import Request
from akas_b200.engine.scheduler import Scheduler
from akas_b200.parts import PagedKVSpec, StateSpec

VOCAB = 1000


class FakeModel:
    def __init__(self, page=4, tokens=64, requests=4, context=64):
        self.cache = CacheManager([PagedKVSpec(1, 16), StateSpec((2, 4))], page, tokens, requests, context, storage=False)
        self.hash = {}
        self.batches = []
        self.ahead = 0  # steps launched before the tokens of the step before them were read
        self.fail_at = None  # the number of the step that raises instead of running, once

    def admit(self, rid):
        self.hash[rid] = 7
        return self.cache.admit(rid)

    def launch(self, entries, requests, previous):
        self.ahead += previous is not None
        assert len(requests) == sum(1 for e in entries if e.want)
        return self.execute(entries, requests, previous)

    @staticmethod
    def collect(handle):
        return list(handle)

    def execute(self, entries, requests, previous=None):
        if self.fail_at is not None and len(self.batches) == self.fail_at:
            self.fail_at = None
            raise RuntimeError("launch failed")
        self.batches.append([(e.request, len(e.tokens)) for e in entries])
        out = []
        for e in entries:
            assert len(e.tokens) > 0
            self.cache.reserve(e.request, len(e.tokens))  # must already be covered by the plan
            tokens = e.tokens
            if e.source >= 0:  # the token that the step before sampled and the host has not seen
                assert len(tokens) == 1 and previous is not None
                tokens = [previous[e.source]]
            for t in tokens:
                self.hash[e.request] = (self.hash[e.request] * 31 + t + 1) % 1000003
            self.cache.advance(e.request, len(e.tokens))
            if e.want:
                assert list(e.want) == [len(e.tokens) - 1]
                out.append(self.hash[e.request] % VOCAB)
        self.cache.check()
        return out


def expected(prompt, n):
    h, out = 7, []
    for t in prompt:
        h = (h * 31 + t + 1) % 1000003
    for _ in range(n):
        out.append(h % VOCAB)
        h = (h * 31 + out[-1] + 1) % 1000003
    return out


MODE = "sync"


@pytest.fixture(params=["sync", "ahead"], autouse=True)
def mode(request):
    global MODE
    MODE = request.param
    yield request.param
    MODE = "sync"


def make(model, **kw):
    events = []
    if MODE == "ahead":
        kw.update(launch=model.launch, collect=model.collect)
    s = Scheduler(model.cache, model.execute, events.extend, admit=model.admit, **kw)
    return s, events


def drain(s, limit=10000):
    turns = 0
    while s.turn():
        turns += 1
        assert turns < limit
    return turns


def test_batched_equals_sequential():
    model = FakeModel(tokens=256, requests=4)
    s, _ = make(model, prefill_chunk=5, prefill_requests=2)
    reqs = [Request([i + 1] * n, 6) for i, n in enumerate((3, 11, 1, 8, 20, 2))]
    for r in reqs:
        s.submit(r)
    drain(s)
    for r in reqs:
        assert r.output == expected(r.prompt, 6) and r.finish_reason == "length" and r.slot is None
    assert not model.cache.live() and model.cache.free_pages() == 64
    assert s.stats["completed"] == 6 and s.stats["tokens"] == 36 and s.stats["max_active"] == 4
    # prompt portions and decoded tokens did share steps
    assert any(any(n == 1 for _, n in b) and any(n > 1 for _, n in b) for b in model.batches)


def test_budgets_are_kept():
    model = FakeModel(tokens=4096, requests=8, context=512)
    s, _ = make(model, prefill_chunk=16, prefill_requests=3, prefill_token_budget=40, decode_prefill_token_budget=8)
    reqs = [Request([1] * 100, 4) for _ in range(6)]
    for r in reqs:
        s.submit(r)
    drain(s)
    assert all(r.output == expected(r.prompt, 4) for r in reqs)
    for batch in model.batches:
        portions = [n for _, n in batch if n > 1]
        decodes = [n for _, n in batch if n == 1]
        assert all(n <= 16 for n in portions) and len(portions) <= 3 and sum(portions) <= 40
    st = s.stats
    assert st["max_prefill_tokens_per_turn"] <= 40 and st["max_prefill_tokens_with_decoding"] <= 8
    assert 594 <= st["prefill_tokens"] <= 600  # every prompt token ran once (a last single token counts as decoding)


def test_default_budget_is_chunk_times_requests():
    model = FakeModel(tokens=4096, requests=8, context=512)
    s, _ = make(model, prefill_chunk=10, prefill_requests=2)
    for _ in range(4):
        s.submit(Request([1] * 50, 2))
    s.turn()
    assert sorted(n for _, n in model.batches[0]) == [10, 10]


def test_cancel_frees_and_others_go_on():
    model = FakeModel(tokens=256)
    s, _ = make(model, prefill_chunk=4)
    a, b = Request([1] * 10, 50), Request([2] * 3, 5)
    s.submit(a), s.submit(b)
    for _ in range(4):
        s.turn()
    a.cancelled.set()
    drain(s)
    assert a.finish_reason == "cancelled" and b.output == expected(b.prompt, 5)
    assert s.stats["cancelled"] == 1 and not model.cache.live()
    c = Request([3], 2)
    c.cancelled.set()
    s.submit(c)
    drain(s)
    assert c.finish_reason == "cancelled" and c.output == []


def test_end_of_sequence_token_stops_a_request():
    model = FakeModel(tokens=256)
    s, _ = make(model)
    want = expected([5, 6], 10)
    r = Request([5, 6], 10, eos_token_id=want[3])
    s.submit(r)
    drain(s)
    assert r.output == want[:4] and r.finish_reason == "stop"


def test_pages_run_out_the_youngest_is_preempted_and_recomputed():
    # 10 pages of 4 tokens; three requests that each grow to 24 tokens cannot all stay
    model = FakeModel(page=4, tokens=40, requests=3, context=40)
    s, _ = make(model, prefill_chunk=8)
    reqs = [Request([i + 1] * 6, 18) for i in range(3)]
    for r in reqs:
        s.submit(r)
    drain(s)
    assert s.stats["preemptions"] > 0
    for r in reqs:
        assert r.output == expected(r.prompt, 18), "a preempted request must be recomputed, not resumed from stale state"
    assert reqs[0].preemptions == 0, "the oldest request is never preempted"
    assert not model.cache.live() and model.cache.free_pages() == 10 and s.stats["pages_in_use_max"] <= 10


def test_admission_waits_for_pages():
    model = FakeModel(page=4, tokens=16, requests=4, context=16)
    s, _ = make(model, prefill_chunk=16)
    a, b = Request([1] * 12, 2), Request([2] * 12, 2)
    s.submit(a), s.submit(b)
    s.turn()
    assert [r for r, _ in model.batches[0]] == [a.id]  # b's first portion has no pages yet
    drain(s)
    assert a.output == expected(a.prompt, 2) and b.output == expected(b.prompt, 2)


def test_a_portion_is_shortened_to_the_free_pages():
    model = FakeModel(page=4, tokens=32, requests=2, context=32)
    s, _ = make(model, prefill_chunk=32)
    a, b = Request([1] * 20, 1), Request([2] * 5, 8)
    s.submit(b)
    s.turn()
    s.submit(a)
    s.turn()  # b holds 2 pages; 6 are free: a's first portion is 24 at most, it wants 20
    assert (a.id, 20) in model.batches[1]
    drain(s)
    assert a.output == expected(a.prompt, 1) and b.output == expected(b.prompt, 8)


def test_events_carry_ids_and_reasons():
    model = FakeModel(tokens=256)
    s, events = make(model)
    r = Request([1, 2, 3], 6)
    s.submit(r)
    drain(s)
    assert [len(e[1]["output_ids"]) for e in events] == [1, 5, 6]  # first token, a group of four, the end
    last = events[-1][1]
    assert last["meta_info"] == dict(prompt_tokens=3, completion_tokens=6, finish_reason=dict(type="length", length=6))
    assert events[0][1]["meta_info"]["finish_reason"] is None


def test_invalid_budgets():
    model = FakeModel()
    with pytest.raises(ValueError):
        make(model, prefill_chunk=0)
    with pytest.raises(ValueError):
        make(model, prefill_token_budget=0)
    s, _ = make(model)
    s.stopped.set()
    with pytest.raises(RuntimeError):
        s.submit(Request([1], 1))


def test_decoding_runs_a_step_ahead(mode):
    """With launch / collect, steady decoding launches each step before the one before it has been read; a request
    that meets its end-of-sequence token has then run one step too many, which is dropped."""
    model = FakeModel(tokens=256, requests=4)
    s, _ = make(model, prefill_chunk=8)
    stop = expected([9, 9, 9], 12)
    reqs = [Request([i + 1] * n, 12) for i, n in enumerate((5, 2, 7))] + [Request([9, 9, 9], 12, eos_token_id=stop[5])]
    for r in reqs:
        s.submit(r)
    drain(s)
    for r in reqs[:3]:
        assert r.output == expected(r.prompt, 12) and r.finish_reason == "length"
    assert reqs[3].output == stop[:6] and reqs[3].finish_reason == "stop"
    assert not model.cache.live() and s.flight is None
    assert all(r.inflight == 0 for r in reqs[:3])
    if mode == "ahead":
        assert model.ahead >= 8  # most decode steps were launched ahead
        decodes = [b for b in model.batches if all(n == 1 for _, n in b)]
        assert sum(1 for b in decodes for rid, _ in b if rid == reqs[3].id) == 6  # five inputs and the dropped step
    else:
        assert model.ahead == 0


def test_a_late_arrival_is_admitted_between_steps_ahead(mode):
    model = FakeModel(tokens=256, requests=2)
    s, _ = make(model, prefill_chunk=4)
    a, b, c = Request([1] * 6, 20), Request([2] * 3, 4), Request([3] * 9, 5)
    s.submit(a), s.submit(b)
    for _ in range(6):
        s.turn()
    s.submit(c)  # no slot is free until b ends
    drain(s)
    assert a.output == expected(a.prompt, 20) and b.output == expected(b.prompt, 4) and c.output == expected(c.prompt, 5)
    assert not model.cache.live()


def test_the_rows_a_decode_step_is_padded_to_are_counted():
    model = FakeModel(tokens=256, requests=4)
    s, _ = make(model, capacity=lambda rows: 1 << (rows - 1).bit_length())
    reqs = [Request([i + 1] * 3, n) for i, n in enumerate((6, 6, 6, 2))]
    for r in reqs:
        s.submit(r)
    drain(s)
    st = s.stats
    decode_only = [b for b in model.batches if all(n == 1 for _, n in b)]
    assert sum(st["capacity_counts"].values()) == len(decode_only)
    assert st["capacity_counts"] == {"4": sum(1 for b in decode_only if len(b) in (3, 4)),
                                     **({"2": n} if (n := sum(1 for b in decode_only if len(b) == 2)) else {}),
                                     **({"1": n} if (n := sum(1 for b in decode_only if len(b) == 1)) else {})}
    assert st["padded_decode_rows"] == sum(1 for b in decode_only if len(b) == 3)


@pytest.mark.parametrize("fail_at", [0, 1, 3, 6])
def test_a_failed_step_is_raised_and_leaves_the_requests_where_they_were(fail_at):
    """The reference puts the selected requests back in order and re-raises (src/akas/scheduling/scheduler.py:170-173).
    Here nothing was taken out: the step after the failure plans the same tokens again."""
    model = FakeModel(tokens=256, requests=4)
    model.fail_at = fail_at
    s, _ = make(model, prefill_chunk=4, prefill_requests=2)
    reqs = [Request([i + 1] * n, 5) for i, n in enumerate((3, 9, 6))]
    for r in reqs:
        s.submit(r)
    raised = 0
    for _ in range(1000):
        try:
            if not s.turn():
                break
        except RuntimeError as error:
            assert "launch failed" in str(error)
            raised += 1
    assert raised == 1
    for r in reqs:
        assert r.output == expected(r.prompt, 5) and r.finish_reason == "length"
    assert not model.cache.live() and model.cache.free_pages() == 64
    model.cache.check()


def test_a_repetition_penalty_keeps_the_host_in_step():
    """The penalty of a request looks at the tokens it has generated: the step after cannot be launched before the
    token in flight is on the host."""
    model = FakeModel(tokens=256, requests=4)
    s, _ = make(model)
    reqs = [Request([i + 1] * 3, 6) for i in range(2)]
    reqs[1].repetition_penalty = 1.3
    for r in reqs:
        s.submit(r)
    drain(s)
    assert model.ahead == 0 and s.stats["steps_ahead"] == 0
    assert all(r.output == expected(r.prompt, 6) for r in reqs)


@pytest.mark.parametrize("seed", range(6))
def test_random_arrivals_cancellations_and_a_small_pool(seed):
    """Requests of random lengths arrive at random turns into a pool that cannot hold them all, some are cancelled on
    the way: whatever the order, every request that was not cancelled generates what it would have generated alone,
    the cache's books balance after every turn, and everything is given back at the end."""
    import random

    rng = random.Random(seed)
    model = FakeModel(page=4, tokens=96, requests=4, context=64)
    s, events = make(model, prefill_chunk=rng.choice([3, 7, 16]), prefill_requests=rng.choice([1, 2, 4]),
                     decode_prefill_token_budget=rng.choice([None, 5]))
    waiting = [Request([rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))], rng.randint(1, 12)) for _ in range(14)]
    submitted, cancelled = [], set()
    for turn in range(10000):
        while waiting and rng.random() < 0.4:
            submitted.append(waiting.pop())
            s.submit(submitted[-1])
        if submitted and rng.random() < 0.05:
            victim = rng.choice(submitted)
            if not victim.finished:
                victim.cancelled.set()
                cancelled.add(victim.id)
        busy = s.turn()
        model.cache.check()
        if not busy and not waiting:
            break
    else:
        raise AssertionError("the scheduler did not finish")
    assert len(submitted) == 14
    for r in submitted:
        if r.finish_reason == "cancelled":
            assert r.id in cancelled and r.output == expected(r.prompt, len(r.output))
        else:
            assert r.finish_reason == "length" and r.output == expected(r.prompt, r.limit)
        assert r.slot is None
    assert not model.cache.live() and model.cache.free_pages() == 24
    assert s.stats["completed"] + s.stats["cancelled"] == 14
