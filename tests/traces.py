"""Ways of cutting the same requests into steps, and helpers that run them and compare with the plain model.

A trace is a list of steps ``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [ids]}``: the format
``bin/trace_run`` reads. Every generator wants the logits of every token, so each way of cutting can be
compared, position by position, with one whole-sequence pass of the plain implementation.
"""

import random

import numpy as np
import torch


def whole(requests):
    """Each request alone, in one step."""
    return [
        dict(step=i, entries=[dict(id=rid, tokens=list(toks), want=list(range(len(toks))))], end=[rid])
        for i, (rid, toks) in enumerate(requests.items())
    ]


def tail_decoded(requests, tail=32):
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [head] + [1] * (len(toks) - head)
        at = 0
        for k in cuts:
            steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=list(toks[at:at + k]), want=list(range(k)))],
                              end=[rid] if at + k == len(toks) else []))
            at += k
    return steps


def portions(requests, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 17)):
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for n, (rid, toks) in enumerate(requests.items()):
        at, i = 0, n
        while at < len(toks):
            k = min(sizes[i % len(sizes)], len(toks) - at)
            i += 1
            steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=list(toks[at:at + k]), want=list(range(k)))],
                              end=[rid] if at + k == len(toks) else []))
            at += k
    return steps


def mixed(requests, prompt_lens, seed=0, live=4, page=64):
    """Up to ``live`` requests at a time: portions of some prompts beside single decoded tokens of others.

    ``prompt_lens[rid]`` tokens of a request are its prompt (fed in portions of random size, at least two
    tokens unless one is left), the rest is fed one token a step as if decoded; a request may sit a step out.
    Returns (steps, max_tokens): the second is the most tokens live requests hold at any time with each
    request rounded up to ``page``, so a pool of that size makes later requests reuse pages of earlier ones.
    """
    rng = random.Random(seed)
    waiting = list(requests.items())
    active = {}
    steps, peak = [], 0
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = [list(toks), 0]
        entries, ended = [], []
        for rid, (toks, at) in list(active.items()):
            if len(active) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            left_prompt = prompt_lens[rid] - at
            if left_prompt > 0:
                k = min(left_prompt, rng.choice((2, 3, 5, 8, 13, 21, 40)))
                if left_prompt - k == 1:
                    k += 1
            else:
                k = 1
            entries.append(dict(id=rid, tokens=toks[at:at + k], want=list(range(k))))
            active[rid][1] = at + k
            if at + k == len(toks):
                ended.append(rid)
        held = sum(-(-max(a[1], 1) // page) * page for a in active.values())
        peak = max(peak, held)
        if entries:
            steps.append(dict(step=len(steps), entries=entries, end=ended))
        for rid in ended:
            del active[rid]
    return steps, peak


def replay(runner, steps):
    """Feeds ``steps`` to a ModelRunner; returns {request: float32 array [len, vocab]} of every wanted row."""
    from akas_b200.engine.batch import StepEntry

    rows = {}
    for step in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        starts = {e["id"]: (runner.cache.length(e["id"]) if e["id"] in runner.cache else 0) for e in step["entries"]}
        logits = runner.step(entries).float().cpu().numpy()
        at = 0
        for e in step["entries"]:
            for w in e["want"]:
                rows.setdefault(e["id"], {})[starts[e["id"]] + w] = logits[at]
                at += 1
        for rid in step["end"]:
            runner.release(rid)
        runner.cache.check()
    return {rid: np.stack([r[p] for p in sorted(r)]) for rid, r in rows.items()}


def worst(got, want):
    """(largest |difference| / largest |reference| over rows, relative L2 error) between two logit arrays."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    scale = np.abs(want).max()
    return float(np.abs(got - want).max() / scale), float(np.linalg.norm(got - want) / np.linalg.norm(want))


def first_bad(got, want, tol):
    """Index of the first position whose error exceeds ``tol`` (relative to the largest reference value)."""
    scale = np.abs(np.asarray(want)).max()
    err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).max(axis=-1) / scale
    bad = np.nonzero(err > tol)[0]
    return int(bad[0]) if len(bad) else None
