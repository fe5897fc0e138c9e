"""Generation through the entry point, long decoding through captured graphs, the first tokens of a
sequence, sampling that does not depend on the batch, and bin/trace_run as a user runs it."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
import tiny
import traces

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 2e-5, "bfloat16": 2e-2}  # of the largest logit; bfloat16 measures 1.3e-2 at most


def _engine(folder, dtype, page, **kw):
    from akas_b200 import Engine, EngineConfig

    options = dict(dtype=dtype, device="cuda:0", page_size=page, max_requests=4, context=512, max_tokens=2048)
    options.update(kw)
    return Engine(str(folder), config=EngineConfig(**options))


@pytest.mark.parametrize("key", ["a", "b"])
def test_greedy_generation_equals_plain_recomputation(key, tmp_path):
    folder = tiny.make_folder(tiny.CONFIGS[key], seed=21, dtype="float32", folder=tmp_path / key)
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(cfg["vocab_size"], [1, 7, 40, 23, 64, 3], seed=2)
    with _engine(folder, "float32", tiny.PAGE[key], prefill_chunk=13, prefill_requests=2) as engine:
        results = engine.generate(prompts, max_tokens=12)
        stats = dict(engine.stats)
    for prompt, result in zip(prompts, results):
        assert result["prompt_tokens"] == prompt and result["finish_reason"] == "length"
        assert result["generated_tokens"] == plain.greedy(cfg, w, prompt, 12)
    assert stats["completed"] == 6 and stats["max_active"] == 4 and stats["max_prefill_tokens_with_decoding"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_graphs(dtype, tmp_path):
    """300 decoded tokens for three requests of different lengths (graph replay, bucket of 4 with one row of
    padding): the logits of every step against one whole pass of the plain model over the final sequences."""
    from akas_b200 import StepEntry

    folder = tiny.make_folder(tiny.TINY_A, seed=22, dtype=dtype, folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(cfg["vocab_size"], [5, 70, 33], seed=3)
    feed = tiny.prompts(cfg["vocab_size"], [300, 300, 300], seed=4)
    with _engine(folder, dtype, 16) as engine:
        runner = engine.runner
        runner.step([StepEntry(i, p, ()) for i, p in enumerate(prompts)])
        rows = [[] for _ in prompts]
        for t in range(300):
            logits = runner.step([StepEntry(i, (feed[i][t],), (0,)) for i in range(3)]).float().cpu().numpy()
            for i in range(3):
                rows[i].append(logits[i])
        assert 4 in runner._graphs and runner.kernels_per_decode_step[4] > 0
    for i, p in enumerate(prompts):
        want = plain.forward(cfg, w, p + feed[i]).numpy()[len(p):]
        bad = traces.first_bad(np.stack(rows[i]), want, TOL[dtype])
        assert bad is None, (i, bad, traces.worst(np.stack(rows[i]), want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype, tmp_path):
    """Positions 0, 1, 2: empty state, a cache of one page, a single key."""
    from akas_b200 import StepEntry

    folder = tiny.make_folder(tiny.TINY_B, seed=23, dtype=dtype, folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    with _engine(folder, dtype, 8) as engine:
        for prompt in ([5], [5, 5], [300, 0, 319]):
            want = plain.forward(cfg, w, prompt).numpy()
            got = engine.runner.step([StepEntry("x", prompt, range(len(prompt)))]).float().cpu().numpy()
            engine.runner.release("x")
            one = np.concatenate([engine.runner.step([StepEntry("y", (t,), (0,))]).float().cpu().numpy() for t in prompt])
            engine.runner.release("y")
            assert traces.first_bad(got, want, TOL[dtype]) is None and traces.first_bad(one, want, TOL[dtype]) is None


def test_sampling_does_not_depend_on_the_batch(tmp_path):
    folder = tiny.make_folder(tiny.TINY_A, seed=24, dtype="float32", std=0.3, folder=tmp_path / "m")
    prompts = tiny.prompts(256, [9, 30, 2, 17], seed=5)
    with _engine(folder, "float32", 16) as engine:
        together = engine.generate(prompts, max_tokens=20, temperature=0.9, top_k=40, top_p=0.95, seed=100)
        alone = [engine.generate(p, max_tokens=20, temperature=0.9, top_k=40, top_p=0.95, seed=100 + i)
                 for i, p in enumerate(prompts)]
        again = engine.generate(prompts, max_tokens=20, temperature=0.9, top_k=40, top_p=0.95, seed=101)
    assert [r["generated_tokens"] for r in together] == [r["generated_tokens"] for r in alone]
    assert [r["generated_tokens"] for r in together] != [r["generated_tokens"] for r in again]
    assert len({tuple(r["generated_tokens"]) for r in together}) == 4


def test_a_step_ahead_changes_nothing(tmp_path):
    """The engine that launches each decode step before it has read the last one's tokens (they go from step to step
    on the device) generates what the engine that waits for every step generates: greedy and sampled, with requests
    that stop at an end-of-sequence token in mid-flight, with and without captured graphs."""
    folder = tiny.make_folder(tiny.TINY_B, seed=27, dtype="float32", std=0.3, folder=tmp_path / "m")
    prompts = tiny.prompts(tiny.TINY_B["vocab_size"], [9, 30, 2, 17], seed=8)
    runs = {}
    for ahead in (False, True):
        for graphs in (True, False):
            with _engine(folder, "float32", 8, run_ahead=ahead, cuda_graphs=graphs) as engine:
                greedy = engine.generate(prompts, max_tokens=24)
                stop = greedy[1]["generated_tokens"][7]  # request 1 meets this token at its 8th place at the latest
                stopped = engine.generate(prompts, max_tokens=24, eos_token_id=stop)
                sampled = engine.generate(prompts, max_tokens=24, temperature=0.8, top_k=50, top_p=0.9, seed=3)
                runs[ahead, graphs] = [[r["generated_tokens"] for r in out] for out in (greedy, stopped, sampled)]
                reasons = [r["finish_reason"] for r in stopped]
                if ahead:
                    assert engine.stats["steps_ahead"] > 30
                else:
                    assert engine.stats["steps_ahead"] == 0
            assert reasons[1] == "stop" and len(runs[ahead, graphs][1][1]) <= 8
    assert runs[True, True] == runs[False, True] == runs[True, False] == runs[False, False]


def test_warm_up_captures_every_bucket_and_changes_nothing(tmp_path):
    folder = tiny.make_folder(tiny.TINY_A, seed=28, dtype="float32", folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(256, [12, 3, 25], seed=9)
    with _engine(folder, "float32", 16, max_requests=6) as engine:
        engine.warm_up()
        graphs = engine.runner._graphs
        assert sorted(graphs) == [1, 2, 4, 8] and all(g.graph is not None for g in graphs.values())
        results = engine.generate(prompts, max_tokens=10)
    for prompt, result in zip(prompts, results):
        assert result["generated_tokens"] == plain.greedy(cfg, w, prompt, 10)


def test_preemption_on_the_device_recomputes_exactly(tmp_path):
    """A pool too small for three growing requests: the youngest is preempted and recomputed; every output
    still equals the plain greedy continuation."""
    folder = tiny.make_folder(tiny.TINY_A, seed=25, dtype="float32", folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(256, [20, 20, 20], seed=6)
    with _engine(folder, "float32", 16, max_tokens=128, context=64, max_requests=3) as engine:
        results = engine.generate(prompts, max_tokens=40)
        assert engine.stats["preemptions"] > 0
    for prompt, result in zip(prompts, results):
        assert result["generated_tokens"] == plain.greedy(cfg, w, prompt, 40)


def test_submit_validates(tmp_path):
    folder = tiny.make_folder(tiny.TINY_A, seed=26, dtype="float32", folder=tmp_path / "m")
    with _engine(folder, "float32", 16, context=32, max_tokens=64) as engine:
        for bad in ([], [256], [-1], [1.5]):
            with pytest.raises(ValueError):
                engine.submit(bad, max_tokens=2)
        with pytest.raises(ValueError):
            engine.submit([1], max_tokens=0)
        with pytest.raises(ValueError):
            engine.submit([1] * 30, max_tokens=3)
        request = engine.submit([1, 2], max_tokens=3)
        engine.cancel(request)
        while engine.step():
            pass
        assert request.finish_reason == "cancelled"
    with pytest.raises(RuntimeError):
        engine.step()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """bin/trace_run as a user calls it: steps on standard input, logits as files, `done <step>` lines."""
    folder = tiny.make_folder(tiny.TINY_B, seed=27, dtype=dtype, folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    reqs = {f"q{i}": p for i, p in enumerate(tiny.prompts(cfg["vocab_size"], [50, 3, 71, 20, 64], seed=7))}
    steps, peak = traces.mixed(reqs, {rid: max(1, len(t) - 5) for rid, t in reqs.items()}, seed=1, live=4, page=64)
    steps.insert(2, dict(step=999, entries=[], end=[]))  # a step that brings nothing
    for i, s in enumerate(steps):
        s["step"] = i
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(peak)],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    want = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    at = {rid: 0 for rid in reqs}
    vocab = cfg["vocab_size"]
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if not wanted:
            assert not path.exists()
            continue
        data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in s["entries"]:
            for k in e["want"]:
                ref = want[e["id"]][at[e["id"]] + k]
                assert np.abs(data[row] - ref).max() <= TOL[dtype] * np.abs(want[e["id"]]).max(), (s["step"], e["id"], k)
                row += 1
            at[e["id"]] += len(e["tokens"])


def test_softcap_and_repetition_penalty(tmp_path):
    """Greedy generation under a repetition penalty: the same tokens alone and beside other requests, none of the
    last `window` tokens chosen again while an unpenalised token is within reach, and the plain recomputation with the
    same rule applied to its logits agrees."""
    folder = tiny.make_folder(tiny.TINY_A, seed=21, dtype="float32", folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(cfg["vocab_size"], [9, 20, 5], seed=3)
    knobs = dict(softcap=5.0, repetition_penalty=4.0, repetition_window=6)

    def expected(prompt, n):
        tokens, out = list(prompt), []
        for _ in range(n):
            x = plain.forward(cfg, w, tokens)[-1].double()
            x = knobs["softcap"] * torch.tanh(x / knobs["softcap"])
            for t in set(out[-knobs["repetition_window"]:]):
                x[t] = x[t] / knobs["repetition_penalty"] if x[t] > 0 else x[t] * knobs["repetition_penalty"]
            out.append(int(torch.argmax(x)))
            tokens.append(out[-1])
        return out

    with _engine(folder, "float32", tiny.PAGE["a"]) as engine:
        alone = engine.generate(prompts[0], max_tokens=12, **knobs)["generated_tokens"]
        batch = engine.generate(prompts, max_tokens=12, **knobs)
        plain_run = engine.generate(prompts[0], max_tokens=12)["generated_tokens"]
    assert batch[0]["generated_tokens"] == alone == expected(prompts[0], 12)
    assert alone != plain_run


def test_host_sampling_agrees_with_the_device(tmp_path):
    """The reference's diagnostic: NumPy's argmax over logits read back, against the argmax kernel."""
    folder = tiny.make_folder(tiny.TINY_B, seed=22, dtype="bfloat16", folder=tmp_path / "m")
    cfg, _ = plain.load_folder(folder)
    prompts = tiny.prompts(cfg["vocab_size"], [5, 33, 12], seed=4)
    with _engine(folder, "bfloat16", tiny.PAGE["b"]) as engine:
        device = [r["generated_tokens"] for r in engine.generate(prompts, max_tokens=10)]
    with _engine(folder, "bfloat16", tiny.PAGE["b"], sampling="host") as engine:
        host = [r["generated_tokens"] for r in engine.generate(prompts, max_tokens=10)]
        with pytest.raises(ValueError, match="greedy"):
            engine.generate(prompts[0], max_tokens=2, temperature=0.5)
    assert host == device


def _every_token_is_a_plain_argmax(cfg, w, prompt, tokens, slack):
    """Whether every generated token is the plain model's greedy choice given the tokens before it, or lies within
    ``slack`` (a share of the largest logit) of it: what greedy decoding in reduced precision can be held to, since
    two logits closer than the rounding may swap. Returns (ok, first bad place, share of exact choices)."""
    if not len(tokens):  # cancelled before its first token
        return True, None, 1.0
    logits = plain.forward(cfg, w, list(prompt) + list(tokens)).numpy()[len(prompt) - 1:-1]
    best = logits.max(axis=-1)
    chosen = logits[np.arange(len(tokens)), tokens]
    within = chosen >= best - slack * np.abs(logits).max()
    exact = float((logits.argmax(axis=-1) == np.asarray(tokens)).mean()) if len(tokens) else 1.0
    bad = np.nonzero(~within)[0]
    return not len(bad), (int(bad[0]) if len(bad) else None), exact


def test_greedy_tokens_in_bfloat16_agree_with_the_float32_engine(tmp_path):
    """One folder of bfloat16 weights (the 32-bit path reads them exactly), two engines, 64 greedy tokens for each of
    five prompts. The float32 engine generates the plain model's tokens. Given those tokens as its past, the bfloat16
    engine would pick the same next token at 95 of 100 places or more (measured: 0.98; with random weights two logits
    lie closer than the rounding now and then, and from there on two free-running continuations part ways, so the
    shared prefix is only printed); and every token of its own free-running continuation is a greedy choice of the
    plain model to within the rounding."""
    from akas_b200 import StepEntry

    folder = tiny.make_folder(tiny.TINY_C, seed=31, dtype="bfloat16", std=0.3, folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    prompts = tiny.prompts(cfg["vocab_size"], [40, 3, 129, 70, 11], seed=12)
    with _engine(folder, "float32", tiny.PAGE["c"]) as engine:
        want = [r["generated_tokens"] for r in engine.generate(prompts, max_tokens=64)]
    with _engine(folder, "bfloat16", tiny.PAGE["c"]) as engine:
        got = [r["generated_tokens"] for r in engine.generate(prompts, max_tokens=64)]
        forced = []
        for i, (prompt, tokens) in enumerate(zip(prompts, want)):  # the float32 engine's tokens as the past
            engine.runner.step([StepEntry(("forced", i), prompt[:-1], ())])
            picks = [int(engine.runner.step([StepEntry(("forced", i), (t,), (0,))]).argmax()) for t in [prompt[-1]] + tokens[:-1]]
            engine.runner.release(("forced", i))
            forced.append(picks)
    shared = agree = 0
    for prompt, a, b, f in zip(prompts, want, got, forced):
        assert a == plain.greedy(cfg, w, prompt, 64)
        shared += next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), 64)
        agree += sum(x == y for x, y in zip(a, f))
        ok, bad, exact = _every_token_is_a_plain_argmax(cfg, w, prompt, b, 2 * TOL["bfloat16"])
        assert ok, f"token {bad} of the bfloat16 continuation is not a greedy choice (exact choices: {exact:.3f})"
        assert exact >= 0.95
    total = 64 * len(prompts)
    print(f"bfloat16 picks the float32 engine's token at {agree} of {total} places; free-running, the continuations "
          f"share {shared} leading tokens")
    assert agree >= 0.95 * total


def test_preemption_and_arrivals_on_the_device_in_bfloat16(tmp_path):
    """Configuration c in bfloat16 with captured graphs and steps launched ahead. First a pool too small for three
    growing requests (the youngest is preempted and recomputed); then requests that arrive at random turns, some
    cancelled on the way, into the same small pool. Every token that was generated is a greedy choice of the plain
    model to within the rounding, nothing is held at the end, and the cache's books balance after every turn."""
    import random

    folder = tiny.make_folder(tiny.TINY_C, seed=32, dtype="bfloat16", std=0.3, folder=tmp_path / "m")
    cfg, w = plain.load_folder(folder)
    page = tiny.PAGE["c"]
    options = dict(max_tokens=6 * page, context=4 * page, max_requests=4, run_ahead=True, cuda_graphs=True,
                   prefill_chunk=48, prefill_requests=2)
    prompts = tiny.prompts(cfg["vocab_size"], [70, 70, 70], seed=13)
    with _engine(folder, "bfloat16", page, **options) as engine:
        results = engine.generate(prompts, max_tokens=100)
        assert engine.stats["preemptions"] > 0 and engine.stats["steps_ahead"] > 0
        for prompt, result in zip(prompts, results):
            assert len(result["generated_tokens"]) == 100
            ok, bad, exact = _every_token_is_a_plain_argmax(cfg, w, prompt, result["generated_tokens"], 2 * TOL["bfloat16"])
            assert ok and exact >= 0.95, (bad, exact)
        assert not engine.runner.cache.live()

        rng = random.Random(5)
        waiting = [(tiny.prompts(cfg["vocab_size"], [rng.randint(1, 90)], seed=40 + i)[0], rng.randint(1, 40)) for i in range(12)]
        submitted, cancelled = [], set()
        for turn in range(20000):
            while waiting and rng.random() < 0.3:
                prompt, limit = waiting.pop()
                submitted.append(engine.submit(prompt, max_tokens=limit))
            if submitted and rng.random() < 0.03:
                victim = rng.choice(submitted)
                if not victim.finished:
                    engine.cancel(victim)
                    cancelled.add(victim.id)
            busy = engine.step()
            engine.runner.cache.check()
            if not busy and not waiting:
                break
        else:
            raise AssertionError("the engine did not finish")
        assert len(submitted) == 12 and engine.stats["preemptions"] > 0
        for r in submitted:
            if r.finish_reason == "cancelled":
                assert r.id in cancelled
            else:
                assert r.finish_reason == "length" and len(r.output) == r.limit
            ok, bad, exact = _every_token_is_a_plain_argmax(cfg, w, r.prompt, r.output, 2 * TOL["bfloat16"])
            assert ok, (r.id, bad, exact)
        assert not engine.runner.cache.live()
        assert engine.runner.cache.min_free_pages() >= 0 and engine.runner.cache.free_pages() == engine.runner.cache.num_pages
