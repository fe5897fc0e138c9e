"""Throughput measurement: prefill and decode tokens a second, with the bytes and flops behind them.

The protocol is kreasof-ai/akas's ``native-token-step-v2`` (src/akas/benchmarking/runner.py:72-105,
src/akas/benchmarking/workload.py:29-38): seeded synthetic prompt ids, a device synchronize at both
boundaries, load and warm-up excluded; prefill includes the head and the first predicted token; decode
counts the steps after it; ``prefill tok/s = sum of prompt lengths / seconds`` and ``decode tok/s =
batch x steps / seconds``. Times here are CUDA-event times on the launching stream.
"""

from __future__ import annotations

import statistics
from typing import Dict, List, Sequence

import numpy as np
import torch

from .engine.batch import StepEntry
from .engine.runner import ModelRunner


def synthetic_prompts(batch: int, prefix: int, vocab: int, seed: int = 17) -> List[List[int]]:
    """src/akas/benchmarking/workload.py:29-38: one generator per (batch, prefix) cell."""
    rng = np.random.default_rng(seed + batch * 4099 + prefix)
    return rng.integers(0, vocab, (batch, prefix)).tolist()


def matrix_params(runner: ModelRunner) -> Dict[str, int]:
    """Parameters of the matrix products a token passes through (per layer run, head apart)."""
    layers = 0
    for entry in runner.model.schedule:
        block = runner.model.blocks[entry.layer]
        for part in (block.mixer, block.ffn):
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.dim() == 2 and value.dtype == runner.dtype:
                    layers += value.numel()
    return dict(layers=layers, head=runner.model.head.numel())


def prefill_flops(runner: ModelRunner, tokens: int, start: int = 0) -> float:
    """Matrix products of ``tokens`` prompt tokens, causal attention over them, and one row of the head."""
    p = matrix_params(runner)
    flops = 2.0 * tokens * p["layers"] + 2.0 * p["head"]
    for entry in runner.model.schedule:
        spec = runner.model.blocks[entry.layer].mixer.spec
        if getattr(spec, "kind", "") == "attention":
            # q.k and p.v over (start + i) keys for the i-th token: 4 flops per (query, key, head, channel)
            pairs = tokens * start + tokens * (tokens + 1) / 2
            flops += 4.0 * pairs * spec.num_heads * spec.head_dim
    return flops


def decode_bytes(runner: ModelRunner, contexts: Sequence[int]) -> float:
    """Bytes one decode step has to read: every weight it uses once, the keys and values of the live
    requests, and their fixed-size state (read and written)."""
    elem = 2 if runner.dtype == torch.bfloat16 else 4
    total = float(runner.weight_bytes)
    if runner.model.head is not runner.model.embedding:
        total -= runner.model.embedding.numel() * elem  # an untied embedding is only gathered from
    for view in runner.cache.views:
        spec = getattr(view, "spec", None)
        if spec is None:
            continue
        if hasattr(spec, "num_kv_heads"):
            per_token = 2 * spec.num_kv_heads * spec.head_dim * elem
            for c in contexts:
                total += per_token * (min(c, spec.window) if spec.window else c)
        else:
            total += 2 * len(contexts) * int(np.prod(spec.shape)) * 4
    return total


def _event_ms(fn) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def fill_requests(runner: ModelRunner, prompts: Sequence[Sequence[int]], chunk: int = 2048, ids=None):
    """Admits one request per prompt and runs the prompts through in portions; returns the request ids."""
    ids = list(ids) if ids is not None else [f"bench-{i}" for i in range(len(prompts))]
    budget = max(chunk, 8192)
    at = {rid: 0 for rid in ids}
    while any(at[rid] < len(p) for rid, p in zip(ids, prompts)):
        entries, used = [], 0
        for rid, p in zip(ids, prompts):
            if at[rid] >= len(p) or used >= budget:
                continue
            k = min(chunk, len(p) - at[rid], budget - used)
            entries.append(StepEntry(rid, p[at[rid]:at[rid] + k], ()))
            at[rid] += k
            used += k
        runner.step(entries)
    return ids


def measure_prefill(runner: ModelRunner, prompt: Sequence[int], repeats: int = 7, warmup: int = 3) -> float:
    """Median milliseconds to run one whole prompt and produce its first token (head and argmax included). The warm-up
    runs also let the step function capture the prompt's shape (it does when a shape comes a third time), so the timed
    runs are replays, as in serving where portions of one size keep coming."""
    times = []
    for i in range(warmup + repeats):
        def run():
            logits = runner.step([StepEntry("prefill", prompt, (len(prompt) - 1,))])
            runner.ops.argmax(logits)
        ms = _event_ms(run)
        runner.release("prefill")
        if i >= warmup:
            times.append(ms)
    return statistics.median(times)


def measure_decode(runner: ModelRunner, batch: int, prefix: int, steps: int, warmup: int, seed: int = 17,
                   chunk: int = 2048, repeats: int = 5) -> Dict[str, float]:
    """Milliseconds per decode step at ``batch`` requests whose prompts of ``prefix`` tokens are cached.

    Each timed step feeds one given (synthetic) token per request and includes the head and the argmax;
    nothing is read back inside the timed region. A region is exactly ``steps`` steps between two synchronisations,
    timed with CUDA events; it is run up to ``repeats`` times, one after the other (the requests keep decoding, as far
    as the context allows), and the median region is reported: a single short region right after a synchronisation
    also holds the host's preparation of its first step and whatever the clocks do on their way up. The entries of
    every step are built beforehand.
    """
    vocab = runner.vocab_size
    prompts = synthetic_prompts(batch, prefix, vocab, seed)
    ids = fill_requests(runner, prompts, chunk)
    room = runner.config.context - prefix - warmup - 1
    repeats = max(1, min(repeats, room // max(steps, 1)))
    total = warmup + repeats * steps
    feed = np.random.default_rng(seed + 1).integers(0, vocab, (total, batch)).tolist()
    entries = [[StepEntry(rid, (feed[i][j],), (0,)) for j, rid in enumerate(ids)] for i in range(total)]

    def run(first, count):
        for i in range(first, first + count):
            runner.ops.argmax(runner.step(entries[i]))

    run(0, warmup)
    regions, launches = [], 0
    for r in range(repeats):
        before = runner.ops.launch_count
        regions.append(_event_ms(lambda: run(warmup + r * steps, steps)))
        launches = runner.ops.launch_count - before
    ms = statistics.median(regions)
    at = sorted(range(repeats), key=lambda r: regions[r])[repeats // 2]  # the region whose time is reported
    contexts = [prefix + warmup + at * steps + steps // 2] * batch
    for rid in ids:
        runner.release(rid)
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3), bytes=decode_bytes(runner, contexts),
                launches=launches, regions_ms=[round(x, 4) for x in regions])


def case_lengths(batch: int, prompt: int, mixed: bool) -> List[int]:
    """Prompt length per slot: all ``prompt``, or staggered as the reference staggers them
    (src/akas/benchmarking/cases.py:30-35)."""
    return [max(1, prompt - i % min(prompt, 7)) if mixed else prompt for i in range(batch)]


def run_matrix(model_dir, config, batches=(1, 8), prompts=(2048,), generated=128, repeats=5, warmup=1, seed=17,
               prefill_chunk=None, depths=(0,), mixed=False) -> dict:
    """The reference's pp/tg matrix (src/akas/benchmarking/cases.py:8-61): for every (batch, prompt length, depth)
    the median prefill and decode tokens a second over ``repeats`` repetitions after ``warmup``. ``depth``: tokens
    already in the cache of every request before its measured prompt; ``mixed``: prompt lengths staggered over the
    slots."""
    from dataclasses import replace

    if any(d < 0 for d in depths) or generated < 1 or min(batches) < 1 or min(prompts) < 1:
        raise ValueError("positive batch/prompt/generation and nonnegative depth required")
    longest = max(depths) + max(prompts) + generated
    need = max(batches) * (longest + 64)
    config = replace(config, max_requests=max(config.max_requests, max(batches)),
                     context=max(config.context, longest + 1), max_tokens=None)
    if config.pool_tokens < need:
        config = replace(config, max_tokens=need)
    runner = ModelRunner(model_dir, config)
    chunk = prefill_chunk or config.prefill_chunk
    rows = []
    for batch in batches:
        for prefix in prompts:
            for depth in depths:
                lengths = case_lengths(batch, prefix, mixed)
                pp, tg = [], []
                for rep in range(warmup + repeats):
                    data = [p[:n] for p, n in zip(synthetic_prompts(batch, prefix, runner.vocab_size, seed), lengths)]
                    ids = [f"m{j}" for j in range(batch)]
                    if depth:
                        fill_requests(runner, synthetic_prompts(batch, depth, runner.vocab_size, seed + 1), chunk, ids)

                    def prefill():
                        fill_requests(runner, [p[:-1] for p in data], chunk, ids)
                        logits = runner.step([StepEntry(rid, (p[-1],), (0,)) for rid, p in zip(ids, data)])
                        return runner.ops.argmax(logits)

                    holder = {}
                    pp_ms = _event_ms(lambda: holder.setdefault("t", prefill()))
                    tokens = holder["t"]

                    def decode():
                        # every step feeds the tokens that the step before picked; they stay on the device (an entry
                        # names its place among them), as in the engine's own loop, so nothing waits for the host
                        t = tokens
                        entries = [StepEntry(rid, (0,), (0,), source=j) for j, rid in enumerate(ids)]
                        for _ in range(generated - 1):
                            t = runner.ops.argmax(runner.step(entries, previous=t))

                    tg_ms = _event_ms(decode)
                    for rid in ids:
                        runner.release(rid)
                    if rep >= warmup:
                        pp.append(sum(lengths) / (pp_ms / 1e3))
                        if generated > 1:
                            tg.append(batch * (generated - 1) / (tg_ms / 1e3))
                rows.append(dict(batch=batch, prompt=prefix, generated=generated, depth=depth, mixed=mixed,
                                 prefill_tokens_per_s=statistics.median(pp),
                                 decode_tokens_per_s=statistics.median(tg) if tg else None))
    return dict(protocol="native-token-step-v2", dtype=config.dtype, seed=seed, repeats=repeats, warmup=warmup,
                prefill_chunk=chunk, rows=rows)


def compare_reports(report: dict, baseline: dict, max_regression: float = 0.1) -> List[dict]:
    """Every measured case against the same case of an earlier report, as the reference's bench gate does
    (src/akas/cli.py:527, 666-680): raises if the baseline lacks a case, returns the changes, and marks a case whose
    prefill or decode rate fell by more than ``max_regression`` of the baseline's."""
    if not 0 <= max_regression < 1:
        raise ValueError("invalid regression setting")
    key = lambda row: (row["batch"], row["prompt"], row.get("generated"), row.get("depth", 0), row.get("mixed", False))
    before = {key(row): row for row in baseline.get("rows", [])}
    changes = []
    for row in report["rows"]:
        old = before.get(key(row))
        if old is None:
            raise ValueError("baseline must cover every measured case")
        change = dict(batch=row["batch"], prompt=row["prompt"], depth=row.get("depth", 0), mixed=row.get("mixed", False))
        for name in ("prefill_tokens_per_s", "decode_tokens_per_s"):
            if row.get(name) and old.get(name):
                change[name + "_ratio"] = row[name] / old[name]
        change["regressed"] = any(v < 1 - max_regression for k, v in change.items() if k.endswith("_ratio"))
        changes.append(change)
    return changes


# --------------------------------------------------------------------------- single kernels


def _time_kernel(fn, iters: int, flush_bytes: int = 256 << 20) -> float:
    """Median milliseconds of ``fn()``; a buffer larger than L2 is rewritten before every timed call."""
    flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda")
    times = []
    for i in range(iters + 3):
        flush.fill_(i & 1)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def bench_linear(m: int, o: int, k: int, mode: str, iters: int = 20) -> dict:
    """One matrix product of the bfloat16 path, cold L2: mode is bf16 | f32 | acc | swiglu | norm | norm_swiglu."""
    from .ops import cuda as ops

    ops.require(ops.libraries_for(torch.bfloat16))
    g = torch.Generator(device="cuda").manual_seed(0)
    w = (torch.randn((o, k), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.bfloat16)
    h = torch.randn((m, k), device="cuda", generator=g)
    nw = torch.ones(k, device="cuda")
    res = torch.zeros((m, o), device="cuda")
    fn = {
        "bf16": lambda: ops.linear(x, w),
        "f32": lambda: ops.linear(x, w, out_dtype=torch.float32),
        "acc": lambda: ops.linear(x, w, residual=res),
        "swiglu": lambda: ops.linear_swiglu(x, w),
        "norm": lambda: ops.norm_linear(h, nw, 1e-5, False, w),
        "norm_swiglu": lambda: ops.norm_linear(h, nw, 1e-5, False, w, None, None, True),
    }[mode]
    ms = _time_kernel(fn, iters)
    nbytes = w.numel() * 2
    return dict(kernel="linear", mode=mode, m=m, o=o, k=k, ms=round(ms, 5), weight_gb_s=round(nbytes / ms / 1e6, 1),
                tflops=round(2.0 * m * o * k / ms / 1e9, 2))


def bench_attention(kind: str, batch: int, context: int, heads: int = 32, kv_heads: int = 8, dim: int = 64,
                    page: int = 64, iters: int = 20) -> dict:
    """Paged attention of the bfloat16 path, cold L2. ``decode``: ``batch`` requests of ``context`` cached tokens,
    one query token each. ``prompt``: ``batch`` requests whose whole ``context`` tokens are queries."""
    from types import SimpleNamespace

    from .ops import cuda as ops

    ops.require(ops.libraries_for(torch.bfloat16))
    g = torch.Generator(device="cuda").manual_seed(0)
    blocks = -(-context // page)
    pages = batch * blocks
    k = torch.randn((pages, kv_heads, page, dim), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((pages, kv_heads, page, dim), device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).view(batch, blocks)
    if kind == "decode":
        n = batch
        seq = torch.arange(batch, dtype=torch.int32, device="cuda")
        pos = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(decode_only=True, max_context=context, query_lens=(1,) * batch, cu_seqlens=None, memo={})
        flops = 4.0 * batch * context * heads * dim
    else:
        n = batch * context
        seq = torch.arange(batch, dtype=torch.int32, device="cuda").repeat_interleave(context)
        pos = torch.arange(context, dtype=torch.int32, device="cuda").repeat(batch)
        cu = torch.arange(0, n + 1, context, dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(decode_only=False, max_context=context, query_lens=(context,) * batch, cu_seqlens=cu, memo={})
        flops = 4.0 * batch * context * (context + 1) / 2 * heads * dim
    q = torch.randn((n, heads * dim), device="cuda", generator=g).to(torch.bfloat16)
    ms = _time_kernel(lambda: ops.paged_attention(q, k, v, table, seq, pos, dim ** -0.5, None, page, ctx), iters)
    kv_bytes = 2.0 * batch * context * kv_heads * dim * 2
    return dict(kernel="attention", kind=kind, batch=batch, context=context, heads=heads, kv_heads=kv_heads, head_dim=dim,
                ms=round(ms, 5), kv_gb_s=round(kv_bytes / ms / 1e6, 1), tflops=round(flops / ms / 1e9, 2))


SHAPES = {
    # the dense LFM2 sizes named by the benchmark configurations (config.json keys; everything else at its default)
    "350m": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=6656),
    "700m": dict(hidden_size=1536, num_attention_heads=24, num_key_value_heads=8, intermediate_size=10240),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288),
}


def shape_config(name: str) -> dict:
    base = dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", num_hidden_layers=16,
                full_attn_idxs=[2, 5, 8, 10, 12, 14], vocab_size=65536, rope_theta=1000000.0, norm_eps=1e-5,
                conv_L_cache=3, conv_bias=False, block_auto_adjust_ff_dim=True, block_multiple_of=256,
                block_ffn_dim_multiplier=1.0, tie_embedding=True, max_position_embeddings=128000)
    base.update(SHAPES[name])
    return base


def _random_engine(shape: str, **options):
    import tempfile

    from . import Engine, EngineConfig
    from .config import config_from_dict
    from .weights import write_random_model

    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        return Engine(folder, config=EngineConfig(dtype="bfloat16", **options))


def bench_serving(shape: str = "350m", requests: int = 256, shortest: int = 128, longest: int = 2048, generated: int = 128,
                  chunk: int = 512, seed: int = 17) -> dict:
    """Many requests at once through the engine: random prompt lengths, prompts cut into portions of ``chunk``
    that share steps with decoding requests. Wall time from the first submit to the last token."""
    import time

    rng = np.random.default_rng(seed)
    lengths = rng.integers(shortest, longest + 1, requests).tolist()
    vocab = shape_config(shape)["vocab_size"]
    prompts = [rng.integers(0, vocab, n).tolist() for n in lengths]
    pool = sum(-(-(n + generated) // 64) * 64 for n in lengths)
    engine = _random_engine(shape, max_requests=requests, context=longest + generated + 64, max_tokens=pool + 64 * requests,
                            prefill_chunk=chunk, prefill_requests=32, prefill_token_budget=8192)
    with engine:
        engine.warm_up()  # the decode graphs of every batch size
        engine.generate(prompts[:4], max_tokens=8)  # kernels and library handles of the prompt path
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        results = engine.generate(prompts, max_tokens=generated)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        stats = dict(engine.stats)
    out = sum(len(r["generated_tokens"]) for r in results)
    return dict(bench="serving", shape=shape, requests=requests, prompt_tokens=sum(lengths), generated_tokens=out,
                seconds=round(seconds, 3), output_tokens_per_s=round(out / seconds, 1),
                total_tokens_per_s=round((out + sum(lengths)) / seconds, 1), steps=stats["steps"],
                steps_ahead=stats["steps_ahead"], preemptions=stats["preemptions"], max_active=stats["max_active"])


def bench_long_context(shape: str = "700m", requests: int = 8, prompt: int = 30000, generated: int = 256,
                       chunk: int = 2048, seed: int = 17) -> dict:
    """A few very long prompts, then decoding: the paged cache and the split-key decode attention under load."""
    vocab = shape_config(shape)["vocab_size"]
    context = -(-(prompt + generated + 64) // 64) * 64
    engine = _random_engine(shape, max_requests=requests, context=context, max_tokens=requests * context,
                            prefill_chunk=chunk, prefill_token_budget=8192)
    runner = engine.runner
    prompts = synthetic_prompts(requests, prompt, vocab, seed)
    pre = []
    for rep in range(2):
        ids = [f"w{rep}-{i}" for i in range(requests)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for rid, tokens in zip(ids, prompts):
            for at in range(0, prompt, chunk):
                part = tokens[at:at + chunk]
                runner.step([StepEntry(rid, part, (len(part) - 1,) if at + chunk >= prompt else ())])
        stop.record()
        torch.cuda.synchronize()
        pre.append(start.elapsed_time(stop))
        if rep == 0:
            for rid in ids:
                runner.release(rid)
    feed = np.random.default_rng(seed + 1).integers(0, vocab, (generated + 8, requests)).tolist()

    def step(i):
        logits = runner.step([StepEntry(rid, (feed[i][j],), (0,)) for j, rid in enumerate(ids)])
        return runner.ops.argmax(logits)

    for i in range(8):
        step(i)
    ms = _event_ms(lambda: [step(8 + i) for i in range(generated)])
    contexts = [prompt + 8 + generated // 2] * requests
    nbytes = decode_bytes(runner, contexts)
    engine.close()
    return dict(bench="long_context", shape=shape, requests=requests, prompt=prompt, generated=generated,
                prefill_tokens_per_s=round(requests * prompt / (pre[-1] / 1e3), 1), prefill_ms=round(pre[-1], 1),
                decode_ms_per_step=round(ms / generated, 4), decode_tokens_per_s=round(requests * generated / (ms / 1e3), 1),
                decode_gb_per_step=round(nbytes / 1e9, 3), decode_gb_s=round(nbytes / (ms / generated / 1e3) / 1e9, 1))


def bench_ops(shape: str = "1.2b", prompt: int = 2048, batch: int = 8, steps: int = 16) -> dict:
    """Where the device time of one prompt of ``prompt`` tokens and of ``steps`` decode steps of ``batch`` requests
    goes, by operation (CUDA events around every call of the step function's operations; no captured graphs)."""
    import tempfile

    from .config import EngineConfig, config_from_dict
    from .ops import cuda as cuda_ops
    from .ops.timed import TimedOps
    from .weights import write_random_model

    cuda_ops.require(cuda_ops.libraries_for(torch.bfloat16))
    timed = TimedOps(cuda_ops)
    config = EngineConfig(dtype="bfloat16", max_requests=batch, context=prompt + steps + 64, cuda_graphs=False)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config, ops=timed)
    prompts = synthetic_prompts(batch, prompt, runner.vocab_size)
    ids = [f"o{j}" for j in range(batch)]
    fill_requests(runner, [p[:-1] for p in prompts[1:]], config.prefill_chunk, ids[1:])  # the others, and a warm-up
    timed.clear()
    runner.step([StepEntry(ids[0], prompts[0][:-1], ())])
    prefill = timed.table()
    tokens = [p[-1] for p in prompts]
    runner.step([StepEntry(rid, (t,), (0,)) for rid, t in zip(ids, tokens)])  # first decode step: set-up costs
    timed.clear()
    for _ in range(steps):
        logits = runner.step([StepEntry(rid, (t,), (0,)) for rid, t in zip(ids, tokens)])
        tokens = timed.argmax(logits).tolist()
    decode = timed.table()
    for row in decode:
        row["ms"] /= steps
    round_rows = lambda rows: [dict(op=r["op"], calls=r["calls"], ms=round(r["ms"], 4), share=round(r["share"], 3)) for r in rows]
    return dict(bench="ops", shape=shape, prompt=prompt, batch=batch, prefill=round_rows(prefill),
                decode_per_step=round_rows(decode))


def bench_ops_mixed(shape: str = "350m", portion: int = 512, decoding: int = 255, shortest: int = 128,
                    longest: int = 2176, steps: int = 4) -> dict:
    """Where the device time of a MIXED step goes, by operation: a prompt portion of ``portion`` tokens (of a request
    that already holds as many) beside ``decoding`` requests with contexts spread evenly from ``shortest`` to
    ``longest``, one decoded token each. Measured for both ways of running the decoded tokens' attention: "split"
    (they go to the split-key decode kernel, the portion to the prompt kernel) and "tiles" (every token is a query
    tile of the prompt kernel). CUDA events around every call of the step function's operations; no captured graphs."""
    import tempfile

    from .config import EngineConfig, config_from_dict
    from .ops import cuda as cuda_ops
    from .ops.timed import TimedOps
    from .weights import write_random_model

    cuda_ops.require(cuda_ops.libraries_for(torch.bfloat16))
    timed = TimedOps(cuda_ops)
    lengths = [shortest + (longest - shortest) * j // max(decoding - 1, 1) for j in range(decoding)]
    context = max(longest, 2 * portion) + steps * (portion + 1) + 64
    pool = sum(-(-(n + steps + 64) // 64) * 64 for n in lengths) + context + 64
    config = EngineConfig(dtype="bfloat16", max_requests=decoding + 1, context=context, max_tokens=pool, cuda_graphs=False)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config, ops=timed)
    rng = np.random.default_rng(7)
    ids = [f"d{j}" for j in range(decoding)]
    fill_requests(runner, [rng.integers(0, runner.vocab_size, n).tolist() for n in lengths], config.prefill_chunk, ids)
    runner.step([StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ())])
    report = dict(bench="ops-mixed", shape=shape, portion=portion, decoding=decoding, contexts=[shortest, longest])
    before = cuda_ops.mixed_attention
    try:
        for policy in ("split", "tiles"):
            cuda_ops.mixed_attention = policy
            for step in range(steps + 1):
                if step == 1:
                    timed.clear()  # the first step of a policy pays for set-up
                entries = [StepEntry(rid, (int(rng.integers(0, runner.vocab_size)),), (0,)) for rid in ids]
                entries.append(StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ()))
                runner.step(entries)
            rows = timed.table()
            total = sum(r["ms"] for r in rows) / steps
            report[policy] = dict(ms_per_step=round(total, 4), tokens_per_step=decoding + portion,
                                  ops=[dict(op=r["op"], calls=r["calls"] // steps, ms=round(r["ms"] / steps, 4),
                                            share=round(r["share"], 3)) for r in rows])
            for rid in ["p"]:  # the portioned request starts over, so that both policies see the same lengths
                runner.release(rid)
            runner.step([StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ())])
    finally:
        cuda_ops.mixed_attention = before
    return report


def bench_timeline(shape: str = "1.2b", batch: int = 8, prompt: int = 2048, context: int = 4096) -> dict:
    """The kernels of ONE captured decode step of ``batch`` requests as the GPU ran them (torch's profiler around a
    graph replay): per kernel name the number of launches, the summed duration, and the time the step advanced while
    it ran, i.e. from the end of the kernels before it to its own end: kernels of the decode path are launched ahead
    of their predecessor's end and wait inside, so durations overlap and their sum exceeds the step."""
    import tempfile

    from torch.profiler import ProfilerActivity, profile

    from .config import EngineConfig, config_from_dict
    from .weights import write_random_model

    config = EngineConfig(dtype="bfloat16", max_requests=max(batch, 1), context=context, max_tokens=batch * context,
                          cuda_graphs=True)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config)
    ids = fill_requests(runner, synthetic_prompts(batch, prompt, runner.vocab_size))

    def decode(steps):
        for i in range(steps):
            runner.ops.argmax(runner.step([StepEntry(rid, (5 + i,), (0,)) for rid in ids]))

    decode(5)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        decode(2)
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type.name == "CUDA" and "Memcpy" not in e.name and "Memset" not in e.name),
                    key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(events) if "embedding" in e.name)  # the second step
    events = events[first:]
    start = done = events[0].time_range.start
    table: Dict[str, list] = {}
    for e in events:
        name = e.name.replace("(anonymous namespace)::", "")
        name = (name[5:] if name.startswith("void ") else name).split("(")[0].strip()
        row = table.setdefault(name, [0, 0.0, 0.0])
        row[0] += 1
        row[1] += e.time_range.end - e.time_range.start
        row[2] += max(0.0, e.time_range.end - max(done, e.time_range.start))
        done = max(done, e.time_range.end)
    rows = [dict(kernel=k, launches=v[0], duration_us=round(v[1], 1), advanced_us=round(v[2], 1))
            for k, v in sorted(table.items(), key=lambda kv: -kv[1][2])]
    return dict(bench="timeline", shape=shape, batch=batch, prompt=prompt, step_us=round(done - start, 1),
                kernels_per_step=len(events), kernels=rows)


def _main():
    import argparse
    import json

    ap = argparse.ArgumentParser(description="single kernels of the bfloat16 path (cold L2, CUDA events), and two whole-engine runs")
    sub = ap.add_subparsers(dest="what", required=True)
    lin = sub.add_parser("linear", help="y = x . w^T with one of the epilogues")
    lin.add_argument("--m", type=int, nargs="+", default=[8])
    lin.add_argument("--o", type=int, default=2048)
    lin.add_argument("--k", type=int, default=2048)
    lin.add_argument("--mode", default="bf16", choices=("bf16", "f32", "acc", "swiglu", "norm", "norm_swiglu"))
    lin.add_argument("--iters", type=int, default=20)
    att = sub.add_parser("attention", help="paged attention over the cache")
    att.add_argument("--kind", default="decode", choices=("decode", "prompt"))
    att.add_argument("--batch", type=int, nargs="+", default=[8])
    att.add_argument("--context", type=int, default=2048)
    att.add_argument("--heads", type=int, default=32)
    att.add_argument("--kv-heads", type=int, default=8)
    att.add_argument("--head-dim", type=int, default=64)
    att.add_argument("--iters", type=int, default=20)
    srv = sub.add_parser("serving", help="many requests through the engine, prompt portions mixed with decoding")
    srv.add_argument("--shape", default="350m", choices=sorted(SHAPES))
    srv.add_argument("--requests", type=int, default=256)
    srv.add_argument("--generated", type=int, default=128)
    srv.add_argument("--chunk", type=int, default=512)
    lng = sub.add_parser("long-context", help="a few very long prompts, then decoding")
    lng.add_argument("--shape", default="700m", choices=sorted(SHAPES))
    lng.add_argument("--requests", type=int, default=8)
    lng.add_argument("--prompt", type=int, default=30000)
    lng.add_argument("--generated", type=int, default=256)
    tml = sub.add_parser("timeline", help="the kernels of one captured decode step as the GPU ran them")
    tml.add_argument("--shape", default="1.2b", choices=sorted(SHAPES))
    tml.add_argument("--batch", type=int, default=8)
    tml.add_argument("--prompt", type=int, default=2048)
    per = sub.add_parser("ops", help="device time of a prompt and of decode steps, by operation")
    per.add_argument("--shape", default="1.2b", choices=sorted(SHAPES))
    per.add_argument("--prompt", type=int, default=2048)
    per.add_argument("--batch", type=int, default=8)
    per.add_argument("--steps", type=int, default=16)
    per.add_argument("--mixed", type=int, nargs=2, metavar=("PORTION", "DECODING"), default=None,
                     help="a mixed step instead: a prompt portion of PORTION tokens beside DECODING decoding requests")
    args = ap.parse_args()
    if args.what == "timeline":
        print(json.dumps(bench_timeline(args.shape, args.batch, args.prompt), indent=1))
        return
    if args.what == "ops" and args.mixed:
        print(json.dumps(bench_ops_mixed(args.shape, args.mixed[0], args.mixed[1], steps=min(args.steps, 8)), indent=1))
        return
    if args.what == "ops":
        print(json.dumps(bench_ops(args.shape, args.prompt, args.batch, args.steps), indent=1))
        return
    if args.what == "serving":
        print(json.dumps(bench_serving(args.shape, args.requests, generated=args.generated, chunk=args.chunk)))
        return
    if args.what == "long-context":
        print(json.dumps(bench_long_context(args.shape, args.requests, args.prompt, args.generated)))
        return
    if args.what == "attention":
        for b in args.batch:
            print(json.dumps(bench_attention(args.kind, b, args.context, args.heads, args.kv_heads, args.head_dim,
                                             iters=args.iters)))
        return
    for m in args.m:
        print(json.dumps(bench_linear(m, args.o, args.k, args.mode, args.iters)))


if __name__ == "__main__":
    _main()
