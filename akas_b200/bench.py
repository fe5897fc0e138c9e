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


def measure_prefill(runner: ModelRunner, prompt: Sequence[int], repeats: int = 3, warmup: int = 1) -> float:
    """Median milliseconds to run one whole prompt and produce its first token (head and argmax included)."""
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
                   chunk: int = 2048) -> Dict[str, float]:
    """Milliseconds per decode step at ``batch`` requests whose prompts of ``prefix`` tokens are cached.

    Each timed step feeds one given (synthetic) token per request and includes the head and the argmax;
    nothing is read back inside the timed region.
    """
    vocab = runner.vocab_size
    prompts = synthetic_prompts(batch, prefix, vocab, seed)
    ids = fill_requests(runner, prompts, chunk)
    feed = np.random.default_rng(seed + 1).integers(0, vocab, (warmup + steps, batch)).tolist()

    def step(i):
        logits = runner.step([StepEntry(rid, (feed[i][j],), (0,)) for j, rid in enumerate(ids)])
        return runner.ops.argmax(logits)

    for i in range(warmup):
        step(i)
    launches_before = runner.ops.launch_count
    ms = _event_ms(lambda: [step(warmup + i) for i in range(steps)])
    contexts = [prefix + warmup + steps // 2] * batch
    for rid in ids:
        runner.release(rid)
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3), bytes=decode_bytes(runner, contexts),
                launches=runner.ops.launch_count - launches_before)


def run_matrix(model_dir, config, batches=(1, 8), prompts=(2048,), generated=128, repeats=5, warmup=1, seed=17,
               prefill_chunk=None) -> dict:
    """The reference's pp/tg matrix (src/akas/benchmarking/cases.py:8-42): for every (batch, prompt length)
    the median prefill and decode tokens a second over ``repeats`` repetitions after ``warmup``."""
    from dataclasses import replace

    need = max(batches) * (max(prompts) + generated + 64)
    config = replace(config, max_requests=max(config.max_requests, max(batches)),
                     context=max(config.context, max(prompts) + generated + 1), max_tokens=None)
    if config.pool_tokens < need:
        config = replace(config, max_tokens=need)
    runner = ModelRunner(model_dir, config)
    chunk = prefill_chunk or config.prefill_chunk
    rows = []
    for batch in batches:
        for prefix in prompts:
            pp, tg = [], []
            for rep in range(warmup + repeats):
                data = synthetic_prompts(batch, prefix, runner.vocab_size, seed)
                ids = [f"m{j}" for j in range(batch)]

                def prefill():
                    fill_requests(runner, [p[:-1] for p in data], chunk, ids)
                    logits = runner.step([StepEntry(rid, (p[-1],), (0,)) for rid, p in zip(ids, data)])
                    return runner.ops.argmax(logits)

                holder = {}
                pp_ms = _event_ms(lambda: holder.setdefault("t", prefill()))
                tokens = holder["t"]

                def decode():
                    t = tokens
                    for _ in range(generated - 1):
                        host = t.tolist()
                        logits = runner.step([StepEntry(rid, (host[j],), (0,)) for j, rid in enumerate(ids)])
                        t = runner.ops.argmax(logits)

                tg_ms = _event_ms(decode)
                for rid in ids:
                    runner.release(rid)
                if rep >= warmup:
                    pp.append(batch * prefix / (pp_ms / 1e3))
                    tg.append(batch * (generated - 1) / (tg_ms / 1e3))
            rows.append(dict(batch=batch, prompt=prefix, generated=generated,
                             prefill_tokens_per_s=statistics.median(pp), decode_tokens_per_s=statistics.median(tg)))
    return dict(protocol="native-token-step-v2", dtype=config.dtype, seed=seed, repeats=repeats, warmup=warmup,
                prefill_chunk=chunk, rows=rows)


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
        ctx = SimpleNamespace(decode_only=True, max_context=context, query_tiles=0, cu_seqlens=None)
        flops = 4.0 * batch * context * heads * dim
    else:
        n = batch * context
        seq = torch.arange(batch, dtype=torch.int32, device="cuda").repeat_interleave(context)
        pos = torch.arange(context, dtype=torch.int32, device="cuda").repeat(batch)
        cu = torch.arange(0, n + 1, context, dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(decode_only=False, max_context=context, query_tiles=batch * -(-context // 64), cu_seqlens=cu)
        flops = 4.0 * batch * context * (context + 1) / 2 * heads * dim
    q = torch.randn((n, heads * dim), device="cuda", generator=g).to(torch.bfloat16)
    ms = _time_kernel(lambda: ops.paged_attention(q, k, v, table, seq, pos, dim ** -0.5, None, page, ctx), iters)
    kv_bytes = 2.0 * batch * context * kv_heads * dim * 2
    return dict(kernel="attention", kind=kind, batch=batch, context=context, heads=heads, kv_heads=kv_heads, head_dim=dim,
                ms=round(ms, 5), kv_gb_s=round(kv_bytes / ms / 1e6, 1), tflops=round(flops / ms / 1e9, 2))


def _main():
    import argparse
    import json

    ap = argparse.ArgumentParser(description="time single kernels of the bfloat16 path (cold L2, CUDA events)")
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
    args = ap.parse_args()
    if args.what == "attention":
        for b in args.batch:
            print(json.dumps(bench_attention(args.kind, b, args.context, args.heads, args.kv_heads, args.head_dim,
                                             iters=args.iters)))
        return
    for m in args.m:
        print(json.dumps(bench_linear(m, args.o, args.k, args.mode, args.iters)))


if __name__ == "__main__":
    _main()
