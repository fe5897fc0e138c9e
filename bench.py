"""Decode and prefill throughput of the engine on one B200, at LFM2-1.2B's layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--dtype bfloat16|float32]
    python bench.py --impl reference        (prints why the reference cannot run here)

A step is one decode step of a batch of 8 requests whose 2,048-token prompts are in the cache
(context 4,096). ``value`` is decoded tokens a second, timed on the device with CUDA events around
exactly ``--steps`` steps after ``--warmup`` untimed ones (the region is repeated up to five times and the median
is reported); ``e2e`` is the same through ``Engine``
(host token ids in, sampled ids read back every step). The one JSON line also carries the prefill of
2,048 tokens, the decode roofline (bytes a step must read / its time, against the measured copy
bandwidth) and decode at batches 1 and 64. Inputs (2.3 GB of weights read every step) are larger
than L2, so no flush is needed between timed steps.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the LFM2-1.2B shape: layer sizes of the published model, random weights
LFM2_1_2B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=2048, num_attention_heads=32,
    num_key_value_heads=8, intermediate_size=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
    block_multiple_of=256, vocab_size=65536, num_hidden_layers=16, full_attn_idxs=[2, 5, 8, 10, 12, 14],
    rope_theta=1000000.0, norm_eps=1e-5, conv_L_cache=3, conv_bias=False, tie_embedding=True,
    max_position_embeddings=128000,
)
BATCH, PROMPT, CONTEXT = 8, 2048, 4096
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, fp32_tflops=75.0)


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in data.items() if isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        rows = [line.strip().split(", ") for line in self.file if line.strip()]
        self.file.close()
        os.unlink(self.file.name)
        sm, top, reasons = [], 0, set()
        for row in rows:
            try:
                sm.append(int(row[0]))
                top = max(top, int(row[1]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[2:]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        return dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=top or None,
                    reasons=sorted(reasons), samples=len(sm))


def reference_arm():
    """Runs nothing of ours. kreasof-ai/akas installs offline only without its dependencies; its kernels are
    TileLang programs that its external compiler and runtime package (``tensor-workspace``, pinned in its
    pyproject.toml; TVM behind it) must build and launch, and no wheel of that package exists here. So the
    arm checks what can be imported and says why it cannot measure."""
    ref = ROOT / "baseline" / "_ref"
    why = None
    if not (ref / "akas").is_dir():
        why = "kreasof-ai/akas is not installed under baseline/_ref"
    else:
        sys.path.insert(0, str(ref))
        try:
            import akas  # noqa: F401
            import tensor  # noqa: F401  (the reference's device runtime: `import tensor` in src/akas/cli.py:135)
        except Exception as error:  # ImportError here; anything else is as final
            why = (f"kreasof-ai/akas installed with --no-deps but cannot run: {type(error).__name__}: {error}; its "
                   "compiler/runtime package tensor-workspace==0.1.0 has no wheel in the offline wheelhouse")
    if why is None:
        why = "the reference imports, but no compiled .tbin program for sm_100a exists and its targets stop at sm_90a"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batches 1 and 64")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    args.steps = max(1, min(args.steps, CONTEXT - PROMPT - args.warmup - 17))

    import torch

    from akas_b200 import Engine, EngineConfig
    from akas_b200.bench import (decode_bytes, measure_decode, measure_prefill, prefill_flops, synthetic_prompts)
    from akas_b200.config import config_from_dict
    from akas_b200.engine.runner import ModelRunner
    from akas_b200.weights import write_random_model

    data = dict(LFM2_1_2B)
    full_layers = data["num_hidden_layers"]
    if args.layers is not None and args.layers < full_layers:
        data["num_hidden_layers"] = args.layers
        data["full_attn_idxs"] = [i for i in data["full_attn_idxs"] if i < args.layers]
    model_config = config_from_dict(data)
    pk = peaks()

    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        t0 = time.time()
        write_random_model(folder, model_config, seed=0, dtype=args.dtype)
        engine_config = EngineConfig(dtype=args.dtype, max_requests=64, context=CONTEXT, max_tokens=64 * CONTEXT,
                                     page_size=64, prefill_chunk=2048, prefill_token_budget=8192)
        runner = ModelRunner(folder, engine_config)
        load_s = time.time() - t0

        # prefill of 2,048 tokens, one request
        prompt = synthetic_prompts(1, PROMPT, model_config.vocab_size)[0]
        pre_ms = measure_prefill(runner, prompt, repeats=7, warmup=3)
        pre_flops = prefill_flops(runner, PROMPT)
        flop_peak = (pk["bf16_tflops"] if args.dtype == "bfloat16" else pk["fp32_tflops"]) * 1e12

        # decode at batch 8: the headline, with clocks sampled during the timed region
        sampler = ClockSampler()
        main_run = measure_decode(runner, BATCH, PROMPT, args.steps, args.warmup)
        clocks = sampler.stop()
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(measure_decode(runner, b, PROMPT, min(args.steps, 128), args.warmup)["tokens_per_s"], 1)

        # end to end through Engine: host ids in, sampled ids read back every step
        engine = Engine(runner)
        prompts = synthetic_prompts(BATCH, PROMPT, model_config.vocab_size)
        e2e_steps = args.steps
        requests = [engine.submit(p, max_tokens=args.warmup + e2e_steps + 16) for p in prompts]  # nobody ends inside the timed steps
        while any(len(r.output) < args.warmup for r in requests):
            engine.step()
        torch.cuda.synchronize()
        # what is alive now (model, prompts, graphs) stays alive: keep the collector from walking it in mid-run
        gc.collect()
        gc.freeze()
        before = sum(len(r.output) for r in requests)
        t1 = time.perf_counter()
        for _ in range(e2e_steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        produced = sum(len(r.output) for r in requests) - before
        for r in requests:
            engine.cancel(r)
        engine.step()
        graph = runner._graphs.get(BATCH)
        h2d = graph.layout.size * 4 if graph is not None else 0

    achieved = main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    kernels_per_step = getattr(runner, "kernels_per_decode_step", {}).get(BATCH, 0) + 1  # + the argmax
    line = {
        "metric": "decode tok/s at batch 8 (LFM2-1.2B shape, 2,048-token prompts cached, context 4,096)",
        "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic token ids (seeded, the reference's generator), random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "LFM2-1.2B shape", "layers": data["num_hidden_layers"], "layers_of_configuration": full_layers,
            "attention_layers": len(data["full_attn_idxs"]), "hidden": 2048, "heads": 32, "kv_heads": 8, "head_dim": 64,
            "ff": model_config.feed_forward_size, "vocab": 65536, "conv_L_cache": 3, "tied": True,
            "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": 64,
            "parallelism": "single GPU", "cuda_graphs": True, "l2": "inputs (weights) larger than L2",
            "timed_regions": len(main_run["regions_ms"]),
        },
        "clocks": clocks,
        "e2e": {"value": round(produced / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": BATCH * 4, "steps": e2e_steps},
        "gpu_launches": kernels_per_step * args.steps,
        "prefill": {"value": round(PROMPT / (pre_ms / 1e3), 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / flop_peak, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "load_s": round(load_s, 1),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
