"""Command line in the manner of kreasof-ai/akas's ``akas`` (src/akas/cli.py:21-111).

    python -m akas_b200 inspect  --model DIR
    python -m akas_b200 generate --model DIR --prompt "5 17 3" [--max-tokens 128] [--context N]
                                 [--raw] [--out FILE.json] [--device 0] [--config JSON]
                                 [--temperature T --top-k K --top-p P --seed S --softcap C
                                  --repetition-penalty Q --repetition-window W --ignore-eos]
    python -m akas_b200 random   --out DIR --config JSON|FILE [--seed 0] [--dtype bfloat16]
    python -m akas_b200 bench    --model DIR [--batches 1 8] [--prompts 2048] [--generated 128] ...
    python -m akas_b200 replay   --model DIR --dtype float32 --out DIR --max-tokens N   (bin/trace_run)

Where the reference has an option, its name and meaning are kept: ``--model``, ``--prompt``,
``--max-tokens`` (default 128), ``--context``, ``--raw``, ``--out`` (the generated token ids as JSON),
``--device`` (ordinal), ``--config`` (a JSON object of engine options); for ``bench``: ``--batches``,
``--prompts``, ``--depths`` (default 0), ``--generated`` (default 128), ``--mixed``, ``--prefill-chunk``,
``--repeats`` (default 5), ``--warmup`` (default 1), ``--seed`` (default 17), ``--out``, ``--baseline`` and
``--max-regression`` (default 0.1). ``--definition`` and ``--bundle`` have no meaning here
(the model folder names its architecture; nothing is compiled ahead of time) and are accepted and ignored.
This engine holds no tokenizer: ``--prompt`` is a list of token ids, and the output is token ids.
"""

from __future__ import annotations

import argparse
import json
import re
import sys
from dataclasses import asdict, replace
from pathlib import Path


def _settings(value):
    try:
        settings = json.loads(value)
        if not isinstance(settings, dict):
            raise ValueError("config must be a JSON object")
        return settings
    except ValueError as error:
        raise argparse.ArgumentTypeError(str(error)) from error


def _token_ids(text: str):
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise argparse.ArgumentTypeError(
            "--prompt takes token ids separated by spaces or commas (this engine holds no tokenizer)"
        ) from None


def _engine_config(args):
    from .config import EngineConfig

    options = dict(getattr(args, "config", {}) or {})
    if getattr(args, "context", None) is not None:
        options["context"] = args.context
    if getattr(args, "dtype", None):
        options["dtype"] = args.dtype
    if getattr(args, "device", None) is not None:
        options["device"] = f"cuda:{args.device}"
    return replace(EngineConfig(), **options)


def _inspect(args):
    from .config import load_config
    from .models import Decoder
    from .parts.base import Runtime
    from .weights import TensorIndex, check_inventory
    import torch

    config = load_config(args.model)
    model = Decoder(config.model_spec(), Runtime(torch.float32, torch.device("cpu"), None))
    index = TensorIndex(args.model)
    check_inventory(model.params(), index)
    inventory = {name: dict(shape=list(shape), dtype=dtype) for name, (_, shape, dtype) in sorted(index.entries.items())}
    print(json.dumps(dict(architecture=config.architecture, config=asdict(config), inventory=inventory), indent=2))


def _generate(args):
    from .engine import Engine

    config = _engine_config(args)
    if args.context is None:
        config = replace(config, context=max(64, len(args.prompt) + args.max_tokens))
    config = replace(config, max_requests=min(config.max_requests, 8), max_tokens=None)
    with Engine(args.model, config=config) as engine:
        result = engine.generate(args.prompt, max_tokens=args.max_tokens, temperature=args.temperature,
                                 top_k=args.top_k, top_p=args.top_p, seed=args.seed, softcap=args.softcap,
                                 repetition_penalty=args.repetition_penalty, repetition_window=args.repetition_window,
                                 eos_token_id=None if args.ignore_eos else engine.runner.model_config.eos_token_id)
    print(" ".join(str(t) for t in result["generated_tokens"]))
    if args.out:
        args.out.write_text(json.dumps(result, indent=2) + "\n")


def _random(args):
    from .config import config_from_dict
    from .weights import write_random_model

    source = args.config.strip()
    # config.json content (a JSON object) or the path of a file that holds it
    data = json.loads(source) if source.startswith("{") else json.loads(Path(source).read_text())
    folder = write_random_model(args.out, config_from_dict(data), seed=args.seed, std=args.std, dtype=args.dtype)
    print(folder)


def _bench(args):
    from .bench import run_matrix

    from .bench import compare_reports

    baseline = json.loads(args.baseline.read_text()) if args.baseline else None
    report = run_matrix(args.model, _engine_config(args), batches=args.batches, prompts=args.prompts,
                        generated=args.generated, repeats=args.repeats, warmup=args.warmup, seed=args.seed,
                        prefill_chunk=args.prefill_chunk, depths=args.depths, mixed=args.mixed)
    if baseline is not None:
        report["changes"] = compare_reports(report, baseline, args.max_regression)
    text = json.dumps(report, indent=2)
    print(text)
    if args.out:
        args.out.write_text(text + "\n")
    if baseline is not None and any(change["regressed"] for change in report["changes"]):
        raise SystemExit(f"throughput fell by more than {args.max_regression:.0%} against {args.baseline}")


def _replay(args):
    import runpy

    script = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    sys.argv = [str(script)] + args.rest
    runpy.run_path(str(script), run_name="__main__")


def main(argv=None):
    parser = argparse.ArgumentParser(prog="akas_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    commands = parser.add_subparsers(dest="command", required=True)

    inspect = commands.add_parser("inspect", help="print the configuration and the tensor inventory of a model folder")
    inspect.add_argument("--model", required=True, type=Path)
    inspect.add_argument("--definition", help="ignored: the folder names its architecture")
    inspect.set_defaults(run=_inspect)

    generate = commands.add_parser("generate", help="generate token ids from a prompt of token ids")
    generate.add_argument("--model", required=True, type=Path)
    generate.add_argument("--definition", help="ignored: the folder names its architecture")
    generate.add_argument("--bundle", help="ignored: nothing is compiled ahead of time")
    generate.add_argument("--config", type=_settings, default={}, help="JSON object of EngineConfig fields")
    generate.add_argument("--prompt", required=True, type=_token_ids)
    generate.add_argument("--max-tokens", default=128, type=int)
    generate.add_argument("--context", type=int, help="most tokens the request may hold")
    generate.add_argument("--raw", action="store_true", help="accepted for parity; prompts are always raw token ids")
    generate.add_argument("--out", type=Path, help="save prompt and generated token ids as JSON")
    generate.add_argument("--device", type=int, default=0)
    generate.add_argument("--dtype", choices=("bfloat16", "float32"))
    generate.add_argument("--temperature", type=float, default=0.0)
    generate.add_argument("--top-k", type=int, default=0)
    generate.add_argument("--top-p", type=float, default=1.0)
    generate.add_argument("--softcap", type=float, default=0.0, help="c > 0: logits become c tanh(logit / c)")
    generate.add_argument("--repetition-penalty", type=float, default=1.0)
    generate.add_argument("--repetition-window", type=int, default=96)
    generate.add_argument("--seed", type=int)
    generate.add_argument("--ignore-eos", action="store_true")
    generate.set_defaults(run=_generate)

    random = commands.add_parser("random", help="write a model folder with seeded random weights")
    random.add_argument("--out", required=True, type=Path)
    random.add_argument("--config", required=True, help="config.json content or path")
    random.add_argument("--seed", type=int, default=0)
    random.add_argument("--std", type=float, default=0.02)
    random.add_argument("--dtype", choices=("bfloat16", "float32", "float16"), default="bfloat16")
    random.set_defaults(run=_random)

    bench = commands.add_parser("bench", help="prefill and decode throughput over batches and prompt lengths")
    bench.add_argument("--model", "--checkpoint", dest="model", required=True, type=Path)
    bench.add_argument("--definition", help="ignored")
    bench.add_argument("--config", type=_settings, default={})
    bench.add_argument("--batches", type=int, nargs="+", default=[1, 8])
    bench.add_argument("--prompts", type=int, nargs="+", default=[2048])
    bench.add_argument("--depths", type=int, nargs="+", default=[0], help="tokens already cached before the prompt")
    bench.add_argument("--generated", type=int, default=128)
    bench.add_argument("--mixed", action="store_true", help="stagger prompt lengths across slots")
    bench.add_argument("--baseline", type=Path, help="an earlier report to compare with")
    bench.add_argument("--max-regression", type=float, default=0.1,
                       help="fail on throughput loss beyond this fraction against the baseline")
    bench.add_argument("--prefill-chunk", type=int)
    bench.add_argument("--repeats", type=int, default=5)
    bench.add_argument("--warmup", type=int, default=1)
    bench.add_argument("--seed", type=int, default=17)
    bench.add_argument("--dtype", choices=("bfloat16", "float32"))
    bench.add_argument("--device", type=int, default=0)
    bench.add_argument("--out", type=Path)
    bench.set_defaults(run=_bench, context=None)

    replay = commands.add_parser("replay", help="trace replay (bin/trace_run)", add_help=False)
    replay.add_argument("rest", nargs=argparse.REMAINDER)
    replay.set_defaults(run=_replay)

    args = parser.parse_args(argv)
    args.run(args)


if __name__ == "__main__":
    main()
