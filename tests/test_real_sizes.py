"""The engine at the real layer sizes against the plain model, under every way of cutting the work.

Every other replay test runs models of width 64 to 128. Here the layers have the widths of LFM2-1.2B
(hidden 2,048, 32 query heads over 8 key/value heads of size 64, feed-forward 8,192 by the sizing rule from
12,288, vocabulary 65,536, pages of 64) with 3 of its 16 layers in the real pattern (conv, conv, attention), so
that the kernels meet the shapes that serving gives them, strung together: a 2,100-token prompt whole (the
paired-SM gate/up product on its default route), its last 32 tokens one by one through the captured decode
graph (key splits, the down projection whose K is cut over a cluster, the 65,536-wide head), portions down to
two tokens, and four requests mixed in a pool so small that pages are used again. A second case has the
widths of LFM2-700M with one attention layer and a 30,000-token prompt in portions of 2,048, then 32 decoded
tokens; its query weights are scaled up so that every query looks at a few far keys rather than at an average
of all of them, and a key that is lost or misplaced shows.

The plain model runs in float64 on the CPU; logits are compared at a few hundred places (every layer but the
last runs the whole sequence there, the last layer and the head the wanted places only). kreasof-ai/akas
replays its real shapes the same way and reports the same four figures: largest error, relative L2 error,
cosine and argmax agreement (src/akas/benchmarking/replay.py:10-92).
"""

import json

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
import tiny
import traces

pytestmark = pytest.mark.gpu

WIDE = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=2048, num_attention_heads=32,
    num_key_value_heads=8, intermediate_size=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
    block_multiple_of=256, vocab_size=65536, num_hidden_layers=3, full_attn_idxs=[2], rope_theta=1000000.0,
    norm_eps=1e-5, conv_L_cache=3, conv_bias=False, tie_embedding=True, max_position_embeddings=128000,
)
LONG = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=1536, num_attention_heads=24,
    num_key_value_heads=8, intermediate_size=10240, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
    block_multiple_of=256, vocab_size=65536, num_hidden_layers=1, full_attn_idxs=[0], rope_theta=1000000.0,
    norm_eps=1e-5, conv_L_cache=3, conv_bias=False, tie_embedding=True, max_position_embeddings=128000,
)
PAGE = 64
# (largest |difference| over largest |reference logit|, relative L2 error, share of rows with the plain model's
# argmax). float32 is the fixed bound of every replay test. The bfloat16 bounds are 1.5 times the worst this test
# measured on a B200: three layers at width 2,048 gave 0.0121 and 0.0097 (argmax 0.957 of the rows: with random
# weights the two largest of 65,536 logits often lie closer than bfloat16 resolves); 30,000 keys gave 0.020 and 0.016.
BOUNDS = {
    ("wide", "float32"): (2e-5, 2e-5, 1.0), ("wide", "bfloat16"): (1.8e-2, 1.5e-2, 0.9),
    ("long", "float32"): (2e-5, 2e-5, 1.0), ("long", "bfloat16"): (3.0e-2, 2.4e-2, 0.9),
}


def _thin(steps, keep):
    """The same steps, wanting logits only at the absolute positions ``keep[request]`` (a set)."""
    at, out = {}, []
    for step in steps:
        entries = []
        for e in step["entries"]:
            start = at.get(e["id"], 0)
            want = [w for w in range(len(e["tokens"])) if start + w in keep[e["id"]]]
            entries.append(dict(id=e["id"], tokens=e["tokens"], want=want))
            at[e["id"]] = start + len(e["tokens"])
        out.append(dict(step=step["step"], entries=entries, end=step["end"]))
    return out


def _figures(got, want):
    """(largest error over largest reference logit, relative L2 error, cosine, share of rows with the same argmax)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = float(np.abs(got - want).max() / np.abs(want).max())
    l2 = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    return err, l2, cos, float((got.argmax(-1) == want.argmax(-1)).mean())


def _compare(got, want, keep, case, dtype, what, report):
    tol, l2_most, same_least = BOUNDS[(case, dtype)]
    for rid in want:
        places = sorted(keep[rid])
        assert got[rid].shape == want[rid].shape, (what, rid, got[rid].shape, want[rid].shape)
        err, l2, cos, same = _figures(got[rid], want[rid])
        report.append(f"{what:28s} {rid:4s} rows {len(places):4d}  max {err:.3g}  L2 {l2:.3g}  cos {cos:.6f}  argmax {same:.3f}")
        bad = traces.first_bad(got[rid], want[rid], tol)
        assert bad is None, f"{what}: request {rid} first differs at position {places[bad]} (max {err:.3g}, L2 {l2:.3g})"
        assert l2 <= l2_most, f"{what}: request {rid}: relative L2 error {l2:.3g}"
        assert same >= same_least, f"{what}: request {rid}: argmax agrees at {same:.3f} of the rows"


def _runner(folder, dtype, tokens, context, graphs):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    return ModelRunner(folder, EngineConfig(dtype=dtype, device="cuda:0", page_size=PAGE, max_tokens=tokens,
                                            max_requests=4, context=context, cuda_graphs=graphs))


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    """The folder, four requests, the places whose logits are compared, and the plain model's logits there."""
    torch.manual_seed(0)
    folder = tiny.make_folder(WIDE, seed=21, std=0.02, dtype="bfloat16", folder=tmp_path_factory.mktemp("wide"))
    cfg, w = plain.load_folder(folder)
    reqs = {f"w{i}": p for i, p in enumerate(tiny.prompts(cfg["vocab_size"], [2100, 520, 130, 300], seed=8))}
    keep = {}
    for rid, toks in reqs.items():
        n = len(toks)
        # the first tokens, a place on each side of every page edge and of the 2,048th token, and the last 40
        places = set(range(min(4, n))) | set(range(max(0, n - 40), n))
        for edge in list(range(PAGE, n, 4 * PAGE)) + [2048]:
            places |= {p for p in (edge - 1, edge) if 0 <= p < n}
        keep[rid] = places
    want = {rid: plain.forward(cfg, w, toks, rows=sorted(keep[rid])).numpy() for rid, toks in reqs.items()}
    return folder, reqs, keep, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_every_way_of_cutting(wide, dtype, capsys):
    folder, reqs, keep, want = wide
    report = []
    # whole prompts, then the last 32 tokens one by one through the captured decode graph, then portions
    runner = _runner(folder, dtype, 4096, 4096, graphs=True)
    for name, steps in (("whole", traces.whole(reqs)), ("last 32 one by one", traces.tail_decoded(reqs, 32)),
                        ("portions down to two", traces.portions(reqs, sizes=(640, 2, 129, 3, 64, 2, 1000, 17, 5, 256)))):
        got = traces.replay(runner, _thin(steps, keep))
        assert not runner.cache.live() and runner.cache.min_free_pages() == runner.cache.num_pages
        _compare(got, want, keep, "wide", dtype, f"{dtype} {name}", report)
    assert runner._graphs and all(g.graph is not None for g in runner._graphs.values())
    if dtype == "bfloat16":
        from akas_b200.ops import cuda

        assert cuda.gemm_pair_status() == 0 and cuda.gemm_tcgen05_status() == 0 and cuda.skinny_status() == 0
        assert cuda.decode_attention_status() == 0 and cuda.prefill_attention_tc_status() == 0
    del runner
    # four live requests, portions of some beside decoded tokens of others, in a pool that holds no more than they need
    prompt_lens = {rid: max(1, len(t) - 12) for rid, t in reqs.items()}
    steps, peak = traces.mixed(reqs, prompt_lens, seed=4, live=4, page=PAGE)
    runner = _runner(folder, dtype, peak, 2176, graphs=False)
    got = traces.replay(runner, _thin(steps, keep))
    assert not runner.cache.live() and runner.cache.min_free_pages() == runner.cache.num_pages
    _compare(got, want, keep, "wide", dtype, f"{dtype} mixed, pages reused", report)
    with capsys.disabled():
        print("\n" + "\n".join(report))


@pytest.fixture(scope="module")
def long_context(tmp_path_factory):
    folder = tiny.make_folder(LONG, seed=22, std=0.02, dtype="bfloat16", folder=tmp_path_factory.mktemp("long"))
    # Queries four times as large: a softmax over 30,000 random keys then rests on a few of them, anywhere in the
    # context, instead of averaging all, so that one lost page or misplaced key changes a logit by far more than rounding.
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(folder / "model.safetensors"))
    tensors["model.layers.0.self_attn.q_layernorm.weight"] = tensors["model.layers.0.self_attn.q_layernorm.weight"] * 4
    save_file(tensors, str(folder / "model.safetensors"))
    cfg, w = plain.load_folder(folder)
    tokens = tiny.prompts(cfg["vocab_size"], [30032], seed=9)[0]
    places = sorted(set(range(2047, 30000, 2048)) | set(range(2048, 30000, 4096)) | set(range(30000, 30032)))
    want = plain.forward(cfg, w, tokens, rows=places).numpy()
    return folder, tokens, places, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_in_portions_then_decoded(long_context, dtype, capsys):
    folder, tokens, places, want = long_context
    steps, at = [], 0
    for size in [2048] * 14 + [30000 - 14 * 2048] + [1] * 32:
        steps.append(dict(step=len(steps), entries=[dict(id="long", tokens=tokens[at:at + size], want=list(range(size)))],
                          end=["long"] if at + size == len(tokens) else []))
        at += size
    keep = {"long": set(places)}
    runner = _runner(folder, dtype, 30080, 30080, graphs=True)
    got = traces.replay(runner, _thin(steps, keep))
    report = []
    _compare(got, {"long": want}, keep, "long", dtype, f"{dtype} 30,000 tokens, then 32", report)
    with capsys.disabled():
        print("\n" + "\n".join(report))
