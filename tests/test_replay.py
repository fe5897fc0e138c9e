"""The step function against the plain implementation, under every way of cutting and batching.

The same tests run twice: on a CPU with the plain PyTorch statements of the kernels (they check the
host logic: batches, pages, slots), and, marked ``gpu``, with the compiled kernels in float32 and in
bfloat16. Tolerances are fixed: float32 results agree with the float64 plain model to rounding;
bfloat16 results carry the rounding of activations to 8 bits of mantissa between kernels.
"""

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
import tiny
import traces

# largest |difference| over largest |reference logit|, per dtype. bfloat16: the bound of a single position; whole
# requests are held to BF16 below.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
# bfloat16 against the float64 plain model, per tiny configuration: (largest |difference| over largest |reference|,
# relative L2 error of a request's logits, share of positions whose argmax is the plain model's). The first is 1.5 times
# what the kernels measure on a B200 (a and b 1.00e-2, c 1.27e-2, in every way of cutting); the L2 bound is the same for
# all (measured 7.7e-3, 7.2e-3, 9.3e-3); the argmax agreement is measured at 0.988 to 0.993.
BF16 = {"a": (1.5e-2, 1e-2, 0.97), "b": (1.5e-2, 1e-2, 0.97), "c": (1.9e-2, 1e-2, 0.97)}
LENGTHS = {"a": [1, 40, 33, 70, 17, 100, 64, 129], "b": [70, 1, 5, 96, 48, 130, 9], "c": [300, 65, 1, 129, 260, 40]}


def _runner(folder, dtype, device, page, max_tokens, ops=None, max_requests=4, context=None):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    cfg = EngineConfig(dtype=dtype, device=device, page_size=page, max_tokens=max_tokens, max_requests=max_requests,
                       context=context or max_tokens, cuda_graphs=False)
    return ModelRunner(folder, cfg, ops=ops)


def _setup(key, dtype, tmp_path):
    folder = tiny.make_folder(tiny.CONFIGS[key], seed={"a": 11, "b": 12, "c": 13}[key], dtype=dtype, folder=tmp_path / key)
    cfg, w = plain.load_folder(folder)
    reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(cfg["vocab_size"], LENGTHS[key], seed=5))}
    want = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    return folder, reqs, want


def _check(got, want, dtype, what, key="c"):
    most, l2_most, agree_least = (TOL[dtype], TOL[dtype], 1.0) if dtype == "float32" else BF16[key]
    same = total = 0
    for rid in want:
        err, l2 = traces.worst(got[rid], want[rid])
        bad = traces.first_bad(got[rid], want[rid], most)
        assert bad is None, f"{what}: request {rid} first differs at position {bad} (max {err:.3g}, L2 {l2:.3g})"
        assert l2 <= l2_most, f"{what}: request {rid} has relative L2 error {l2:.3g} > {l2_most}"
        same += int((np.argmax(got[rid], -1) == np.argmax(want[rid], -1)).sum())
        total += len(want[rid])
    if dtype != "float32":  # in float32 an argmax may differ where two logits are equal to rounding
        assert same >= agree_least * total, f"{what}: argmax agrees at {same} of {total} positions"


def _run_modes(key, dtype, device, ops, tmp_path, modes):
    folder, reqs, want = _setup(key, dtype, tmp_path)
    page = tiny.PAGE[key]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    for mode in modes:
        if mode == "mixed":
            prompt_lens = {rid: max(1, len(t) - 9) for rid, t in reqs.items()}
            steps, peak = traces.mixed(reqs, prompt_lens, seed=3, live=4, page=page)
            runner = _runner(folder, dtype, device, page, peak, ops, context=longest)
        else:
            steps = getattr(traces, mode)(reqs)
            runner = _runner(folder, dtype, device, page, longest, ops)
        got = traces.replay(runner, steps)
        assert not runner.cache.live()
        assert runner.cache.min_free_pages() == runner.cache.num_pages
        _check(got, want, dtype, f"{key}/{dtype}/{mode}", key)


MODES = ["whole", "tail_decoded", "portions", "mixed"]


@pytest.mark.parametrize("key", ["a", "b"])
def test_replay_host_logic_on_cpu(key, tmp_path):
    from akas_b200.ops import reference

    _run_modes(key, "float32", "cpu", reference, tmp_path, MODES)


def test_a_step_that_cannot_run_leaves_no_request_behind(tmp_path):
    """Every entry is checked before anybody is admitted; when the pages run out while the step's requests are being
    given theirs, the requests that this very step brought in are released again, and the others keep what they had."""
    from akas_b200.cache.manager import OutOfPages
    from akas_b200.engine.batch import StepEntry
    from akas_b200.ops import reference

    folder = tiny.make_folder(tiny.CONFIGS["a"], seed=11, dtype="float32", folder=tmp_path / "a")
    page = tiny.PAGE["a"]
    runner = _runner(folder, "float32", "cpu", page, 3 * page, reference, context=3 * page)
    free = runner.cache.free_pages()
    with pytest.raises(ValueError, match="wanted places"):
        runner.step([StepEntry("a", [1, 2, 3], (0,)), StepEntry("b", [4, 5], (7,))])
    assert not runner.cache.live() and runner.cache.free_pages() == free
    with pytest.raises(OutOfPages):  # "a" takes two pages, "b" would need two more
        runner.step([StepEntry("a", list(range(2 * page)), ()), StepEntry("b", list(range(page + 1)), ())])
    assert not runner.cache.live() and runner.cache.free_pages() == free
    runner.step([StepEntry("c", [1, 2], ())])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("c", [3], ()), StepEntry("d", list(range(3 * page)), ())])
    assert runner.cache.live() == ["c"] and runner.cache.length("c") == 2
    logits = runner.step([StepEntry("c", [3], (0,))])  # and "c" goes on where it was
    want = plain.forward(*plain.load_folder(folder), [1, 2, 3]).numpy()[-1:]
    assert traces.first_bad(logits.numpy(), want, TOL["float32"]) is None
    runner.release("c")
    assert runner.cache.free_pages() == free


@pytest.mark.gpu
def test_logits_of_a_captured_step_last_until_the_next_step(tmp_path):
    """A step that replays a captured graph returns the graph's own output buffer: the next step of that shape
    overwrites it. Whoever wants the logits longer clones them; without graphs every step returns a tensor of its own."""
    from akas_b200.config import EngineConfig
    from akas_b200.engine.batch import StepEntry
    from akas_b200.engine.runner import ModelRunner

    folder = tiny.make_folder(tiny.CONFIGS["a"], seed=11, dtype="float32", folder=tmp_path / "a")
    cfg, w = plain.load_folder(folder)
    page = tiny.PAGE["a"]
    want = plain.forward(cfg, w, [5, 6, 7, 8, 9]).numpy()
    for graphs in (True, False):
        runner = ModelRunner(folder, EngineConfig(dtype="float32", device="cuda:0", page_size=page, max_tokens=4 * page,
                                                  max_requests=2, context=4 * page, cuda_graphs=graphs))
        runner.step([StepEntry("r", [5, 6, 7], ())])
        first = runner.step([StepEntry("r", [8], (0,))])
        kept = first.clone()
        second = runner.step([StepEntry("r", [9], (0,))])
        assert traces.first_bad(kept.cpu().numpy(), want[3:4], TOL["float32"]) is None
        assert traces.first_bad(second.cpu().numpy(), want[4:5], TOL["float32"]) is None
        if graphs:
            assert first.data_ptr() == second.data_ptr() and torch.equal(first, second) and not torch.equal(first, kept)
        else:
            assert first.data_ptr() != second.data_ptr() and torch.equal(first, kept)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b", "c"])
@pytest.mark.parametrize("mode", MODES)
def test_replay_gpu(key, dtype, mode, tmp_path):
    _run_modes(key, dtype, "cuda:0", None, tmp_path, [mode])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ways_of_cutting_agree_with_each_other(dtype, tmp_path):
    """Whole, decoded, portioned and mixed runs of the same request differ by rounding only."""
    folder, reqs, want = _setup("a", dtype, tmp_path)
    page = tiny.PAGE["a"]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    base = traces.replay(_runner(folder, dtype, "cuda:0", page, longest), traces.whole(reqs))
    tol = 5e-6 if dtype == "float32" else TOL[dtype]
    for mode in ("tail_decoded", "portions"):
        got = traces.replay(_runner(folder, dtype, "cuda:0", page, longest), getattr(traces, mode)(reqs))
        for rid in reqs:
            assert traces.first_bad(got[rid], base[rid], tol) is None, (mode, rid, traces.worst(got[rid], base[rid]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b", "c"])
def test_captured_steps_agree_with_the_plain_model(key, dtype, tmp_path):
    """With graphs on: the same traces, so that single-token steps replay the captured decode graphs, and a trace of
    equal portions (two requests side by side, ten tokens each per step), whose step shape repeats and is captured
    after its second appearance. Captured or not, the logits are the plain model's."""
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    folder, reqs, want = _setup(key, dtype, tmp_path)
    page = tiny.PAGE[key]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page

    def runner(tokens):
        return ModelRunner(folder, EngineConfig(dtype=dtype, device="cuda:0", page_size=page, max_tokens=tokens,
                                                max_requests=4, context=longest, cuda_graphs=True))

    r = runner(longest)
    _check(traces.replay(r, traces.tail_decoded(reqs)), want, dtype, "tail decoded, captured", key)
    assert r._graphs and all(g.graph is not None for g in r._graphs.values())

    # the two longest requests side by side in portions of ten tokens, logits wanted at the last two places of each
    a, b = sorted(reqs, key=lambda rid: -len(reqs[rid]))[:2]
    n = min(len(reqs[a]), len(reqs[b])) // 10 * 10
    steps = [{"step": i, "entries": [{"id": rid, "tokens": reqs[rid][at:at + 10], "want": [8, 9]} for rid in (a, b)],
              "end": [a, b] if at + 10 >= n else []} for i, at in enumerate(range(0, n, 10))]
    r = runner(2 * longest)
    got = traces.replay(r, steps)
    assert len(r._shape_graphs) == 1 and next(iter(r._shape_graphs.values())).graph is not None
    for rid in (a, b):
        places = [p for at in range(0, n, 10) for p in (at + 8, at + 9)]
        bad = traces.first_bad(got[rid], want[rid][places], TOL[dtype])
        assert bad is None, (rid, bad, traces.worst(got[rid], want[rid][places]))


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["a", "b", "c"])
def test_prompts_run_on_the_hand_written_products_and_agree_with_the_library(key, tmp_path, monkeypatch):
    """By default every product of more than 16 tokens runs on the tcgen05 kernels (for pairs of SMs where TMA can write
    the rows, the one-block kernel where it cannot: configuration b has a vocabulary whose rows it cannot); nothing
    reaches the library. With the library in their place the logits are the plain model's too."""
    from akas_b200.ops import cuda

    calls = {"paired": 0}
    paired = cuda.paired_product

    def counted(*args, **kwargs):
        calls["paired"] += 1
        return paired(*args, **kwargs)

    def refused(*args, **kwargs):
        raise AssertionError("a product reached the library")

    monkeypatch.setattr(cuda, "paired_product", counted)
    library = cuda._functions.get("akas_gemm_bf16")
    monkeypatch.setitem(cuda._functions, "akas_gemm_bf16", refused)
    _run_modes(key, "bfloat16", "cuda:0", None, tmp_path, ["whole", "portions"])
    assert calls["paired"] > 0
    assert cuda.gemm_pair_status() == 0 and cuda.gemm_tcgen05_status() == 0
    if library is not None:
        monkeypatch.setitem(cuda._functions, "akas_gemm_bf16", library)
    else:
        monkeypatch.delitem(cuda._functions, "akas_gemm_bf16")
    monkeypatch.setattr(cuda, "products", "library")
    _run_modes(key, "bfloat16", "cuda:0", None, tmp_path / "library", ["whole"])


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["a", "b", "c"])
@pytest.mark.parametrize("graphs", [False, True])
def test_decode_steps_as_chains_agree_with_the_plain_model(key, graphs, tmp_path, monkeypatch):
    """With AKAS_B200_DECODE_CHAIN=1 the products, convolutions and embedding of a decode step run as persistent
    launches with grid-wide barriers between operations (csrc/decode_chain.cu), cut where an attention layer needs its
    own kernels; eagerly and inside captured graphs the logits are the plain model's, and no bounded wait runs out."""
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner
    from akas_b200.ops import cuda

    monkeypatch.setattr(cuda, "decode_chain", "1")
    folder, reqs, want = _setup(key, "bfloat16", tmp_path)
    page = tiny.PAGE[key]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    runner = ModelRunner(folder, EngineConfig(dtype="bfloat16", device="cuda:0", page_size=page, max_tokens=4 * longest,
                                              max_requests=4, context=longest, cuda_graphs=graphs))
    before = cuda.launch_count
    _check(traces.replay(runner, traces.tail_decoded(reqs)), want, "bfloat16", "tail decoded, chained", key)
    prompt_lens = {rid: max(1, len(t) - 9) for rid, t in reqs.items()}
    steps, _ = traces.mixed(reqs, prompt_lens, seed=3, live=4, page=page)
    _check(traces.replay(runner, steps), want, "bfloat16", "mixed, chained", key)
    assert cuda.chain_status() == 0 and cuda.launch_count > before


@pytest.mark.gpu
def test_timed_operations_change_nothing_and_account_for_the_step(tmp_path):
    """The wrapper that brackets every operation with CUDA events runs the same kernels: same logits, and a table
    that names the operations of a prompt and of a decoded token."""
    from akas_b200.ops import cuda
    from akas_b200.ops.timed import TimedOps

    folder, reqs, want = _setup("c", "bfloat16", tmp_path)
    page = tiny.PAGE["c"]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    cuda.require(cuda.libraries_for(torch.bfloat16))
    timed = TimedOps(cuda)
    got = traces.replay(_runner(folder, "bfloat16", "cuda:0", page, longest, timed), traces.tail_decoded(reqs))
    _check(got, want, "bfloat16", "timed operations")
    rows = {row["op"]: row for row in timed.table()}
    assert {"embedding", "paged_attention", "short_conv", "linear"} <= set(rows)
    assert all(row["calls"] > 0 and row["ms"] > 0 for row in rows.values())
    assert abs(sum(row["share"] for row in rows.values()) - 1.0) < 1e-6
    timed.clear()
    assert timed.table() == []
