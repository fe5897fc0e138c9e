"""Which kernel a product of a prompt portion is given to: the decision is host logic and is tested without a device."""

import pytest

from akas_b200.ops import cuda


def test_products_above_sixteen_tokens_run_on_the_hand_written_kernels(monkeypatch):
    monkeypatch.setattr(cuda, "products", "own")
    route = cuda._product_route
    bf16, f32, acc, swiglu = cuda._OUT_BF16, cuda._OUT_F32, cuda._OUT_ACC, cuda._OUT_SWIGLU
    # the LFM2 shapes: every product goes to the kernel for pairs of SMs
    assert route(2048, 6144, bf16) == "paired" and route(2048, 2048, acc) == "paired" and route(8192, 2048, acc) == "paired"
    assert route(2048, 16384, swiglu) == "paired" and route(2048, 65536, f32) == "paired"
    # rows that TMA cannot write (a pitch that is no multiple of 16 bytes) go to the one-block kernel's masked read-outs
    assert route(64, 500, f32) == "paired" and route(64, 502, f32) == "block" and route(64, 500, bf16) == "block"
    assert route(64, 504, bf16) == "paired" and route(64, 1001, acc) == "block"
    assert route(64, 2 * 24, swiglu) == "paired" and route(64, 2 * 20, swiglu) == "unfused"  # the product, then SwiGLU by itself
    monkeypatch.setattr(cuda, "products", "library")
    assert {route(2048, 2048, m) for m in (bf16, f32, acc, swiglu)} == {"library"}


def test_key_parts_of_decode_attention():
    """Two blocks per SM's worth of (request, KV head) parts, at least two parts, at least four 64-key tiles a part."""
    parts = cuda.decode_splits
    assert parts(8, 8, 1, 4096) == 5 and parts(64, 8, 1, 4096) == 2 and parts(1, 8, 1, 4096) == 16
    assert parts(8, 8, 1, 256) == 1 and parts(8, 8, 1, 700) == 3 and parts(256, 8, 1, 2304) == 2
    assert parts(1, 1, 1, 10 ** 6) == 64
    # the kernel merges its parts itself while the blocks are few: 8 requests yes, 64 requests no (a merge kernel then)
    merged = cuda._merges_in_cluster
    import unittest.mock as mock
    with mock.patch.object(cuda, "_sm_count", return_value=148):
        assert merged(64, 5, 64, 64) and not merged(512, 2, 64, 64) and not merged(64, 16, 64, 64)
        assert not merged(64, 5, 128, 64) and not merged(64, 5, 64, 16)


def test_plan_of_decode_attention():
    """Key parts and which kernel: a block per (token, KV head, key part) while that is at most three blocks per SM, a
    fixed number of blocks that walk those items beyond; up to 8 parts that meet inside their cluster where a part stays
    within 8 tiles, rather than more parts and a merge kernel."""
    import unittest.mock as mock

    import torch

    plan = cuda.decode_plan
    bf16 = torch.bfloat16
    with mock.patch.object(cuda, "_sm_count", return_value=148), mock.patch.object(cuda, "_items_places", return_value=592):
        assert plan(8, 32, 8, 64, 64, 4096, bf16) == (5, False)
        assert plan(1, 32, 8, 64, 64, 4096, bf16) == (8, False)         # 16 parts would need a merge kernel
        assert plan(1, 32, 8, 64, 64, 30000, bf16) == (38, False)       # long parts: as many as fill the GPU
        assert plan(64, 32, 8, 64, 64, 4096, bf16) == (2, True)         # 1,024 items for 444 places
        assert plan(32, 32, 8, 64, 64, 4096, bf16) == (2, True)
        assert plan(16, 32, 8, 64, 64, 4096, bf16) == (3, False)
        assert plan(128, 32, 8, 64, 64, 8192, bf16) == (2, False)       # 2,048 blocks: the hardware spreads them as they come
        assert plan(64, 32, 8, 128, 64, 4096, bf16) == (2, False)       # the TMA-fed kernels take head size 64 only
        assert plan(64, 32, 8, 64, 16, 4096, bf16) == (2, False)        # and pages of whole 64-key tiles
        assert plan(64, 32, 8, 64, 64, 4096, torch.float32) == (2, False)
        with mock.patch.object(cuda, "decode_items", "0"):
            assert plan(64, 32, 8, 64, 64, 4096, bf16) == (2, False)
    with mock.patch.object(cuda, "_sm_count", return_value=148), mock.patch.object(cuda, "_items_places", return_value=0):
        assert plan(64, 32, 8, 64, 64, 4096, bf16) == (2, False)        # the kernel cannot run on this device


def test_reports_are_compared_case_by_case():
    from akas_b200.bench import case_lengths, compare_reports

    row = lambda prefill, decode, **kw: dict(batch=2, prompt=64, generated=8, depth=0, mixed=False,
                                             prefill_tokens_per_s=prefill, decode_tokens_per_s=decode, **kw)
    before, after = dict(rows=[row(1000.0, 100.0)]), dict(rows=[row(950.0, 80.0)])
    change, = compare_reports(after, before, 0.1)
    assert change["regressed"] and abs(change["decode_tokens_per_s_ratio"] - 0.8) < 1e-9
    assert not compare_reports(after, before, 0.25)[0]["regressed"]
    with pytest.raises(ValueError, match="cover every measured case"):
        compare_reports(dict(rows=[dict(row(1.0, 1.0), depth=16)]), before)
    with pytest.raises(ValueError):
        compare_reports(after, before, 1.0)
    assert case_lengths(9, 64, True) == [64, 63, 62, 61, 60, 59, 58, 64, 63] and case_lengths(3, 2, True) == [2, 1, 2]
    assert case_lengths(3, 64, False) == [64, 64, 64]
