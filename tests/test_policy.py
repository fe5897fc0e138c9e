"""Which kernel a product of a prompt portion is given to: the decision is host logic and is tested without a device."""

import pytest

from akas_b200.ops import cuda


@pytest.fixture
def b200(monkeypatch):
    monkeypatch.setattr(cuda, "_sms", 148)
    monkeypatch.setattr(cuda, "products", "auto")
    monkeypatch.setattr(cuda, "paired_sms", "1")
    return monkeypatch


def test_gate_up_route_on_the_lfm2_shapes(b200):
    route = cuda._swiglu_route
    # 1.2B shape: K 2,048, F 8,192
    assert route(512, 2048, 8192) == "library" and route(1024, 2048, 8192) == "library"
    assert route(1536, 2048, 8192) == "paired" and route(2048, 2048, 8192) == "paired" and route(8448, 2048, 8192) == "paired"
    # 700M shape: K 1,536, F 6,912
    assert route(2048, 1536, 6912) == "library" and route(8192, 1536, 6912) == "paired"
    # 350M shape: K 1,024, F 4,608
    assert route(2048, 1024, 4608) == "library" and route(8192, 1024, 4608) == "library"
    # decode steps never come here, and an inner size that is no multiple of 8 cannot be fed by TMA
    assert route(16, 2048, 8192) == "library" and route(2048, 2044, 8192) == "library"


def test_gate_up_route_under_the_switches(b200):
    route = cuda._swiglu_route
    b200.setattr(cuda, "products", "library")
    assert route(2048, 2048, 8192) == "library"
    b200.setattr(cuda, "products", "tcgen05")
    assert route(2048, 2048, 8192) == "paired" and route(64, 2048, 8192) == "block"  # too few tiles for 74 pairs
    b200.setattr(cuda, "paired_sms", "0")
    assert route(2048, 2048, 8192) == "block"
    b200.setattr(cuda, "products", "auto")
    assert route(2048, 2048, 8192) == "block" and route(1536, 2048, 8192) == "library"


def test_plain_products_go_to_the_library_unless_told_otherwise(b200):
    assert not cuda._tcgen05_takes(2048, 2048)
    b200.setattr(cuda, "products", "tcgen05")
    assert cuda._tcgen05_takes(2048, 2048) and not cuda._tcgen05_takes(16, 2048) and not cuda._tcgen05_takes(2048, 2044)


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
