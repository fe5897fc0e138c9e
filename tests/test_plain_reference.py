"""The plain implementation against outputs of the reference project's own NumPy model, and its parts
against direct restatements of the formulas."""

from pathlib import Path

import numpy as np
import torch

import plain_lfm2 as plain
from golden.make_golden import GOLDEN_MODELS, golden_config, golden_tokens, golden_weights

GOLDEN = Path(__file__).parent / "golden" / "lfm2_numpy_reference.npz"


def test_plain_matches_the_reference_numpy_model():
    data = np.load(GOLDEN)
    for key, m in GOLDEN_MODELS.items():
        cfg = golden_config(m)
        w = {k: torch.from_numpy(v).double() for k, v in golden_weights(m).items()}
        tokens = golden_tokens(m)
        assert np.array_equal(tokens, data[f"{key}_tokens"])
        whole = plain.forward(cfg, w, tokens).numpy()
        for n, want in zip(data[f"{key}_lengths"], data[f"{key}_logits"]):
            got = plain.forward(cfg, w, tokens[:n])[-1].numpy()
            assert np.abs(got - want).max() < 5e-6 * max(1.0, np.abs(want).max()), (key, n)
            assert np.abs(whole[n - 1] - got).max() < 1e-12  # causal: a prefix does not see what follows


def test_short_conv_is_the_recurrence_of_the_reference_kernel():
    """src/akas/ops/convolution/kernel.py:66-88 in kreasof-ai/akas, for L = 4 with a bias."""
    g = torch.Generator().manual_seed(0)
    T, C, L = 9, 6, 4
    x = torch.randn(T, C, generator=g, dtype=torch.float64)
    w_in, w_out = torch.randn(3 * C, C, generator=g, dtype=torch.float64), torch.randn(C, C, generator=g, dtype=torch.float64)
    taps, bias = torch.randn(C, L, generator=g, dtype=torch.float64), torch.randn(C, generator=g, dtype=torch.float64)
    got = plain.short_conv(x, w_in, taps, bias, w_out)
    bcx = x @ w_in.T
    hist = torch.zeros(L - 1, C, dtype=torch.float64)
    rows = []
    for t in range(T):
        cur = bcx[t, :C] * bcx[t, 2 * C:]
        acc = bias + cur * taps[:, L - 1]
        for i in range(L - 1):
            acc = acc + hist[i] * taps[:, i]
        rows.append(bcx[t, C:2 * C] * acc)
        hist = torch.cat((hist[1:], cur[None]))
    assert torch.allclose(got, torch.stack(rows) @ w_out.T, atol=1e-12)


def test_rope_pairs_i_with_i_plus_half():
    pos = torch.tensor([0, 3])
    cos, sin = plain.rope_tables(pos, 8, 10000.0, torch.float64)
    x = torch.arange(16, dtype=torch.float64).reshape(2, 1, 8)
    y = plain.apply_rope(x, cos, sin)
    assert torch.equal(y[0], x[0])  # position 0 rotates nothing
    for i in range(4):
        th = 3 * 10000.0 ** (-2 * i / 8)
        a, b = x[1, 0, i], x[1, 0, i + 4]
        assert abs(y[1, 0, i] - (a * np.cos(th) - b * np.sin(th))) < 1e-12
        assert abs(y[1, 0, i + 4] - (a * np.sin(th) + b * np.cos(th))) < 1e-12


def test_window_hides_old_keys():
    g = torch.Generator().manual_seed(1)
    C, H, KH, D = 32, 4, 2, 8
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, wq, wk, wv, wo = r(12, C), r(H * D, C), r(KH * D, C), r(KH * D, C), r(C, H * D)
    qn, kn = torch.ones(D, dtype=torch.float64), torch.ones(D, dtype=torch.float64)
    full = plain.attention(x, wq, wk, wv, wo, qn, kn, 1e-5, H, KH, D, 1e4)
    win = plain.attention(x, wq, wk, wv, wo, qn, kn, 1e-5, H, KH, D, 1e4, window=5)
    assert torch.allclose(full[:5], win[:5]) and not torch.allclose(full[5:], win[5:])
    tail = plain.attention(x[3:], wq, wk, wv, wo, qn, kn, 1e-5, H, KH, D, 1e4, window=5)
    # relative positions only: the last query of a window of 5 sees the same keys in both runs
    assert torch.allclose(win[-1], tail[-1], atol=1e-9)


def test_greedy_breaks_ties_to_the_lowest_id():
    cfg = golden_config(GOLDEN_MODELS["a"])
    w = {k: torch.from_numpy(v).double() for k, v in golden_weights(GOLDEN_MODELS["a"]).items()}
    w["model.embed_tokens.weight"][7] = w["model.embed_tokens.weight"][3]  # two ids with equal logits everywhere
    logits = plain.forward(cfg, w, [1, 2])[-1]
    assert logits[3] == logits[7]
    w["model.embedding_norm.weight"] *= 0  # every logit equal: the lowest id wins
    assert plain.greedy(cfg, w, [1, 2], 2) == [0, 0]
