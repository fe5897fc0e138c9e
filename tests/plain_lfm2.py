"""A plain, slow LFM2 forward pass: whole sequences, no cache, one function per part.

It is the oracle of the test-suite. It shares no code with the ``akas_b200``
package: it reads ``config.json`` keys and safetensors names by itself and
computes everything with ordinary torch tensor expressions in float64 (or any
dtype the caller asks for). Each function cites the file of kreasof-ai/akas whose
formula it restates (paths are relative to that project's root).

``tests/golden/`` holds outputs of the reference project's own NumPy model for a
tiny random model; ``tests/test_plain_reference.py`` checks this file against
them, so the formulas here do not rest on a reading of the sources alone. Two
options have no counterpart that runs in the reference (``conv_L_cache != 3``
and ``conv_bias``): those rest on the formulas cited at ``short_conv``; ``conv_bias``
is read as the architecture's three biases (projection in, taps, projection out).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- config


def feed_forward_width(cfg: dict) -> int:
    """SwiGLU width from config.json. src/akas/models/lfm2/config.py:30-37."""
    ff = cfg.get("intermediate_size", cfg.get("block_ff_dim"))
    if cfg.get("block_auto_adjust_ff_dim", False):
        ff = int(2 * ff / 3)
        mult = cfg.get("block_ffn_dim_multiplier")
        if mult is not None:
            multiple = cfg.get("block_multiple_of", 256)
            ff = math.ceil(int(mult * ff) / multiple) * multiple
    return ff


def layer_kinds(cfg: dict) -> list[str]:
    """'attention' or 'conv' per layer. src/akas/models/lfm2/config.py:38-47."""
    kinds = cfg.get("layer_types")
    if kinds is None:
        idx = cfg["full_attn_idxs"]
        kinds = ["attention" if i in idx else "conv" for i in range(cfg["num_hidden_layers"])]
    return ["attention" if k in ("full_attention", "attention") else k for k in kinds]


def rope_theta(cfg: dict) -> float:
    """src/akas/models/lfm2/config.py:48,60."""
    rope = cfg.get("rope_parameters") or {}
    return float(rope.get("rope_theta", cfg.get("rope_theta", 1000000.0)))


def head_dim(cfg: dict) -> int:
    """src/akas/models/lfm2/config.py:22-24 (an explicit head_dim key wins here)."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w. src/akas/ops/normalization/kernel.py:440-444."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rope_tables(positions: torch.Tensor, dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """theta_i = pos * base^(-2i/d), i in [0, d/2). src/akas/ops/attention/kernel.py:814,927-939.

    The reference forms this product with compensated float32 arithmetic so that
    it stays accurate at long positions; float64 gives the same value directly.
    """
    i = torch.arange(dim // 2, dtype=torch.float64)
    freq = torch.tensor(theta, dtype=torch.float64) ** (-2.0 * i / dim)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (i, i + d/2). x: [T, heads, d]. src/akas/ops/attention/kernel.py:975-992."""
    half = x.shape[-1] // 2
    left, right = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((left * c - right * s, left * s + right * c), dim=-1)


def short_conv(x, in_proj, conv_weight, conv_bias, out_proj, in_bias=None, out_bias=None):
    """Gated causal depthwise short convolution over one whole sequence.

    x: [T, C]; in_proj: [3C, C]; conv_weight: [C, L]; conv_bias: [C] or None;
    out_proj: [C, C]; in_bias: [3C] or None; out_bias: [C] or None (LFM2's ``conv_bias`` option gives all three
    biases or none; the reference refuses the option, src/akas/models/lfm2/config.py:87, so the two projection
    biases are plain linear-layer biases: added to the product). The projection's three parts are B, C-gate, x in that order;
    u = B*x; tap L-1 multiplies the current token, earlier taps the earlier u (zero
    before the sequence starts); the C gate multiplies the tap sum.
    src/akas/ops/convolution/kernel.py:43-91 (general L), with the bias added to the
    tap sum before the gate as in src/akas/ops/convolution/kernel.py:318-333.
    """
    T, C = x.shape
    L = conv_weight.shape[1]
    bcx = x @ in_proj.T
    if in_bias is not None:
        bcx = bcx + in_bias
    b, gate, xv = bcx[:, :C], bcx[:, C : 2 * C], bcx[:, 2 * C :]
    u = b * xv
    padded = torch.cat((torch.zeros(L - 1, C, dtype=x.dtype), u), dim=0)
    acc = torch.zeros_like(u)
    for j in range(L):
        acc = acc + padded[j : j + T] * conv_weight[:, j]
    if conv_bias is not None:
        acc = acc + conv_bias
    out = (gate * acc) @ out_proj.T
    return out if out_bias is None else out + out_bias


def attention(x, wq, wk, wv, wo, q_norm, k_norm, eps, heads, kv_heads, dim, theta, window=None, rotary=None, rows=None):
    """GQA attention over one whole sequence with per-head QK RMSNorm, then RoPE.

    ``rotary`` (not an option of LFM2): only the first ``rotary`` channels of each head are rotated, with
    frequencies base^(-2i/rotary) and pairs (i, i + rotary/2); the rest pass through
    (src/akas/ops/attention/kernel.py:1301-1337).
    ``rows``: compute the output for these query positions only (keys and values are still those of the whole
    sequence); the result then has ``len(rows)`` rows.

    Query head H reads KV head H // (heads / kv_heads); scale d^-0.5; key j visible
    to query t iff j <= t (and j > t - window when a window is given).
    src/akas/models/lfm2/_composition.py:234-307; src/akas/ops/attention/kernel.py:589-699;
    tests/support/numpy_reference.py:138-173.
    """
    T = x.shape[0]
    at = torch.arange(T) if rows is None else torch.as_tensor(rows, dtype=torch.long)
    q = (x[at] @ wq.T).reshape(len(at), heads, dim)
    k = (x @ wk.T).reshape(T, kv_heads, dim)
    v = (x @ wv.T).reshape(T, kv_heads, dim)
    q = rms_norm(q, q_norm, eps)
    k = rms_norm(k, k_norm, eps)
    pos = torch.arange(T)
    rot = dim if rotary is None else rotary
    cos, sin = rope_tables(pos, rot, theta, x.dtype)
    q = torch.cat((apply_rope(q[..., :rot], cos[at], sin[at]), q[..., rot:]), dim=-1)
    k = torch.cat((apply_rope(k[..., :rot], cos, sin), k[..., rot:]), dim=-1)
    group = heads // kv_heads
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * (dim ** -0.5)
    visible = pos[None, :] <= at[:, None]
    if window is not None:
        visible &= pos[None, :] > at[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    prob = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", prob, v).reshape(len(at), heads * dim)
    return out @ wo.T


def swiglu(x, w1, w3, w2):
    """silu(x W1^T) * (x W3^T), then W2. src/akas/ops/activation/kernel.py:86-90."""
    gate = x @ w1.T
    up = x @ w3.T
    return (gate / (1 + torch.exp(-gate)) * up) @ w2.T


# --------------------------------------------------------------------------- model


def load_folder(folder, dtype=torch.float64):
    """config.json as a dict and every tensor of model.safetensors in ``dtype``."""
    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {k: v.to(dtype) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, weights


def forward(cfg: dict, w: dict, tokens, window=None, rows=None) -> torch.Tensor:
    """Logits at every position of one sequence: [T, vocab]; with ``rows``, at those positions only: [len(rows), vocab]
    (every layer but the last still runs the whole sequence; the last one, the final norm and the head run the rows).

    src/akas/models/lfm2/_composition.py:108-380: embedding; per layer
    h += mixer(norm(h)); h += ffn(norm(h)); final norm; head (lm_head.weight when
    the checkpoint has it, else the embedding).
    """
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(cfg.get("norm_eps", 1e-5))
    heads, kv_heads, dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim(cfg)
    theta = rope_theta(cfg)
    h = w["model.embed_tokens.weight"][tokens]
    kinds = layer_kinds(cfg)
    sel = None if rows is None else torch.as_tensor(rows, dtype=torch.long)
    for i, kind in enumerate(kinds):
        p = f"model.layers.{i}."
        last = sel is not None and i == len(kinds) - 1
        x = rms_norm(h, w[p + "operator_norm.weight"], eps)
        if kind == "conv":
            cw = w[p + "conv.conv.weight"]
            cw = cw.reshape(cw.shape[0], cw.shape[-1])
            mixed = short_conv(
                x, w[p + "conv.in_proj.weight"], cw, w.get(p + "conv.conv.bias"), w[p + "conv.out_proj.weight"],
                w.get(p + "conv.in_proj.bias"), w.get(p + "conv.out_proj.bias"),
            )
            if last:
                mixed = mixed[sel]
        else:
            a = p + "self_attn."
            mixed = attention(
                x, w[a + "q_proj.weight"], w[a + "k_proj.weight"], w[a + "v_proj.weight"],
                w[a + "out_proj.weight"], w[a + "q_layernorm.weight"], w[a + "k_layernorm.weight"],
                eps, heads, kv_heads, dim, theta, window, rows=sel if last else None,
            )
        h = (h[sel] if last else h) + mixed
        x = rms_norm(h, w[p + "ffn_norm.weight"], eps)
        f = p + "feed_forward."
        h = h + swiglu(x, w[f + "w1.weight"], w[f + "w3.weight"], w[f + "w2.weight"])
    if sel is not None and not kinds:
        h = h[sel]
    x = rms_norm(h, w["model.embedding_norm.weight"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ head.T


def greedy(cfg: dict, w: dict, prompt, max_tokens: int) -> list[int]:
    """Greedy continuation by whole-sequence recomputation; ties go to the lowest id.

    src/akas/ops/vocabulary/kernel.py:146-150.
    """
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(cfg, w, seq)[-1]
        token = int(torch.nonzero(logits == logits.max())[0])
        out.append(token)
        seq.append(token)
    return out
