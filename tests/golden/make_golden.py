"""Writes tests/golden/lfm2_numpy_reference.npz from the reference project's own CPU model.

    python tests/golden/make_golden.py --reference <checkout of kreasof-ai/akas>

The reference's NumPy LFM2 forward (tests/support/numpy_reference.py:69-187 in that
project) imports and runs on a CPU without its compiler. Its class is built by hand
here (its constructor wants a GGUF file): a directly constructed ``Config``, random
weights under the project's logical tensor names, float32 key/value caches and
float32 projections (``projection_half=False``). It hard-codes a three-tap
convolution without bias, so both golden models have ``conv_L_cache = 3`` and no
bias; in every other size and option they differ from each other.

The file holds, for each model, the token ids and the logits of the last position
for several prompt lengths. Weights are not stored: ``golden_weights`` below draws
them again from the seed, under Hugging Face names.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np

GOLDEN_MODELS = {
    "a": dict(
        seed=1201, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, ff=192, vocab_size=256,
        layer_types=["conv", "full_attention", "conv", "full_attention"], rope_theta=10000.0, norm_eps=1e-5,
        tied=True, lengths=[1, 2, 3, 17, 40],
    ),
    "b": dict(
        seed=1202, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, ff=256, vocab_size=320,
        layer_types=["full_attention", "conv", "full_attention", "conv", "conv", "full_attention"],
        rope_theta=1000000.0, norm_eps=1e-6, tied=False, lengths=[1, 4, 33, 70],
    ),
}


def golden_config(m: dict) -> dict:
    """The config.json of a golden model (block_ff_dim is taken as it stands)."""
    return dict(
        architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=m["hidden_size"],
        num_attention_heads=m["num_attention_heads"], num_key_value_heads=m["num_key_value_heads"],
        intermediate_size=m["ff"], block_auto_adjust_ff_dim=False, vocab_size=m["vocab_size"],
        num_hidden_layers=len(m["layer_types"]), layer_types=list(m["layer_types"]), rope_theta=m["rope_theta"],
        norm_eps=m["norm_eps"], conv_L_cache=3, conv_bias=False, tie_embedding=m["tied"],
    )


def golden_weights(m: dict) -> dict[str, np.ndarray]:
    """Seeded float32 weights under Hugging Face names: N(0, 0.05) matrices, 1 + N(0, 0.1) norms."""
    rng = np.random.default_rng(m["seed"])
    c, f, v = m["hidden_size"], m["ff"], m["vocab_size"]
    h, kh = m["num_attention_heads"], m["num_key_value_heads"]
    d = c // h

    def mat(*shape):
        return rng.normal(0, 0.05, shape).astype(np.float32)

    def vec(n):
        return (1 + rng.normal(0, 0.1, n)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(v, c), "model.embedding_norm.weight": vec(c)}
    if not m["tied"]:
        w["lm_head.weight"] = mat(v, c)
    for i, kind in enumerate(m["layer_types"]):
        p = f"model.layers.{i}."
        w[p + "operator_norm.weight"] = vec(c)
        w[p + "ffn_norm.weight"] = vec(c)
        w[p + "feed_forward.w1.weight"] = mat(f, c)
        w[p + "feed_forward.w3.weight"] = mat(f, c)
        w[p + "feed_forward.w2.weight"] = mat(c, f)
        if kind == "conv":
            w[p + "conv.in_proj.weight"] = mat(3 * c, c)
            w[p + "conv.conv.weight"] = rng.normal(0, 0.3, (c, 1, 3)).astype(np.float32)
            w[p + "conv.out_proj.weight"] = mat(c, c)
        else:
            a = p + "self_attn."
            w[a + "q_proj.weight"] = mat(h * d, c)
            w[a + "k_proj.weight"] = mat(kh * d, c)
            w[a + "v_proj.weight"] = mat(kh * d, c)
            w[a + "out_proj.weight"] = mat(c, h * d)
            w[a + "q_layernorm.weight"] = vec(d)
            w[a + "k_layernorm.weight"] = vec(d)
    return w


def golden_tokens(m: dict) -> np.ndarray:
    return np.random.default_rng(m["seed"] + 7).integers(0, m["vocab_size"], max(m["lengths"])).astype(np.int32)


def _reference_logits(reference_root: Path, m: dict) -> np.ndarray:
    sys.path.insert(0, str(reference_root / "src"))
    sys.path.insert(0, str(reference_root))
    from akas.models.lfm2.config import Config
    from akas.models.lfm2.weights import huggingface_names
    from tests.support.numpy_reference import Reference

    kinds = tuple("attention" if k == "full_attention" else k for k in m["layer_types"])
    config = Config(
        m["hidden_size"], m["ff"], m["num_attention_heads"], m["num_key_value_heads"], kinds, m["vocab_size"],
        3, m["norm_eps"], m["rope_theta"], 4096,
    )
    hf = golden_weights(m)
    names = huggingface_names(config, output=not m["tied"])
    logical = {}
    for name, hf_name in names.items():
        value = hf[hf_name]
        if name.endswith("shortconv.conv.weight"):
            value = value.reshape(value.shape[0], value.shape[-1])
        logical[name] = value
    ref = object.__new__(Reference)
    ref.config = config
    ref.context = 128
    ref.weights = logical
    ref.half_weights = None
    tokens = golden_tokens(m)
    rows = []
    for n in m["lengths"]:
        ref.reset()
        ref.caches = {
            i: (np.zeros((ref.context, config.kv_heads, config.head_dim), np.float32),
                np.zeros((ref.context, config.kv_heads, config.head_dim), np.float32))
            for i in ref.caches
        }
        rows.append(ref._chunk(tokens[:n], projection_half=False))
    return np.stack(rows).astype(np.float32)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", required=True, type=Path, help="checkout of kreasof-ai/akas")
    args = ap.parse_args()
    out = {}
    for key, m in GOLDEN_MODELS.items():
        out[f"{key}_tokens"] = golden_tokens(m)
        out[f"{key}_lengths"] = np.asarray(m["lengths"], np.int32)
        out[f"{key}_logits"] = _reference_logits(args.reference, m)
    target = Path(__file__).with_name("lfm2_numpy_reference.npz")
    np.savez_compressed(target, **out)
    print("wrote", target, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
