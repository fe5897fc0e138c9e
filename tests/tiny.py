"""Tiny LFM2 configurations that differ in every size and option, and helpers to make their folders.

A: 4 layers conv/attn/conv/attn, hidden 64, 4 heads over 2 kv heads, head_dim 16, ff 192, vocab 256,
   theta 1e4, eps 1e-5, 3 taps, no bias, tied head, pages of 16.
B: 6 layers with attention at 0, 2 and 5, hidden 96, 3 heads over 1 kv head, head_dim 32, ff 256 (by the
   auto-adjust rule from 384 with multiple 64), vocab 320, theta 1e6, eps 1e-6, 4 taps, bias, untied head,
   pages of 8.
C: the sizes at which the serving kernels take over from the general ones (used on the GPU only): 3 layers
   attn/conv/attn, hidden 128, 2 heads over 1 kv head, head_dim 64, ff 320, vocab 500, 3 taps, tied head, pages
   of 64: tensor-memory prompt attention, tensor-core decode attention with one block-table look-up per tile,
   decode products whose K is cut over a cluster.
"""

import json
import tempfile
from pathlib import Path

import torch

TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, intermediate_size=192, block_auto_adjust_ff_dim=False, vocab_size=256,
    num_hidden_layers=4, layer_types=["conv", "full_attention", "conv", "full_attention"], rope_theta=10000.0,
    norm_eps=1e-5, conv_L_cache=3, conv_bias=False, tie_embedding=True, max_position_embeddings=4096,
)
TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=96, num_attention_heads=3,
    num_key_value_heads=1, intermediate_size=384, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
    block_multiple_of=64, vocab_size=320, num_hidden_layers=6, full_attn_idxs=[0, 2, 5],
    rope_parameters={"rope_theta": 1000000.0}, norm_eps=1e-6, conv_L_cache=4, conv_bias=True, tie_embedding=False,
    max_position_embeddings=4096,
)
TINY_C = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=128, num_attention_heads=2,
    num_key_value_heads=1, intermediate_size=320, block_auto_adjust_ff_dim=False, vocab_size=500,
    num_hidden_layers=3, full_attn_idxs=[0, 2], rope_theta=1000000.0, norm_eps=1e-5, conv_L_cache=3,
    conv_bias=False, tie_embedding=True, max_position_embeddings=4096,
)
PAGE = {"a": 16, "b": 8, "c": 64}
CONFIGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C}


def make_folder(config: dict, seed: int, std: float = 0.05, dtype: str = "float32", folder=None) -> Path:
    """Writes a model folder for ``config`` with the package's random-weights mode; returns its path."""
    from akas_b200.config import config_from_dict
    from akas_b200.weights import write_random_model

    folder = Path(folder or tempfile.mkdtemp(prefix="akas-tiny-"))
    write_random_model(folder, config_from_dict(config), seed=seed, std=std, dtype=dtype)
    # keep the original keys (auto-adjust rule, full_attn_idxs) so that reading them is exercised too
    (folder / "config.json").write_text(json.dumps(config, indent=2))
    return folder


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
