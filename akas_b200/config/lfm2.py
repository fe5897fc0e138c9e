"""Typed configuration of the dense LFM2 decoder, read from its own config.json keys.

The keys, their defaults and the feed-forward sizing rule are those that
kreasof-ai/akas reads (src/akas/models/lfm2/config.py:26-92). Unlike that reader
this one accepts any head size that is a multiple of 16, any ``conv_L_cache >= 2``
and ``conv_bias``; it refuses what the engine cannot compute, naming the key.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple

from .specs import (
    AttentionSpec,
    LayerSpec,
    ModelSpec,
    RMSNormSpec,
    RopeSpec,
    ShortConvSpec,
    SwiGLUSpec,
)

ARCHITECTURE = "Lfm2ForCausalLM"
_LAYER_KINDS = {"full_attention": "attention", "attention": "attention", "conv": "conv"}


class ConfigError(ValueError):
    """config.json asks for something the engine does not build, or contradicts itself."""


@dataclass(frozen=True)
class Lfm2Config:
    hidden_size: int
    feed_forward_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    layer_kinds: Tuple[str, ...]  # "attention" or "conv"
    vocab_size: int
    conv_kernel: int  # conv_L_cache
    conv_bias: bool
    norm_eps: float
    rope_theta: float
    tie_embedding: bool
    max_position_embeddings: int
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading

    @staticmethod
    def feed_forward_width(data: Mapping[str, Any]) -> int:
        """src/akas/models/lfm2/config.py:30-37: int(2F/3), then multiplier and rounding up."""
        ff = data.get("intermediate_size", data.get("block_ff_dim"))
        if type(ff) is not int or ff <= 0:
            raise ConfigError("intermediate_size (or block_ff_dim) must be a positive integer")
        if data.get("block_auto_adjust_ff_dim", False):
            ff = int(2 * ff / 3)
            multiplier = data.get("block_ffn_dim_multiplier")
            if multiplier is not None:
                multiple = data.get("block_multiple_of", 256)
                if type(multiple) is not int or multiple <= 0:
                    raise ConfigError("block_multiple_of must be a positive integer")
                ff = math.ceil(int(multiplier * ff) / multiple) * multiple
        return ff

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Lfm2Config":
        if data.get("model_type", "lfm2") != "lfm2":
            raise ConfigError(f"model_type {data.get('model_type')!r} is not 'lfm2'")
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "vocab_size"):
            if type(data.get(key)) is not int or data[key] <= 0:
                raise ConfigError(f"{key} must be a positive integer, got {data.get(key)!r}")
        hidden, count = data["hidden_size"], data["num_hidden_layers"]
        heads, kv_heads = data["num_attention_heads"], data["num_key_value_heads"]

        kinds = data.get("layer_types")
        if kinds is None:
            idx = data.get("full_attn_idxs")
            if not isinstance(idx, list) or any(type(i) is not int or not 0 <= i < count for i in idx):
                raise ConfigError("layer_types is absent and full_attn_idxs is not a list of layer indices")
            kinds = ["attention" if i in idx else "conv" for i in range(count)]
        unknown = sorted({str(k) for k in kinds} - set(_LAYER_KINDS))
        if unknown:
            raise ConfigError(f"layer_types holds unknown kinds {unknown}; known: {sorted(_LAYER_KINDS)}")
        kinds = tuple(_LAYER_KINDS[k] for k in kinds)
        if len(kinds) != count:
            raise ConfigError(f"layer_types has {len(kinds)} entries but num_hidden_layers is {count}")

        rope = data.get("rope_parameters") or {}
        if rope.get("rope_type", "default") != "default" or data.get("rope_scaling"):
            raise ConfigError("only the default rope type without scaling is built")
        theta = rope.get("rope_theta", data.get("rope_theta", 1000000.0))
        eps = data.get("norm_eps", 1e-5)
        for key, value in (("rope_theta", theta), ("norm_eps", eps)):
            if not isinstance(value, (int, float)) or not math.isfinite(value) or value <= 0:
                raise ConfigError(f"{key} must be a positive finite number, got {value!r}")

        head_dim = data.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        if type(head_dim) is not int or head_dim <= 0 or head_dim % 16 or head_dim > 256:
            raise ConfigError(f"head_dim {head_dim!r} must be a multiple of 16, at most 256")
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        conv = data.get("conv_L_cache", 3)
        if type(conv) is not int or not 2 <= conv <= 16:
            raise ConfigError(f"conv_L_cache {conv!r} must be an integer from 2 to 16")
        if not data.get("block_use_swiglu", True):
            raise ConfigError("block_use_swiglu=false is not built")
        if not data.get("use_pos_enc", True):
            raise ConfigError("use_pos_enc=false is not built")
        context = data.get("max_position_embeddings", 128000)
        if type(context) is not int or context <= 0:
            raise ConfigError("max_position_embeddings must be a positive integer")
        eos = data.get("eos_token_id")
        return cls(
            hidden_size=hidden,
            feed_forward_size=cls.feed_forward_width(data),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            layer_kinds=kinds,
            vocab_size=data["vocab_size"],
            conv_kernel=conv,
            conv_bias=bool(data.get("conv_bias", False)),
            norm_eps=float(eps),
            rope_theta=float(theta),
            tie_embedding=bool(data.get("tie_embedding", data.get("tie_word_embeddings", True))),
            max_position_embeddings=context,
            eos_token_id=eos if type(eos) is int else None,
        )

    @classmethod
    def from_json(cls, path) -> "Lfm2Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        """A config.json that reads back as this configuration."""
        data = dict(
            architectures=[ARCHITECTURE],
            model_type="lfm2",
            hidden_size=self.hidden_size,
            intermediate_size=self.feed_forward_size,
            block_ff_dim=self.feed_forward_size,
            block_auto_adjust_ff_dim=False,
            num_hidden_layers=len(self.layer_kinds),
            layer_types=["full_attention" if k == "attention" else "conv" for k in self.layer_kinds],
            full_attn_idxs=[i for i, k in enumerate(self.layer_kinds) if k == "attention"],
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads,
            vocab_size=self.vocab_size,
            conv_L_cache=self.conv_kernel,
            conv_bias=self.conv_bias,
            norm_eps=self.norm_eps,
            rope_theta=self.rope_theta,
            tie_embedding=self.tie_embedding,
            max_position_embeddings=self.max_position_embeddings,
            torch_dtype="bfloat16",
        )
        if self.head_dim * self.num_attention_heads != self.hidden_size:
            data["head_dim"] = self.head_dim
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # ------------------------------------------------------------------ the model it describes

    def model_spec(self) -> ModelSpec:
        """Layer by layer: operator_norm, mixer, ffn_norm, SwiGLU; Hugging Face tensor names
        (src/akas/models/lfm2/weights.py:445-485)."""
        norm = RMSNormSpec(self.hidden_size, self.norm_eps)
        head_norm = RMSNormSpec(self.head_dim, self.norm_eps)
        rope = RopeSpec(self.head_dim, self.rope_theta)
        layers = []
        for i, kind in enumerate(self.layer_kinds):
            prefix = f"model.layers.{i}."
            if kind == "attention":
                mixer = AttentionSpec(
                    self.hidden_size, self.num_attention_heads, self.num_key_value_heads, self.head_dim,
                    qk_norm=head_norm, position=rope,
                    names={"q_norm.weight": "q_layernorm.weight", "k_norm.weight": "k_layernorm.weight"},
                )
                mixer_prefix = prefix + "self_attn."
            else:
                mixer = ShortConvSpec(self.hidden_size, self.conv_kernel, self.conv_bias)
                mixer_prefix = prefix + "conv."
            layers.append(
                LayerSpec(
                    mixer=mixer,
                    ffn=SwiGLUSpec(self.hidden_size, self.feed_forward_size),
                    mixer_norm=norm,
                    ffn_norm=norm,
                    mixer_prefix=mixer_prefix,
                    ffn_prefix=prefix + "feed_forward.",
                    mixer_norm_name=prefix + "operator_norm.weight",
                    ffn_norm_name=prefix + "ffn_norm.weight",
                )
            )
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            layers=tuple(layers),
            final_norm=norm,
            embedding_name="model.embed_tokens.weight",
            final_norm_name="model.embedding_norm.weight",
            head_name="lm_head.weight",
            head_optional=self.tie_embedding,
            max_context=self.max_position_embeddings,
        )
