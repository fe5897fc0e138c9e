"""Weights by tensor name: what is kept in which dtype, and the one error that lists everything wrong."""

import json

import pytest
import torch
from safetensors.torch import load_file as _load_file
from safetensors.torch import save_file

import tiny
from akas_b200.config import config_from_dict
from akas_b200.models import Decoder
from akas_b200.ops import reference
from akas_b200.parts import Runtime
from akas_b200.weights import WeightError, load_weights, random_tensors, write_random_model


def load_file(path):
    """Copies out of the file mapping, so that the file may be rewritten afterwards."""
    return {k: v.clone() for k, v in _load_file(path).items()}


def _model(config, dtype=torch.float32):
    return Decoder(config.model_spec(), Runtime(dtype, torch.device("cpu"), reference))


def test_random_mode_is_seeded_and_complete(tmp_path):
    config = config_from_dict(tiny.TINY_B)
    a, b, c = random_tensors(config, 5, dtype="float32"), random_tensors(config, 5, dtype="float32"), random_tensors(config, 6, dtype="float32")
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert set(a) == {n for n, p in _model(config).params().items() if not p.optional} | {"lm_head.weight"}
    assert a["model.layers.1.conv.conv.weight"].shape == (96, 1, 4) and "model.layers.1.conv.conv.bias" in a
    assert a["model.layers.1.conv.in_proj.bias"].shape == (288,) and a["model.layers.1.conv.out_proj.bias"].shape == (96,)
    assert abs(a["model.layers.0.operator_norm.weight"].mean() - 1) < 0.05
    assert abs(a["model.layers.0.self_attn.q_proj.weight"].std() - 0.02) < 0.005
    folder = write_random_model(tmp_path / "m", config, seed=5)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["Lfm2ForCausalLM"]
    stored = load_file(str(folder / "model.safetensors"))
    assert all(t.dtype == torch.bfloat16 for t in stored.values())


@pytest.mark.parametrize("dtype,stored", [(torch.float32, "bfloat16"), (torch.bfloat16, "float32"), (torch.bfloat16, "bfloat16")])
def test_dtypes_after_loading(tmp_path, dtype, stored):
    config = config_from_dict(tiny.TINY_A)
    folder = write_random_model(tmp_path / "m", config, seed=1, dtype=stored)
    model = _model(config, dtype)
    load_weights(model, folder)
    mixer = model.blocks[1].mixer
    assert mixer.w_qkv.dtype == dtype and model.embedding.dtype == dtype  # operands of matrix products
    assert mixer.q_norm.weight.dtype == torch.float32  # norm weights, taps and biases stay in 32-bit
    assert model.blocks[0].mixer.taps.dtype == torch.float32 and model.blocks[0].mixer.taps.shape == (64, 3)
    assert model.head is model.embedding  # tied
    file = load_file(str(folder / "model.safetensors"))
    assert torch.equal(mixer.w_qkv[:64], file["model.layers.1.self_attn.q_proj.weight"].to(dtype))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = config_from_dict(tiny.TINY_B)
    folder = write_random_model(tmp_path / "m", config, seed=1, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.0.self_attn.k_proj.weight"]
    del tensors["model.embedding_norm.weight"]
    tensors["model.layers.9.ghost.weight"] = torch.zeros(3)
    tensors["model.layers.1.conv.in_proj.weight"] = torch.zeros(5, 96)
    tensors["model.layers.2.ffn_norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as error:
        load_weights(_model(config), folder)
    text = str(error.value)
    for word in ("missing tensors (2)", "model.layers.0.self_attn.k_proj.weight", "model.embedding_norm.weight",
                 "unexpected tensors (1)", "model.layers.9.ghost.weight", "wrong shapes (1)",
                 "model.layers.1.conv.in_proj.weight: checkpoint [5, 96], model [288, 96]", "unusable dtypes (1)"):
        assert word in text, word


def test_conv_bias_means_three_biases(tmp_path):
    """``conv_bias: true`` puts a bias on the in projection, the taps and the out projection; a checkpoint that lacks
    one of the three is refused, and one without the option that carries any is refused too."""
    config = config_from_dict(tiny.TINY_B)
    folder = write_random_model(tmp_path / "m", config, seed=1, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    for lost in ("model.layers.1.conv.in_proj.bias", "model.layers.3.conv.out_proj.bias"):
        kept = {k: v for k, v in tensors.items() if k != lost}
        save_file(kept, str(folder / "model.safetensors"))
        with pytest.raises(WeightError, match=lost.replace(".", r"\.")):
            load_weights(_model(config), folder)
    save_file(tensors, str(folder / "model.safetensors"))
    model = _model(config)
    load_weights(model, folder)
    assert model.blocks[1].mixer.bias_in.shape == (288,) and model.blocks[1].mixer.bias_out.dtype == torch.float32
    plain_config = config_from_dict({**tiny.TINY_B, "conv_bias": False})
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(_model(plain_config), folder)


def test_head_follows_the_checkpoint_as_the_reference_does(tmp_path):
    """Untied but no lm_head.weight: an error. Tied but lm_head.weight present: it is used."""
    untied = config_from_dict(tiny.TINY_B)
    folder = write_random_model(tmp_path / "u", untied, seed=1, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    head = tensors.pop("lm_head.weight")
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(_model(untied), folder)
    tied = config_from_dict({**tiny.TINY_B, "tie_embedding": True})
    model = _model(tied)
    load_weights(model, folder)
    assert model.head is model.embedding
    tensors["lm_head.weight"] = head
    save_file(tensors, str(folder / "model.safetensors"))
    model = _model(tied)
    load_weights(model, folder)
    assert torch.equal(model.head, head)


def test_sharded_folder_and_escaping_shard(tmp_path):
    config = config_from_dict(tiny.TINY_A)
    folder = write_random_model(tmp_path / "m", config, seed=1, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    weight_map = {n: "model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors"
                  for i, n in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    model = _model(config)
    load_weights(model, folder)
    assert torch.equal(model.embedding, tensors["model.embed_tokens.weight"])
    weight_map[names[0]] = "../outside.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(WeightError, match="inside"):
        load_weights(_model(config), folder)
    with pytest.raises(FileNotFoundError):
        load_weights(_model(config), tmp_path)
