"""The command line: the subcommands that need no device (random, inspect) here; generate and bench on the GPU."""

import json

import pytest

import tiny
from akas_b200.cli import main


def _config_text():
    data = dict(tiny.TINY_B)
    data.setdefault("architectures", ["Lfm2ForCausalLM"])
    return json.dumps(data)


def test_random_writes_a_folder_that_inspect_reads(tmp_path, capsys):
    main(["random", "--out", str(tmp_path / "inline"), "--config", _config_text(), "--seed", "4", "--dtype", "float32"])
    (tmp_path / "c.json").write_text(_config_text())
    main(["random", "--out", str(tmp_path / "file"), "--config", str(tmp_path / "c.json"), "--seed", "4", "--dtype", "float32"])
    capsys.readouterr()
    main(["inspect", "--model", str(tmp_path / "inline")])
    report = json.loads(capsys.readouterr().out)
    assert report["architecture"] == "Lfm2ForCausalLM"
    assert report["config"]["vocab_size"] == tiny.TINY_B["vocab_size"]
    assert "model.embed_tokens.weight" in report["inventory"]
    # the same seed gives the same tensors, whichever way the configuration came in
    assert (tmp_path / "inline" / "model.safetensors").read_bytes() == (tmp_path / "file" / "model.safetensors").read_bytes()


def test_prompt_must_be_token_ids(tmp_path):
    with pytest.raises(SystemExit):
        main(["generate", "--model", str(tmp_path), "--prompt", "hello world"])


@pytest.mark.gpu
def test_generate_and_bench_run(tmp_path, capsys):
    main(["random", "--out", str(tmp_path / "m"), "--config", _config_text(), "--seed", "5"])
    capsys.readouterr()
    main(["generate", "--model", str(tmp_path / "m"), "--prompt", "5,17 3", "--max-tokens", "6", "--out", str(tmp_path / "o.json")])
    printed = capsys.readouterr().out.split()
    saved = json.loads((tmp_path / "o.json").read_text())
    assert saved["prompt_tokens"] == [5, 17, 3] and [int(t) for t in printed] == saved["generated_tokens"]
    assert len(saved["generated_tokens"]) <= 6 and saved["finish_reason"] in ("length", "stop")
    main(["generate", "--model", str(tmp_path / "m"), "--prompt", "5 17 3", "--max-tokens", "6", "--temperature", "0.7",
          "--top-k", "20", "--seed", "2", "--dtype", "float32", "--ignore-eos"])
    assert len(capsys.readouterr().out.split()) == 6
    main(["bench", "--model", str(tmp_path / "m"), "--batches", "1", "2", "--prompts", "32", "--generated", "4", "--repeats", "2"])
    report = json.loads(capsys.readouterr().out)
    assert all(row["decode_tokens_per_s"] > 0 and row["prefill_tokens_per_s"] > 0 for row in report["rows"])
    # with tokens cached before the prompt, staggered lengths, and a comparison with an earlier report
    earlier = tmp_path / "earlier.json"
    main(["bench", "--model", str(tmp_path / "m"), "--batches", "3", "--prompts", "20", "--depths", "0", "24", "--mixed",
          "--generated", "3", "--repeats", "1", "--out", str(earlier)])
    report = json.loads(capsys.readouterr().out)
    assert [(row["depth"], row["mixed"]) for row in report["rows"]] == [(0, True), (24, True)]
    main(["bench", "--model", str(tmp_path / "m"), "--batches", "3", "--prompts", "20", "--depths", "0", "24", "--mixed",
          "--generated", "3", "--repeats", "1", "--baseline", str(earlier), "--max-regression", "0.99"])
    changes = json.loads(capsys.readouterr().out)["changes"]
    assert len(changes) == 2 and not any(change["regressed"] for change in changes)
