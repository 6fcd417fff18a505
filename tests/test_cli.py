"""The command line's parts that need no GPU: usage errors, the random-weights writer, what
`info` reports, and that `replay` is the trace replay program with its own options."""

from __future__ import annotations

import json

from cases import TINY_A
from ayaka_b200 import cli


def test_no_command_is_a_usage_error(capsys):
    assert cli.main([]) == cli.EXIT_USAGE
    assert "run" in capsys.readouterr().err


def test_random_writes_a_model_folder(tmp_path, capsys):
    config = tmp_path / "config.json"
    config.write_text(json.dumps({**TINY_A, "architectures": ["GPT2LMHeadModel"]}))
    out = tmp_path / "model"
    assert cli.main(["random", str(config), str(out), "--seed", "3"]) == cli.EXIT_OK
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    assert cli.main(["random", str(tmp_path / "missing.json"), str(out)]) == cli.EXIT_MISSING
    capsys.readouterr()


def test_info_reports_architectures_parts_and_sources(capsys):
    assert cli.main(["info", "--output", "json"]) == cli.EXIT_OK
    report = json.loads(capsys.readouterr().out)
    assert report["architectures"] == ["GPT2LMHeadModel"]
    assert "attention" in report["parts"]["mixer"] and "dense" in report["parts"]["feed_forward"]
    assert "layer_norm" in report["parts"]["norm"] and "learned" in report["parts"]["position"]
    assert {"gemm_tc", "attention_decode", "norm", "sampling"} <= set(report["cuda_sources"])
    assert cli.main(["info"]) == cli.EXIT_OK
    assert "architectures: GPT2LMHeadModel" in capsys.readouterr().out


def test_replay_takes_the_replay_programs_options(tmp_path, capsys):
    # a missing required option is the replay program's usage error ...
    assert cli.main(["replay", "--model", str(tmp_path)]) == 2
    assert "--dtype" in capsys.readouterr().err
    # ... and its help lists them
    assert cli.main(["replay", "--help"]) == 0
    assert "--max-tokens" in capsys.readouterr().out


def test_run_refuses_a_prompt_that_is_no_token_ids(tmp_path, capsys):
    folder = tmp_path / "model"
    folder.mkdir()
    assert cli.main(["run", str(folder), "-p", "hello"]) == cli.EXIT_USAGE
    assert "token ids" in capsys.readouterr().err
    assert cli.main(["run", str(tmp_path / "none"), "-p", "1 2"]) == cli.EXIT_MISSING
    capsys.readouterr()
