"""Command line pieces that need no GPU: help, random, show, argument errors."""
import json
import os

import pytest

from cima_b200.cli import main


def test_help_random_show(tmp_path, capsys):
    assert main(["help"]) == 0
    assert "cima run <MODEL_DIR>" in capsys.readouterr().out
    assert main(["run", "--help"]) == 0
    out = capsys.readouterr().out
    assert "--temperature" in out and "--max-tokens" in out
    d = str(tmp_path / "m")
    assert main(["random", d, "--shape", "tiny-b", "--seed", "4"]) == 0
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["vocab_size"] == 1000
    capsys.readouterr()
    assert main(["show", d]) == 0
    out = capsys.readouterr().out
    assert "Qwen2ForCausalLM" in out and "3 layers" in out
    with pytest.raises(SystemExit, match="unknown shape"):
        main(["random", d, "--shape", "nope"])
    with pytest.raises(SystemExit, match="not a token id"):
        main(["run", d, "hello"])
    with pytest.raises(SystemExit, match="temperature out of range"):
        main(["run", d, "1", "2", "--temp", "99"])
    assert main(["frobnicate"]) == 2
