"""The command line without a GPU: model folders from a configuration and a seed, model description."""
from __future__ import annotations

import json
import os
import subprocess
import sys

from helpers import ROOT, TINY_E


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "inferctl"), *args], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_random_then_models(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_E))
    out = _run("random", "--config", str(cfg), "--seed", "3", "--out", str(tmp_path / "m"), "--float32-vectors")
    assert out["architecture"] == "Qwen2ForCausalLM"
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    info = _run("models", "--model", str(tmp_path / "m"))
    assert info["config"]["hidden_size"] == 96 and info["tensors"] == 3 * 12 + 3
    assert [g["window"] for g in info["cache_groups"]] == [None, 40]


def test_random_then_models_of_the_second_architecture(tmp_path):
    """The same two commands for a Kunonex configuration: the folder it writes is read back by its own keys,
    and the description lists a latent stream per cache group and the state every run keeps."""
    from helpers import KX_A
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(KX_A))
    out = _run("random", "--config", str(cfg), "--seed", "4", "--out", str(tmp_path / "k"))
    assert out["architecture"] == "Kunonex"
    info = _run("models", "--model", str(tmp_path / "k"))
    assert info["architecture"] == "Kunonex" and info["config"]["width"] == 64 and info["config"]["loop"]["times"] == 2
    assert len(info["cache_groups"]) == 2
    from inferflux_b200.config import load_config
    assert load_config(str(tmp_path / "k")) == load_config(dict(KX_A))
