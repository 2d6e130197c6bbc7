"""The command line (no GPU: option parsing and the random-weights mode; generation needs a GPU)."""
import json
import os
import subprocess
import sys

import pytest

from tiny import ROOT, TINY_A

PKG = os.path.join(ROOT, "llm-inference-engine-v6_b200")


def run_cli(*args):
    env = dict(os.environ, PYTHONPATH=PKG)
    return subprocess.run([sys.executable, "-m", "llmengine", *args], capture_output=True, text=True, env=env, timeout=600)


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    r = run_cli("--random-weights", str(out), "--config", str(cfg), "--seed", "3", "--dtype", "bf16")
    assert r.returncode == 0, r.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert json.loads(r.stdout)["seed"] == 3
    assert run_cli("--random-weights", str(out)).returncode == 2
    assert run_cli().returncode == 2


@pytest.mark.gpu
def test_generation_from_the_command_line(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert run_cli("--random-weights", str(out), "--config", str(cfg), "--dtype", "fp32").returncode == 0
    r = run_cli("--model", str(out), "--prompt-ids", "5,17,3,200", "--max-new", "6", "--block-size", "4", "--num-blocks", "32")
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert lines[0]["token_ids"][:4] == [5, 17, 3, 200] and len(lines[0]["token_ids"]) == 10 and lines[0]["finish_reason"] == "length"
    r2 = run_cli("--model", str(out), "--prompt-len", "9", "--requests", "3", "--max-new", "4", "--budget", "5",
                 "--block-size", "4", "--num-blocks", "64", "--temperature", "0.8", "--seed", "2")
    assert r2.returncode == 0, r2.stderr
    lines = [json.loads(l) for l in r2.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 4 and lines[-1]["generated"] == 12 and [l["seq_id"] for l in lines[:3]] == [0, 1, 2]
    bad = run_cli("--model", str(out), "--prompt-ids", "5,999", "--max-new", "2")
    assert bad.returncode == 1 and "out of range" in bad.stderr
