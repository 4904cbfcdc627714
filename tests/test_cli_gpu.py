"""The command line: ``mrun random`` writes a folder, ``mrun run`` generates from token ids with the
reference's option names, prints the ids, and refuses bad flags before loading anything."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

import plain_qwen3 as plain
from tiny_models import TINY, random_tokens

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
MRUN = os.path.join(ROOT, "bin", "mrun")


def run(*args):
    return subprocess.run([sys.executable, MRUN, *args], capture_output=True, text=True, timeout=600)


def test_usage_errors_need_no_model():
    for flags, text in ((["--max-tokens", "0"], "--max-tokens must be at least 1"),
                        (["--temperature", "-1"], "temperature must be 0 or more"),
                        (["--top-p", "0"], "top_p must be in (0, 1]"),
                        (["--budget-gib", "8", "--context", "4K"], "--context cannot be used with --budget-gib"),
                        (["--budget-gib", "0"], "at least 1 GiB")):
        result = run("run", "/nonexistent", "--prompt", "1,2", *flags)
        assert result.returncode == 2 and text in result.stderr
    assert run("run", "/nonexistent", "--prompt", "").returncode == 2


@pytest.mark.gpu
def test_random_then_run(tmp_path):
    config = dict(TINY["A"]["config"], model_type="qwen3", architectures=["Qwen3ForCausalLM"])
    (tmp_path / "cfg.json").write_text(json.dumps(config))
    folder = str(tmp_path / "model")
    made = run("random", folder, "--config", str(tmp_path / "cfg.json"), "--seed", "11", "--std", "0.08")
    assert made.returncode == 0, made.stderr
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    cfg, weights = plain.load_folder(folder)
    prompt = random_tokens(cfg["vocab_size"], 17, seed=1)
    ids = tmp_path / "prompt.txt"
    ids.write_text(" ".join(map(str, prompt)))

    result = run("run", folder, "--prompt", str(ids), "--max-tokens", "8", "--dtype", "float32", "--ignore-eos")
    assert result.returncode == 0, result.stderr
    tokens = [int(t) for t in result.stdout.strip().split(",")]
    assert tokens == plain.generate(cfg, weights, prompt, 8)
    assert "prompt: 17 tokens" in result.stderr and "generation: 8 tokens" in result.stderr

    # --stop: the output ends before the first stop sequence (of token ids) that appears
    stopped = run("run", folder, "--prompt", str(ids), "--max-tokens", "8", "--dtype", "float32", "--ignore-eos",
                  "--stop", f"{tokens[4]},{tokens[5]}", "--stop", "100000")
    assert stopped.returncode == 0, stopped.stderr
    first = next(i for i in range(7) if tokens[i:i + 2] == tokens[4:6])
    assert [int(t) for t in stopped.stdout.strip().split(",")] == tokens[:first]
    assert f"(stop [{tokens[4]}, {tokens[5]}])" in stopped.stderr
    many = run("run", folder, "--prompt", str(ids), "--stop", "1", "--stop", "2", "--stop", "3", "--stop", "4", "--stop", "5")
    assert many.returncode != 0 and "at most 4 stop sequences" in many.stderr

    inline = run("run", folder, "--prompt", ",".join(map(str, prompt)), "--max-tokens", "8", "--dtype", "float32",
                 "--temperature", "0.8", "--seed", "5", "--ignore-eos")
    again = run("run", folder, "--prompt", ",".join(map(str, prompt)), "--max-tokens", "8", "--dtype", "float32",
                "--temperature", "0.8", "--seed", "5", "--ignore-eos")
    assert inline.returncode == 0 and inline.stdout == again.stdout
    assert [int(t) for t in inline.stdout.strip().split(",")] == plain.generate(cfg, weights, prompt, 8, temperature=0.8, seed=5)

    info = run("run", folder, "--info", "--context", "1K")
    assert info.returncode == 0 and json.loads(info.stdout)["capacity_tokens"] == 1024
    memory = json.loads(info.stdout)["memory"]
    assert memory["binding"] == "context"
    assert memory["budget_bytes"] == memory["weights_bytes"] + memory["scratch_bytes"] + memory["cache_bytes"]

    # without --context: the most that fits, at most the model's longest sequence
    most = json.loads(run("run", folder, "--info", "--budget-gib", "1").stdout)
    assert most["capacity_tokens"] == cfg["max_position_embeddings"] and most["memory"]["binding"] == "budget-gib"
    # a budget above the automatic one and a context beyond the model are refused with the figures
    above = run("run", folder, "--info", "--budget-gib", "100000")
    assert above.returncode == 4 and "above the automatic budget" in above.stderr
    beyond = run("run", folder, "--info", "--context", "1M")
    assert beyond.returncode == 4 and "beyond the 1024 tokens" in beyond.stderr

    bad = run("run", str(tmp_path), "--prompt", "1")
    assert bad.returncode == 1 and "config.json" in bad.stderr
