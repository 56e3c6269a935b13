"""bin/generate as a user runs it: a model folder on disk, token ids on the command line, one JSON
line with the generated ids on standard output (the reference's scripts load a checkpoint and
print a sample the same way, scripts/download_checkpoint.py:20-41)."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

import plain_gpt
from harness import TOLERANCE, make_model_dir, plain_logits, tokens_for

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def generate(model_dir, prompt, *options):
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model", str(model_dir),
           "--prompt-ids", ",".join(map(str, prompt)), *map(str, options)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [line for line in proc.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, proc.stdout
    out = json.loads(lines[0])
    assert out["prompt_ids"] == list(prompt)
    return out, proc


@pytest.mark.parametrize("which", "AB")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_by_the_command_line(tmp_path, which, dtype):
    model_dir, cfg, tensors = make_model_dir(tmp_path, which, 31, dtype)
    prompt = tokens_for(cfg, 9, 4)
    out, proc = generate(model_dir, prompt, "--temperature", 0, "--max-new-tokens", 12, "--dtype", dtype,
                         "--kv-block-size", 8, "--num-kv-blocks", 32)
    ids = out["token_ids"]
    assert len(ids) == 12 and out["finish_reason"] == "length"
    assert "params:" in proc.stderr
    if dtype == "float32":
        assert ids == plain_gpt.greedy_generate(prompt, tensors, cfg.n_layer, cfg.n_head,
                                                cfg.layer_norm_epsilon, 12)
    else:
        # every token is the plain argmax of its own prefix, or ties with it within rounding
        want = plain_logits(cfg, tensors, (prompt + ids)[:-1])
        for i, token in enumerate(ids):
            row = want[len(prompt) - 1 + i]
            assert row.max() - row[token] <= 2 * TOLERANCE[dtype], (i, token, int(row.argmax()))


def test_seeded_sampling_and_vocabulary_limit_by_the_command_line(tmp_path):
    model_dir, cfg, _ = make_model_dir(tmp_path, "B", 32, "bfloat16")
    prompt = tokens_for(cfg, 6, 5)
    options = ["--temperature", 0.8, "--top-k", 50, "--seed", 1, "--max-new-tokens", 16]
    first, _ = generate(model_dir, prompt, *options)
    second, _ = generate(model_dir, prompt, *options)
    assert first["token_ids"] == second["token_ids"] and len(first["token_ids"]) == 16
    other, _ = generate(model_dir, prompt, "--temperature", 0.8, "--top-k", 50, "--seed", 2,
                        "--max-new-tokens", 16)
    assert other["token_ids"] != first["token_ids"]
    limited, _ = generate(model_dir, prompt, "--temperature", 1.5, "--seed", 3, "--max-new-tokens", 24,
                          "--vocab-limit", 11)
    assert all(t < 11 for t in limited["token_ids"])
