"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits in files.
The same requests are replayed whole, with the last 32 tokens one by one, in portions, and
mixed with page reuse, in 32-bit and bfloat16, and compared with the plain implementation."""

from __future__ import annotations

import itertools
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from harness import TOLERANCE, make_model_dir, plain_logits, tokens_for

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def run_trace(model_dir, dtype, out_dir, max_tokens, steps, page_tokens=16):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), "--page-tokens", str(page_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return proc


def read_logits(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4").reshape(-1, vocab))


def collect(out_dir, steps, vocab):
    """Logits per request in position order, from the files of a trace."""
    got: dict[str, list] = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if not wanted:
            assert not (Path(out_dir) / f"{s['step']}.f32").exists()
            continue
        logits = read_logits(out_dir, s["step"], vocab)
        assert logits.shape[0] == wanted
        row = 0
        for e in s["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(logits[row: row + n])
            row += n
    return {k: torch.cat(v) for k, v in got.items()}


@pytest.mark.parametrize("which,dtype", list(itertools.product("AB", ["float32", "bfloat16"])))
def test_replay_four_ways(tmp_path, which, dtype):
    model_dir, cfg, tensors = make_model_dir(tmp_path, which, 21, dtype)
    tol = TOLERANCE[dtype]
    n = cfg.n_positions
    reqs = {f"r{i}": tokens_for(cfg, length, 70 + i)
            for i, length in enumerate([n, n - 7, 45, 2, n // 2, 33])}
    want = {k: plain_logits(cfg, tensors, v) for k, v in reqs.items()}

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(reqs.items())]
    run_trace(model_dir, dtype, tmp_path / "whole", 64 * ((n + 63) // 64), steps)
    whole = collect(tmp_path / "whole", steps, cfg.vocab_size)
    for k in reqs:
        assert (whole[k].double() - want[k]).abs().max() <= tol, f"whole {k}"

    # 2. most of it in one step, the last 32 tokens one by one
    k, v = "r0", reqs["r0"]
    steps = [{"step": 0, "entries": [{"id": k, "tokens": v[:-32], "want": list(range(len(v) - 32))}], "end": []}]
    for j in range(32):
        steps.append({"step": j + 1, "end": [k] if j == 31 else [],
                      "entries": [{"id": k, "tokens": [v[len(v) - 32 + j]], "want": [0]}]})
    run_trace(model_dir, dtype, tmp_path / "tail", 64 * ((n + 63) // 64), steps)
    assert (collect(tmp_path / "tail", steps, cfg.vocab_size)[k].double() - want[k]).abs().max() <= tol

    # 3. portions of changing size, down to two tokens; only some logits wanted
    sizes = itertools.cycle([11, 2, 5, 2, 17, 3, 2])
    steps, pos = [], 0
    while pos < len(v):
        m = min(next(sizes), len(v) - pos)
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": k, "tokens": v[pos: pos + m], "want": [0, m - 1] if m > 1 else [0]}]})
        pos += m
    run_trace(model_dir, dtype, tmp_path / "portions", 64 * ((n + 63) // 64), steps)
    got = collect(tmp_path / "portions", steps, cfg.vocab_size)[k]
    places, pos = [], 0
    for s in steps:
        m = len(s["entries"][0]["tokens"])
        places += [pos + w for w in s["entries"][0]["want"]]
        pos += m
    assert (got.double() - want[k][places]).abs().max() <= tol

    # 4. mixed: up to four live, some left out of a step, a pool that forces page reuse
    order = list(reqs)
    live, waiting, pos = [], list(order), dict.fromkeys(order, 0)
    sizes = itertools.cycle([7, 1, 2, 1, 13, 1, 3, 2])
    gen = torch.Generator().manual_seed(5)
    steps = []
    while live or waiting:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, end = [], []
        for rid in live:
            if len(live) > 1 and torch.rand((), generator=gen).item() < 0.2:
                continue
            m = min(next(sizes), len(reqs[rid]) - pos[rid])
            entries.append({"id": rid, "tokens": reqs[rid][pos[rid]: pos[rid] + m], "want": list(range(m))})
            pos[rid] += m
            if pos[rid] == len(reqs[rid]):
                end.append(rid)
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
        live = [r for r in live if r not in end]
    # the most that four live requests hold, each rounded up to 64
    most = sum(sorted(64 * ((len(t) + 63) // 64) for t in reqs.values())[-4:])
    assert most < sum(64 * ((len(t) + 63) // 64) for t in reqs.values())       # so pages are used again
    run_trace(model_dir, dtype, tmp_path / "mixed", most, steps)
    mixed = collect(tmp_path / "mixed", steps, cfg.vocab_size)
    for k in reqs:
        assert (mixed[k].double() - want[k]).abs().max() <= tol, f"mixed {k}"


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "float32"), ("C", "bfloat16")])
def test_replay_with_a_request_released_half_way_and_recomputed(tmp_path, which, dtype):
    """Preemption by recomputation inside a mixed replay: request v runs through half of its tokens
    beside two others, is ended (its pages go back and are taken by a newcomer), and comes again
    under the same id from its first token, in portions of 13 beside the others' single tokens.
    Logits at every position of both passes are compared (the reference's preemption test compares
    generated tokens, tests/test_paged.py:107-143)."""
    model_dir, cfg, tensors = make_model_dir(tmp_path, which, 23, dtype)
    tol = TOLERANCE[dtype]
    n = cfg.n_positions
    reqs = {"v": tokens_for(cfg, n - 3, 81), "o1": tokens_for(cfg, n // 2 + 5, 82), "o2": tokens_for(cfg, 37, 83),
            "late": tokens_for(cfg, n // 2, 84)}
    want = {k: plain_logits(cfg, tensors, t) for k, t in reqs.items()}
    pos = dict.fromkeys(reqs, 0)
    steps = []

    def step(parts, end=()):
        entries = []
        for rid, m in parts:
            m = min(m, len(reqs[rid]) - pos[rid])
            if m > 0:
                entries.append({"id": rid, "tokens": reqs[rid][pos[rid]: pos[rid] + m], "want": list(range(m))})
                pos[rid] += m
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})

    half = (n - 3) // 2
    step([("v", half - 4), ("o1", 9), ("o2", 2)])
    for _ in range(4):
        step([("v", 1), ("o1", 1), ("o2", 3)])
    first_pass = len(steps)
    step([("o1", 1), ("o2", 1)], end=["v"])                    # v gives everything back
    pos["v"] = 0
    step([("late", n // 2), ("o1", 1)])                        # a newcomer takes the freed pages
    step([("o2", 50)], end=["late", "o2"])
    while pos["v"] < len(reqs["v"]) or pos["o1"] < len(reqs["o1"]):
        step([("v", 13), ("o1", 1)])
    steps[-1]["end"] = ["v", "o1"]
    live_most = sum(64 * ((len(reqs[k]) + 63) // 64) for k in ("v", "o1", "o2"))
    run_trace(model_dir, dtype, tmp_path / "preempt", live_most, steps, page_tokens=8)
    first = collect(tmp_path / "preempt", steps[:first_pass], cfg.vocab_size)
    rest = collect(tmp_path / "preempt", steps[first_pass:], cfg.vocab_size)
    assert (first["v"].double() - want["v"][:half]).abs().max() <= tol, "first pass of v"
    assert (rest["v"].double() - want["v"]).abs().max() <= tol, "v recomputed"
    if dtype == "float32":
        assert torch.equal(rest["v"][:half], first["v"]), "recomputation differs from the first pass"
    for k in ("o1", "o2"):
        both = torch.cat([first[k], rest[k]])
        assert (both.double() - want[k]).abs().max() <= tol, k
    assert (rest["late"].double() - want["late"]).abs().max() <= tol, "late"


def test_trace_run_reports_bad_input(tmp_path):
    model_dir, cfg, _ = make_model_dir(tmp_path, "A", 3, "float32")
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", "float32",
           "--out", str(tmp_path / "o"), "--max-tokens", "64"]
    step = {"step": 0, "entries": [{"id": "a", "tokens": [cfg.vocab_size + 5], "want": [0]}], "end": []}
    proc = subprocess.run(cmd, input=json.dumps(step) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "vocabulary" in proc.stderr
