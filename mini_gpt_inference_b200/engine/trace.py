"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``ModelRunner.step``, the step function that generation uses, with the same cache
manager and kernels.  The reference has nothing like it; the closest are its test
helper that steps an engine to completion (tests/test_paged.py:32-42) and its
decode-only timing loop (bench/bench_hardware.py:79-92).

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants logits, ``<out>/<step>.f32`` receives them as little-endian float32
``[wanted, vocab]`` in the order of the entries and of ``want``.  After every step a line
``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_ROUND = 64      # default of --page-round
LIVE_REQUESTS = 8    # default of --live-requests


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each request's count rounded "
                         "up to a multiple of --page-round")
    ap.add_argument("--page-tokens", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--page-round", type=int, default=PAGE_ROUND,
                    help="the multiple to which --max-tokens counts each request rounded up "
                         "(a multiple of --page-tokens; default 64)")
    ap.add_argument("--live-requests", type=int, default=LIVE_REQUESTS,
                    help="most requests that are live at a time (state slots; default 8)")
    ap.add_argument("--device", default="cuda:0")
    return ap.parse_args(argv)


def main(argv=None, stdin=None, stdout=None) -> int:
    args = parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    import numpy as np
    import torch

    from ..kernels.ops import default_ops
    from .build import load_model, make_runner
    from .runner import StepEntry

    if (args.max_tokens <= 0 or args.page_tokens <= 0 or args.page_round <= 0 or args.live_requests <= 0
            or args.page_round % args.page_tokens != 0):
        print("trace_run: --max-tokens, --page-tokens, --page-round and --live-requests must be "
              "positive, and --page-tokens must divide --page-round", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    ops = default_ops(args.device)
    loaded = load_model(args.model, dtype=args.dtype, device=args.device)
    pool_tokens = (args.max_tokens + args.page_round - 1) // args.page_round * args.page_round
    runner = make_runner(loaded, ops, page_tokens=args.page_tokens,
                         num_pages=pool_tokens // args.page_tokens, max_requests=args.live_requests)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(str(e["id"]), e["tokens"], e.get("want", []))
                   for e in record.get("entries", [])]
        logits = runner.step(entries) if entries else None
        if logits is not None and logits.shape[0] > 0:
            host = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            np.ascontiguousarray(host).tofile(out_dir / f"{step}.f32")
        elif entries:
            torch.cuda.synchronize()
        if entries:
            ops.check_status()                 # a kernel that gave up waiting ends the replay
        for rid in record.get("end", []):
            runner.finish(str(rid))
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0
