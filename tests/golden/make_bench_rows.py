"""Plain-implementation logits for the step that bench.py times, stored so that the benchmark can
check (outside its timed region) that the decode step it measures computes the right thing.

Run on the CPU from the repository root (about a minute):

    python tests/golden/make_bench_rows.py

The model is the benchmark's default: the 50M layer sizes (8 layers, width 512, 8 heads, MLP 2048,
vocabulary 50304, 2048 positions, biases on) with ``random_tensors(model, 0, bfloat16)``.  Eight
requests of 2,048 seeded random tokens each go through ``tests/plain_gpt.py`` whole, in 64-bit;
the logits of each request's last position (what a decode step at context 2,048 returns) are
stored at 256 evenly spaced vocabulary ids, with the id of the largest logit, in
``tests/golden/bench_decode_rows.json``.  bench.py prefills the first 2,047 tokens of the same
requests, decodes token 2,048 as a batch of eight, and compares.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import plain_gpt  # noqa: E402
from mini_gpt_inference_b200.config import GPTConfig, lookup  # noqa: E402
from mini_gpt_inference_b200.parts import DecoderModel  # noqa: E402
from mini_gpt_inference_b200.weights import random_tensors  # noqa: E402

CONFIG = dict(vocab_size=50304, n_positions=2048, n_layer=8, n_head=8, n_embd=512, n_inner=2048,
              bias=True, layer_norm_epsilon=1e-5)
BATCH, LENGTH, TOKEN_SEED, WEIGHT_SEED, COLUMNS = 8, 2048, 4242, 0, 256


def main() -> None:
    cfg = GPTConfig.from_dict(CONFIG)
    model = DecoderModel(lookup(cfg.architecture).describe(cfg))
    tensors = random_tensors(model, WEIGHT_SEED, torch.bfloat16)
    gen = torch.Generator().manual_seed(TOKEN_SEED)
    columns = torch.linspace(0, cfg.vocab_size - 1, COLUMNS).long()
    rows, argmax, spread = [], [], []
    for r in range(BATCH):
        tokens = torch.randint(0, cfg.vocab_size, (LENGTH,), generator=gen).tolist()
        logits = plain_gpt.forward_logits(tokens, tensors, cfg.n_layer, cfg.n_head,
                                          cfg.layer_norm_epsilon, rows=[LENGTH - 1])[0]
        rows.append([round(float(v), 6) for v in logits[columns]])
        argmax.append(int(logits.argmax()))
        spread.append(float(logits.std()))
        print(f"request {r}: argmax {argmax[-1]}, std {spread[-1]:.4f}", flush=True)
    out = {"config": CONFIG, "weights": {"seed": WEIGHT_SEED, "dtype": "bfloat16"},
           "tokens": {"seed": TOKEN_SEED, "batch": BATCH, "length": LENGTH,
                      "how": "torch.Generator().manual_seed(seed); torch.randint(0, vocab, (length,)) per request, in order"},
           "columns": columns.tolist(), "logits": rows, "argmax": argmax,
           "logits_std": round(sum(spread) / len(spread), 6)}
    path = Path(__file__).with_name("bench_decode_rows.json")
    path.write_text(json.dumps(out, separators=(",", ":")) + "\n")
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
