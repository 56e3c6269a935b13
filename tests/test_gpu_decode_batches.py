"""Decoding many requests together: more than 64 rows take the token-major tensor-core projection
with padding rows up to the graph sizes 128 and 256 (position -1, cache slot -1), and more than
256 rows leave the replayed graphs altogether.  Every row is compared with the plain logits of
its own sequence.

Every request is a prefix of one of eight base sequences (lengths differ from row to row), so a
handful of plain passes give the wanted logits of hundreds of requests.
"""

from __future__ import annotations

import pytest
import torch

from harness import TOLERANCE, assert_close, gpu_runner, make_tensors, plain_logits, tokens_for
from mini_gpt_inference_b200.config import GPTConfig
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

HEAD64 = dict(vocab_size=1003, n_positions=96, n_layer=2, n_head=3, n_embd=192, n_inner=520,
              bias=True, layer_norm_epsilon=1e-5)
# 32 heads of 16: a decode batch of 200 needs 6,400 "last block" counters of the split attention;
# contexts beyond 256 positions have two key blocks at this head size, so the counters are used
MANY_HEADS = dict(vocab_size=331, n_positions=300, n_layer=2, n_head=32, n_embd=512, n_inner=136,
                  bias=False, layer_norm_epsilon=2e-5)
BASES = 8
STEPS = 3


def _setup(config, dtype, pages, max_requests, page_tokens=16, ops=None):
    cfg = GPTConfig.from_dict(config)
    tensors = make_tensors(cfg, 13, dtype, sharp=False)
    bases = [tokens_for(cfg, cfg.n_positions, 200 + b) for b in range(BASES)]
    want = [plain_logits(cfg, tensors, b) for b in bases]
    runner = gpu_runner(cfg, tensors, dtype, page_tokens, pages, max_requests, ops=ops)
    for p in runner.storage.k + runner.storage.v:
        p.fill_(float("nan"))
    return cfg, bases, want, runner


def _decode_together(runner, bases, want, rows, tol, tag, steps=STEPS, shortest=20):
    lengths = [shortest + (7 * i) % 45 + (i % 3) for i in range(rows)]
    assert max(lengths) + steps <= len(bases[0])
    ids = [f"{tag}{i}" for i in range(rows)]
    for i, rid in enumerate(ids):
        runner.step([StepEntry(rid, bases[i % BASES][: lengths[i]], [])])
    for s in range(steps):
        got = runner.step([StepEntry(rid, [bases[i % BASES][lengths[i] + s]], [0])
                           for i, rid in enumerate(ids)])
        assert got.shape[0] == rows and not torch.isnan(got).any()
        expected = torch.stack([want[i % BASES][lengths[i] + s] for i in range(rows)])
        assert_close(got, expected, tol, f"{rows} rows, decode step {s}",
                     places=[(rid, lengths[i] + s) for i, rid in enumerate(ids)])
    for rid in ids:
        runner.finish(rid)
    runner.ops.check_status()
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def head64(request):
    dtype = request.param
    cfg, bases, want, runner = _setup(HEAD64, dtype, pages=300 * 5 + 8, max_requests=300)
    return bases, want, runner, dtype, TOLERANCE[dtype]


@pytest.mark.parametrize("rows", [65, 100, 128, 200, 256, 300])
def test_decode_batches_above_64_rows(head64, rows):
    bases, want, runner, dtype, tol = head64
    replays = runner.graph_replays
    _decode_together(runner, bases, want, rows, tol, f"n{rows}_")
    if dtype == "bfloat16":
        # up to 256 rows a decode step is a replayed graph; beyond, it is launched kernel by kernel
        assert runner.graph_replays - replays == (STEPS if rows <= 256 else 0)


def test_graphs_of_small_batches_survive_a_large_batch():
    """A graph captured for 4 rows keeps the addresses of its attention's counters.  A batch of 200
    rows of 32 heads then needs more counters than were there; the small graph, replayed
    afterwards, must still find its own (zeroed) ones."""
    from mini_gpt_inference_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda:0")                 # a kernel set of its own: its counters start small
    cfg, bases, want, runner = _setup(MANY_HEADS, "bfloat16", pages=200 * 19 + 8, max_requests=200, ops=ops)
    tol = TOLERANCE["bfloat16"]
    _decode_together(runner, bases, want, 4, tol, "a", shortest=247)
    _decode_together(runner, bases, want, 200, tol, "b", shortest=247)
    _decode_together(runner, bases, want, 4, tol, "c", steps=6, shortest=247)
    _decode_together(runner, bases, want, 3, tol, "d", shortest=247)
    assert runner.graph_replays == 3 + 3 + 6 + 3
    assert ops._retired_counters, "the large batch was expected to outgrow the first counters"
