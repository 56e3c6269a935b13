"""A configuration with the head size of the 50M model (64), small enough for the plain
implementation: the bfloat16 step then runs the tensor-core kernels that the tiny configurations
never reach (tcgen05 projections and prompt attention, the small-batch projection, the split
decode attention and the CUDA-graph replay), and every way of cutting must still agree with
the plain logits.  Sizes that are no power of two where the kernels allow it."""

from __future__ import annotations

import itertools

import pytest
import torch

from harness import TOLERANCE, assert_close, gpu_runner, make_tensors, plain_logits, tokens_for
from mini_gpt_inference_b200.config import GPTConfig
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

CONFIG = dict(vocab_size=1003, n_positions=700, n_layer=2, n_head=3, n_embd=192, n_inner=520,
              bias=True, layer_norm_epsilon=1e-5)


@pytest.fixture(scope="module")
def setup():
    cfg = GPTConfig.from_dict(CONFIG)
    out = {}
    for dtype in ("float32", "bfloat16"):
        tensors = make_tensors(cfg, 9, dtype, sharp=False)
        out[dtype] = (tensors, {})
    return cfg, out


def _want(cfg, cache, tensors, tokens):
    key = tuple(tokens)
    if key not in cache:
        cache[key] = plain_logits(cfg, tensors, tokens)
    return cache[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_tokens", [16, 64])
def test_cuttings_at_head_size_64(setup, dtype, page_tokens):
    cfg, per_dtype = setup
    tensors, cache = per_dtype[dtype]
    tol = TOLERANCE[dtype]
    runner = gpu_runner(cfg, tensors, dtype, page_tokens, num_pages=3 * (704 // page_tokens) + 4)
    tokens = tokens_for(cfg, 700, 5)
    want = _want(cfg, cache, tensors, tokens)

    # whole, alone: query tiles of 128, key chunks of 512, a ragged last tile
    got = runner.step([StepEntry("whole", tokens, list(range(700)))])
    assert_close(got, want, tol, "whole prompt of 700")
    runner.finish("whole")

    # most of it in one step, the last 32 tokens one by one (graph replay, split attention)
    outs = [runner.step([StepEntry("tail", tokens[:668], list(range(668)))])]
    for t in range(668, 700):
        outs.append(runner.step([StepEntry("tail", tokens[t: t + 1], [0])]))
    assert_close(torch.cat(outs), want, tol, "prefill then 32 single tokens")
    runner.finish("tail")
    if dtype == "bfloat16":
        assert runner.graph_replays >= 32

    # portions of changing size beside the decoding of two other requests
    other = {k: tokens_for(cfg, n, s) for k, n, s in (("o1", 300, 6), ("o2", 140, 7))}
    want_other = {k: _want(cfg, cache, tensors, v) for k, v in other.items()}
    pos = {"p": 0, "o1": 0, "o2": 0}
    seqs = {"p": tokens, **other}
    got = {k: [] for k in seqs}
    sizes = itertools.cycle([130, 2, 67, 1, 200, 129, 5])
    first = True
    while any(pos[k] < len(seqs[k]) for k in seqs):
        entries, order = [], []
        for k in seqs:
            if pos[k] >= len(seqs[k]):
                continue
            if k == "p":
                n = min(next(sizes), len(seqs[k]) - pos[k])
            else:
                n = min(97 if first else 1, len(seqs[k]) - pos[k])     # a prompt portion, then decoding
            entries.append(StepEntry(k, seqs[k][pos[k]: pos[k] + n], list(range(n))))
            order.append((k, n))
            pos[k] += n
        first = False
        logits = runner.step(entries)
        row = 0
        for k, n in order:
            got[k].append(logits[row: row + n])
            row += n
    assert_close(torch.cat(got["p"]), want, tol, "portions beside decoding")
    for k in other:
        assert_close(torch.cat(got[k]), want_other[k], tol, f"decoding request {k}")
    runner.ops.check_status()


def test_batched_decoding_at_every_graph_size(setup):
    """1 to 9 requests decoding together: the small-batch projection (up to 8 rows), the
    tensor-core projection with the batch on the narrow side (9 rows), padded graph rows."""
    cfg, per_dtype = setup
    tensors, cache = per_dtype["bfloat16"]
    runner = gpu_runner(cfg, tensors, "bfloat16", 16, num_pages=9 * 8 + 4, max_requests=16)
    prompts = {f"r{i}": tokens_for(cfg, 40 + 7 * i, 30 + i) for i in range(9)}
    want = {k: _want(cfg, cache, tensors, v) for k, v in prompts.items()}
    for k, v in prompts.items():
        runner.step([StepEntry(k, v[:-12], [])])
    for step in range(12):
        live = list(prompts)[: 9 - (step % 9) if step else 9]          # 9, 8, 7, ... rows
        logits = runner.step([StepEntry(k, [prompts[k][runner.length_of(k)]], [0]) for k in live])
        for i, k in enumerate(live):
            p = runner.length_of(k) - 1
            assert (logits[i].double().cpu() - want[k][p]).abs().max() <= TOLERANCE["bfloat16"], (step, k)
    runner.ops.check_status()
