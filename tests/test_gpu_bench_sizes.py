"""The layer sizes and the context that the benchmark times (width 512, 8 heads of 64, MLP 2048,
vocabulary 50304, 2048 positions, pages of 64), with two layers so that the plain implementation
stays quick: a prompt of two thousand tokens (key chunks merged four ways), then single tokens up
to the end of the position table, alone and in batches of 8 and 64 whose contexts are all beyond
1,500 tokens, so that every key block of the split decode attention holds keys and its merge
(in the same kernel for small grids, in a second kernel for large ones) has something to merge.

Every request is a prefix of one of eight base sequences, so one plain pass per base gives the
wanted logits of all of them; only the wanted rows meet the 50304-wide head.  The cache starts as
NaN: a query that reads a row its own request did not write turns its logits into NaN.
"""

from __future__ import annotations

import pytest
import torch

from harness import TOLERANCE, assert_close, gpu_runner, make_tensors, plain_logits, tokens_for
from mini_gpt_inference_b200.config import GPTConfig
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

CONFIG = dict(vocab_size=50304, n_positions=2048, n_layer=2, n_head=8, n_embd=512, n_inner=2048,
              bias=True, layer_norm_epsilon=1e-5)
PAGE = 64
BASES = 8
DECODE_STEPS = {1: 32, 8: 32, 64: 6}


class Oracle:
    """Plain logits of prefixes of the base sequences, computed one base at a time, on demand."""

    def __init__(self, cfg, tensors):
        self.cfg, self.tensors = cfg, tensors
        self.bases = [tokens_for(cfg, cfg.n_positions, 100 + b) for b in range(BASES)]
        self._rows: dict[tuple[int, int], torch.Tensor] = {}

    def need(self, base: int, positions) -> None:
        missing = sorted({p for p in positions if (base, p) not in self._rows})
        if missing:
            upto = missing[-1] + 1
            logits = plain_logits(self.cfg, self.tensors, self.bases[base][:upto], rows=missing)
            for p, row in zip(missing, logits):
                self._rows[(base, p)] = row

    def rows(self, base: int, positions) -> torch.Tensor:
        self.need(base, positions)
        return torch.stack([self._rows[(base, p)] for p in positions])


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request):
    dtype = request.param
    cfg = GPTConfig.from_dict(CONFIG)
    tensors = make_tensors(cfg, 9, dtype, sharp=False)
    oracle = Oracle(cfg, tensors)
    probe = oracle.rows(0, [5, 900, 2047])
    # 32-bit: the absolute bound of the other tests.  bfloat16: 3% of the logits' spread, as at the
    # other large widths (activations are rounded to 8 bits between kernels; a lost key block or a
    # block merged twice moves logits by tens of percent).
    tol = TOLERANCE[dtype] if dtype == "float32" else 0.03 * float(probe.std())
    runner = gpu_runner(cfg, tensors, dtype, PAGE, num_pages=64 * (2048 // PAGE) + 8, max_requests=64)
    for pages in runner.storage.k + runner.storage.v:
        pages.fill_(float("nan"))
    return cfg, oracle, runner, dtype, tol


def test_long_prompt_then_single_tokens(setup):
    cfg, oracle, runner, dtype, tol = setup
    tokens = oracle.bases[0]
    head = 2048 - 32
    wanted = sorted(set(range(0, head, 97)) | set(range(head - 40, head)) | {127, 128, 511, 512, 513, 1024})
    got = runner.step([StepEntry("long", tokens[:head], wanted)])
    assert not torch.isnan(got).any()
    assert_close(got, oracle.rows(0, wanted), tol, "prompt of 2016 tokens", places=wanted)
    outs = []
    for t in range(head, 2048):
        outs.append(runner.step([StepEntry("long", tokens[t: t + 1], [0])]))
    assert_close(torch.cat(outs), oracle.rows(0, list(range(head, 2048))), tol,
                 "32 single tokens after 2016", places=list(range(head, 2048)))
    runner.finish("long")
    runner.ops.check_status()
    assert runner.manager.stats()["allocated_blocks"] == 0


def test_prompt_in_portions_across_key_chunks(setup):
    """The same long prompt in portions whose edges fall beside the edges of pages (64), query
    tiles (128) and key chunks (512): logits of each portion's first and last token."""
    cfg, oracle, runner, dtype, tol = setup
    tokens = oracle.bases[1]
    sizes = [511, 2, 127, 129, 255, 64, 448, 3, 380, 129]
    assert sum(sizes) <= 2048
    pos, places, outs = 0, [], []
    for n in sizes:
        outs.append(runner.step([StepEntry("cut", tokens[pos: pos + n], [0, n - 1])]))
        places += [pos, pos + n - 1]
        pos += n
    assert_close(torch.cat(outs), oracle.rows(1, places), tol, "portions of a long prompt", places=places)
    runner.finish("cut")
    runner.ops.check_status()


@pytest.mark.parametrize("batch", [8, 64])
def test_batched_decoding_at_long_contexts(setup, batch):
    cfg, oracle, runner, dtype, tol = setup
    steps = DECODE_STEPS[batch]
    # request i: a prefix of base i % 8 whose length differs from every other's
    lengths = [1500 + 8 * i + (i % 5) for i in range(batch)]
    assert max(lengths) + steps <= 2048 and min(lengths) >= 1500
    ids = [f"b{batch}_{i}" for i in range(batch)]
    for b in range(min(BASES, batch)):                      # one plain pass per base sequence
        oracle.need(b, [lengths[i] + s for i in range(b, batch, BASES) for s in range(steps)])
    for i, rid in enumerate(ids):
        runner.step([StepEntry(rid, oracle.bases[i % BASES][: lengths[i]], [])])
    for s in range(steps):
        entries = [StepEntry(rid, [oracle.bases[i % BASES][lengths[i] + s]], [0])
                   for i, rid in enumerate(ids)]
        got = runner.step(entries)
        assert not torch.isnan(got).any(), f"step {s}: a cache row that is not the request's own was read"
        want = torch.cat([oracle.rows(i % BASES, [lengths[i] + s]) for i in range(batch)])
        assert_close(got, want, tol, f"batch of {batch}, decode step {s}",
                     places=[(rid, lengths[i] + s) for i, rid in enumerate(ids)])
    if dtype == "bfloat16":
        assert runner.graph_replays >= steps
    for rid in ids:
        runner.finish(rid)
    runner.ops.check_status()
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0
