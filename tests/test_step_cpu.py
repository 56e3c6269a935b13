"""The step function, the parts and the cache manager together, run on the CPU with a torch
test double in place of the CUDA kernel set: checks the batch description, the page tables
and the cutting logic without a GPU.  (The product has no CPU path; see tests/torch_ops.py.)"""

from __future__ import annotations

import itertools

import pytest
import torch

from harness import PAGE_TOKENS, assert_close, make_tensors, plain_logits, tiny_config, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200.cache import CacheFullError
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry, StepError


def cpu_runner(cfg, tensors, page_tokens, num_pages, max_requests=8):
    loaded = load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")
    return make_runner(loaded, TorchOps(), page_tokens, num_pages, max_requests)


@pytest.mark.parametrize("which", "AB")
def test_cuttings_agree_with_plain(which):
    cfg = tiny_config(which)
    tensors = make_tensors(cfg, 3, "float32", sharp=True)
    pt = PAGE_TOKENS[which]
    runner = cpu_runner(cfg, tensors, pt, 3 * (cfg.n_positions // pt))
    n = cfg.n_positions
    reqs = {"a": tokens_for(cfg, n, 1), "b": tokens_for(cfg, n - 5, 2), "c": tokens_for(cfg, 9, 3)}
    want = {k: plain_logits(cfg, tensors, v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}
    pos = dict.fromkeys(reqs, 0)
    sizes = itertools.cycle([13, 1, 2, 7, 1, 1, 5, 2])
    while any(pos[k] < len(reqs[k]) for k in reqs):
        entries, order = [], []
        for k in reqs:
            if pos[k] == len(reqs[k]):
                continue
            m = min(next(sizes), len(reqs[k]) - pos[k])
            entries.append(StepEntry(k, reqs[k][pos[k]: pos[k] + m], list(range(m))))
            order.append((k, m))
            pos[k] += m
        out = runner.step(entries)
        row = 0
        for k, m in order:
            got[k].append(out[row: row + m])
            row += m
        runner.manager.check()
    for k in reqs:
        assert_close(torch.cat(got[k]), want[k], 5e-6, f"request {k}")
        runner.finish(k)
    assert runner.manager.stats()["allocated_blocks"] == 0


def test_batch_description():
    cfg = tiny_config("A")
    runner = cpu_runner(cfg, make_tensors(cfg, 1, "float32"), 16, 8)
    runner.step([StepEntry("a", list(range(20)), [])])
    ctx_entries = [StepEntry("a", [7], [0]), StepEntry("b", [1, 2, 3], [0, 2])]
    runner._validate(ctx_entries)
    runner._reserve(ctx_entries)
    ctx = runner.build_context(ctx_entries)
    assert ctx.num_tokens == 4 and ctx.num_requests == 2 and not ctx.decode_only
    assert ctx.token_ids.tolist() == [7, 1, 2, 3]
    assert ctx.positions.tolist() == [20, 0, 1, 2]
    assert ctx.token_request.tolist() == [0, 1, 1, 1]
    assert ctx.req_q_start.tolist() == [0, 1] and ctx.req_q_len.tolist() == [1, 3]
    assert ctx.req_ctx_before.tolist() == [20, 0]
    assert ctx.logit_rows.tolist() == [0, 1, 3]
    table_a = runner.manager.block_table("a", 0)
    assert ctx.block_tables[0][0, :2].tolist() == table_a and ctx.block_tables[0][0, 2] == -1
    assert ctx.slot_mapping[0][0] == table_a[1] * 16 + 4
    assert ctx.max_q_len == 3 and ctx.max_ctx_after == 21
    assert len(set(ctx.req_state_slot.tolist())) == 2


def test_wanting_nothing_returns_none_and_still_fills_the_cache():
    cfg = tiny_config("A")
    tensors = make_tensors(cfg, 2, "float32")
    runner = cpu_runner(cfg, tensors, 16, 8)
    tokens = tokens_for(cfg, 30, 4)
    assert runner.step([StepEntry("a", tokens[:29], [])]) is None
    out = runner.step([StepEntry("a", tokens[29:], [0])])
    assert_close(out, plain_logits(cfg, tensors, tokens)[-1:], 5e-6, "after a silent prefill")


def test_errors():
    cfg = tiny_config("A")
    runner = cpu_runner(cfg, make_tensors(cfg, 1, "float32"), 16, 2)
    with pytest.raises(StepError, match="twice"):
        runner.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(StepError, match="no tokens"):
        runner.step([StepEntry("a", [], [])])
    with pytest.raises(StepError, match="vocabulary"):
        runner.step([StepEntry("a", [-1], [])])
    with pytest.raises(CacheFullError):
        runner.step([StepEntry("a", [1] * 33, [])])
    assert not runner.manager.has("a")                       # a refused step leaves no trace
    runner.manager.check()
