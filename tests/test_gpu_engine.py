"""Generation through the Python entry point on the GPU: greedy tokens equal the plain
implementation's, through prompt portions, mixed steps and preemption; long decoding; seeded
sampling is repeatable and independent of the batch."""

from __future__ import annotations

import pytest
import torch

import plain_gpt
from harness import TOLERANCE, make_tensors, plain_logits, tiny_config, tokens_for

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, Request, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model

pytestmark = pytest.mark.gpu


def engine_for(which, dtype, sharp=True, seed=5, **kw):
    cfg = tiny_config(which)
    tensors = make_tensors(cfg, seed, dtype, sharp)
    loaded = load_model(config=cfg, tensors=tensors, dtype=dtype, device="cuda:0")
    return cfg, tensors, LLMEngine(loaded, EngineConfig(dtype=dtype, **kw))


def assert_greedy(cfg, tensors, prompt, generated, tol):
    """Every generated token is the plain argmax, or ties with it within the tolerance."""
    seq = prompt + generated
    want = plain_logits(cfg, tensors, seq[:-1])
    for i, token in enumerate(generated):
        row = want[len(prompt) - 1 + i]
        assert row.max() - row[token] <= 2 * tol, (i, token, int(row.argmax()))


@pytest.mark.parametrize("which", "AB")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(which, dtype):
    cfg, tensors, engine = engine_for(which, dtype, block_size=8, num_blocks=64, max_batch_size=3,
                                      max_num_batched_tokens=16, max_prefill_chunk=7)
    prompts = [tokens_for(cfg, n, 40 + i) for i, n in enumerate([5, 1, 23, 12, 2, 17])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 10 and out["finish_reason"] == "length"
        assert_greedy(cfg, tensors, prompt, out["token_ids"], TOLERANCE[dtype])
        if dtype == "float32":
            assert out["token_ids"] == plain_gpt.greedy_generate(
                prompt, tensors, cfg.n_layer, cfg.n_head, cfg.layer_norm_epsilon, 10)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_and_recompute_on_gpu(dtype):
    cfg, tensors, engine = engine_for("A", dtype, block_size=2, num_blocks=14, max_batch_size=3,
                                      max_num_batched_tokens=8)
    prompts = [tokens_for(cfg, n, 60 + i) for i, n in enumerate([6, 5, 7, 4])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=9, temperature=0.0))
    assert engine.scheduler.num_preemptions > 0
    for prompt, out in zip(prompts, outs):
        assert_greedy(cfg, tensors, prompt, out["token_ids"], TOLERANCE[dtype])
    assert engine.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_to_the_end_of_the_position_table(dtype):
    cfg, tensors, engine = engine_for("B", dtype, block_size=8, num_blocks=32, max_batch_size=2)
    prompt = tokens_for(cfg, 3, 9)
    n = cfg.n_positions - 3
    out = engine.generate([prompt], SamplingParams(max_tokens=n, temperature=0.0))[0]
    assert len(out["token_ids"]) == n
    assert_greedy(cfg, tensors, prompt, out["token_ids"], TOLERANCE[dtype])


def test_seeded_sampling_is_repeatable_and_independent_of_the_batch():
    cfg, tensors, engine = engine_for("B", "bfloat16", sharp=False, block_size=8, num_blocks=64,
                                      max_batch_size=4)
    prompt = tokens_for(cfg, 6, 3)
    params = SamplingParams(max_tokens=12, temperature=1.0, top_k=50, top_p=0.95, seed=77)
    alone = engine.generate([prompt], params)[0]["token_ids"]
    again = engine.generate([prompt], params)[0]["token_ids"]
    others = [tokens_for(cfg, 9, 4), tokens_for(cfg, 2, 5)]
    mixed = engine.generate([others[0], prompt, others[1]],
                            [SamplingParams(max_tokens=5, temperature=0.8, seed=1), params,
                             SamplingParams(max_tokens=20, temperature=0.0)])[1]["token_ids"]
    assert alone == again == mixed
    different = engine.generate([prompt], SamplingParams(max_tokens=12, temperature=1.0, seed=78))
    assert different[0]["token_ids"] != alone
    assert len(set(alone)) > 2                               # it does sample, not argmax


def test_vocab_limit_masks_padding_ids():
    cfg = tiny_config("A")
    tensors = make_tensors(cfg, 5, "float32")
    loaded = load_model(config=cfg, tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=32,
                                            max_batch_size=2), vocab_limit=10)
    outs = engine.generate([tokens_for(cfg, 5, 1)] * 2,
                           [SamplingParams(max_tokens=8, temperature=0.0),
                            SamplingParams(max_tokens=8, temperature=1.5, seed=3)])
    assert all(t < 10 for o in outs for t in o["token_ids"])
