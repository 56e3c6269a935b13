"""The Python entry point end to end on the CPU test double: scheduler, step function and
cache together produce the plain implementation's greedy tokens, also when prompts are cut
into portions and requests are preempted and recomputed (mirrors the reference's
tests/test_paged.py:45-143, which compares with its static-cache generation)."""

from __future__ import annotations

import pytest

import plain_gpt
from harness import make_tensors, tiny_config, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, Request, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model


def engine_for(which, engine_cfg, seed=5):
    cfg = tiny_config(which)
    tensors = make_tensors(cfg, seed, "float32", sharp=True)
    loaded = load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")
    return cfg, tensors, LLMEngine(loaded, engine_cfg, ops=TorchOps())


def plain_greedy(cfg, tensors, prompt, n):
    return plain_gpt.greedy_generate(prompt, tensors, cfg.n_layer, cfg.n_head,
                                     cfg.layer_norm_epsilon, n)


@pytest.mark.parametrize("which", "AB")
def test_generate_matches_plain_greedy(which):
    ecfg = EngineConfig(block_size=8, num_blocks=64, max_batch_size=3, max_num_batched_tokens=16,
                        max_prefill_chunk=7, dtype="float32", device="cpu")
    cfg, tensors, engine = engine_for(which, ecfg)
    assert engine.warm_up() == {"decode_graphs_captured": 0}      # nothing to capture where steps are not replayed
    prompts = [tokens_for(cfg, n, 40 + i) for i, n in enumerate([5, 1, 23, 12, 2, 17])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(cfg, tensors, prompt, 6)
        assert out["finish_reason"] == "length"
    stats = engine.stats()
    assert stats["allocated_blocks"] == 0 and stats["free_state_slots"] == 3
    engine.runner.manager.check()


def test_forced_preemption_recomputes_and_still_matches():
    # as tests/test_paged.py:107-143: a pool so small that running requests must give way
    ecfg = EngineConfig(block_size=2, num_blocks=14, max_batch_size=3, max_num_batched_tokens=8,
                        dtype="float32", device="cpu")
    cfg, tensors, engine = engine_for("A", ecfg)
    prompts = [tokens_for(cfg, n, 60 + i) for i, n in enumerate([6, 5, 7, 4])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=9, temperature=0.0))
    assert engine.scheduler.num_preemptions > 0
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(cfg, tensors, prompt, 9)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_finish_reasons_and_admission_checks():
    ecfg = EngineConfig(block_size=8, num_blocks=16, max_batch_size=2, dtype="float32", device="cpu")
    cfg, tensors, engine = engine_for("A", ecfg)
    prompt = tokens_for(cfg, 4, 1)
    first = plain_greedy(cfg, tensors, prompt, 3)
    # end-of-text beats length (src/minigpt_infer/engine/engine.py:186-194)
    engine.add_request(Request("eot", prompt, SamplingParams(max_tokens=1, temperature=0.0),
                               eot_token_id=first[0]))
    engine.add_request(Request("stop", prompt, SamplingParams(max_tokens=5, temperature=0.0,
                                                              stop_token_ids=[first[1]])))
    reasons = {}
    while engine.has_unfinished_requests():
        for out in engine.step():
            if out.finished:
                reasons[out.request_id] = out.finish_reason
    assert reasons == {"eot": "eot", "stop": "stop"}
    with pytest.raises(ValueError, match="position table"):
        engine.add_request(Request("long", prompt, SamplingParams(max_tokens=cfg.n_positions)))
    with pytest.raises(ValueError, match="vocabulary"):
        engine.add_request(Request("bad", [cfg.vocab_size], SamplingParams(max_tokens=1)))
    with pytest.raises(ValueError, match="empty"):
        engine.add_request(Request("none", [], SamplingParams(max_tokens=1)))


def test_cancel_frees_pages():
    ecfg = EngineConfig(block_size=4, num_blocks=16, max_batch_size=2, dtype="float32", device="cpu")
    cfg, tensors, engine = engine_for("A", ecfg)
    engine.add_request(Request("a", tokens_for(cfg, 9, 2), SamplingParams(max_tokens=20, temperature=0.0)))
    engine.step()
    assert engine.stats()["allocated_blocks"] == 3
    assert engine.cancel_request("a") and not engine.cancel_request("a")
    assert engine.stats()["allocated_blocks"] == 0 and not engine.has_unfinished_requests()


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_random_arrivals_small_pools_and_cancellations(seed):
    """Requests arrive while others run, in pools and budgets drawn at random (small enough to
    force portions, waiting and preemption); some are cancelled half-way.  After every step the
    cache manager's books must balance; a request that finishes has the plain greedy tokens, a
    cancelled one a prefix of them; nothing is held at the end."""
    import random

    rng = random.Random(seed)
    which = "AB"[seed % 2]
    block = rng.choice([2, 4, 8])
    longest = 24
    ecfg = EngineConfig(block_size=block,
                        num_blocks=rng.randint(-(-longest // block) + 1, 2 * longest // block),
                        max_batch_size=rng.randint(2, 4), max_num_batched_tokens=rng.choice([8, 13, 32]),
                        max_prefill_chunk=rng.choice([None, 5, 9]), dtype="float32", device="cpu")
    cfg, tensors, engine = engine_for(which, ecfg, seed=7 + seed)
    asked = {}
    for i in range(10):
        n_prompt = rng.randint(1, 14)
        asked[f"r{i}"] = (tokens_for(cfg, n_prompt, 100 * seed + i), rng.randint(1, longest - n_prompt))
    todo = list(asked)
    cancel_at = {f"r{rng.randrange(10)}": rng.randint(1, 6) for _ in range(2)}
    got, reasons, alive = {}, {}, {}
    steps = 0
    while todo or engine.has_unfinished_requests():
        for _ in range(rng.randint(0, 2)):
            if todo:
                rid = todo.pop(0)
                prompt, new = asked[rid]
                engine.add_request(Request(rid, prompt, SamplingParams(max_tokens=new, temperature=0.0)))
                got[rid], alive[rid] = [], 0
        for out in engine.step():
            got[out.request_id].extend(out.new_token_ids)
            if out.finished:
                reasons[out.request_id] = out.finish_reason
        engine.runner.manager.check()
        for rid in alive:
            alive[rid] += 1
            if cancel_at.get(rid) == alive[rid] and rid not in reasons and engine.cancel_request(rid):
                reasons[rid] = "cancelled"
        steps += 1
        assert steps < 2000, "the engine does not finish"
    assert set(reasons) == set(asked)
    for rid, (prompt, new) in asked.items():
        want = plain_greedy(cfg, tensors, prompt, new)
        if reasons[rid] == "cancelled":
            assert got[rid] == want[: len(got[rid])], rid
        else:
            assert reasons[rid] == "length" and got[rid] == want, rid
    stats = engine.stats()
    assert stats["allocated_blocks"] == 0 and stats["running"] == 0 and stats["waiting"] == 0
    engine.runner.manager.check()
