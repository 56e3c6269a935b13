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


def _run_stream(engine, cfg, arrivals, cancel_at=None):
    """Drive the engine step by step, adding requests at given step numbers; returns per request
    (tokens, finish reason) and the number of steps."""
    results, step = {}, 0
    pending = sorted(arrivals, key=lambda a: a[0])
    while pending or engine.has_unfinished_requests():
        while pending and pending[0][0] <= step:
            _, req = pending.pop(0)
            engine.add_request(req)
            results[req.request_id] = [[], None]
        if cancel_at and step == cancel_at[0]:
            engine.cancel_request(cancel_at[1])
        for out in engine.step():
            results[out.request_id][0].extend(out.new_token_ids)
            if out.finished:
                results[out.request_id][1] = out.finish_reason
        step += 1
        assert step < 2000
    return results


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_decoding_gives_the_same_answers_one_step_late(dtype):
    """With the host one step behind the device (tokens fed back on the device, ids read late),
    every request gets the same tokens and finish reasons as with the host in lock step: also
    when a request ends on an end-of-text or stop token that the host sees only after the next
    step was launched, when requests arrive in the middle, and when one is cancelled."""
    base = dict(block_size=8, num_blocks=40, max_batch_size=4, max_num_batched_tokens=16, max_prefill_chunk=9)
    answers = []
    for overlap in (False, True):
        cfg, tensors, engine = engine_for("B", dtype, sharp=False, overlap_decode=overlap, **base)
        prompts = [tokens_for(cfg, n, 80 + i) for i, n in enumerate([7, 3, 12, 5, 9])]
        # what the first request generates decides its end-of-text and the second's stop token
        probe = engine.generate([prompts[0], prompts[1]], SamplingParams(max_tokens=9, temperature=0.0))
        eot = probe[0]["token_ids"][4]
        stop = probe[1]["token_ids"][6]
        arrivals = [
            (0, Request("a", prompts[0], SamplingParams(max_tokens=30, temperature=0.0), eot_token_id=eot)),
            (0, Request("b", prompts[1], SamplingParams(max_tokens=30, temperature=0.0, stop_token_ids=[stop]))),
            (3, Request("c", prompts[2], SamplingParams(max_tokens=11, temperature=0.7, top_k=20, seed=5))),
            (9, Request("d", prompts[3], SamplingParams(max_tokens=1, temperature=0.0))),
            (10, Request("e", prompts[4], SamplingParams(max_tokens=25, temperature=0.0))),
        ]
        results = _run_stream(engine, cfg, arrivals, cancel_at=(14, "e"))
        assert results["a"][1] == "eot" and results["a"][0][-1] == eot
        assert results["b"][1] == "stop" and results["b"][0][-1] == stop
        assert results["c"][1] == "length" and len(results["c"][0]) == 11
        assert results["d"] == [results["d"][0], "length"] and len(results["d"][0]) == 1
        assert engine.stats()["allocated_blocks"] == 0 and engine.stats()["free_state_slots"] == 4
        engine.runner.manager.check()
        if overlap:
            assert engine.num_overlapped_steps > 5
        else:
            assert engine.num_overlapped_steps == 0
        answers.append({k: v for k, v in results.items() if k != "e"})
    assert answers[0] == answers[1]


@pytest.mark.parametrize("overlap", [False, True])
def test_a_kernel_that_gave_up_stops_generation(overlap):
    """A kernel whose bounded wait ran out leaves a code in the status word and skips its work.
    The engine reads that word with every step's ids: generation raises instead of returning
    tokens sampled from invalid logits, the word is cleared, and the engine works afterwards."""
    from mini_gpt_inference_b200.kernels.library import KernelLibraryError

    cfg, tensors, engine = engine_for("A", "bfloat16", block_size=8, num_blocks=32, max_batch_size=2,
                                      overlap_decode=overlap)
    prompt = tokens_for(cfg, 5, 3)
    params = SamplingParams(max_tokens=6, temperature=0.0)
    good = engine.generate([prompt], params)[0]["token_ids"]
    engine.runner.ops.status.fill_(3)                       # what such a kernel would have written
    with pytest.raises(KernelLibraryError, match="gave up waiting"):
        engine.generate([prompt], params)
    assert int(engine.runner.ops.status.item()) == 0
    # a fresh engine on the same kernel set is unaffected
    _, _, again = engine_for("A", "bfloat16", block_size=8, num_blocks=32, max_batch_size=2,
                             overlap_decode=overlap)
    assert again.generate([prompt], params)[0]["token_ids"] == good


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_seven_with_portions_of_13_and_forced_preemption(dtype):
    """The second tiny configuration as the task's list words it (MLP 384, eps 1e-5, pages of 8):
    prompts of 1 to 100 tokens, seven running at a time, prompt portions of at most 13 tokens, and a
    pool too small for seven long requests, so that some give way and are recomputed."""
    cfg, tensors, engine = engine_for("C", dtype, sharp=False, block_size=8, num_blocks=44, max_batch_size=7,
                                      max_num_batched_tokens=32, max_prefill_chunk=13)
    lengths = [100, 1, 57, 13, 88, 26, 14, 2, 71, 39]
    prompts = [tokens_for(cfg, n, 90 + i) for i, n in enumerate(lengths)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=14, temperature=0.0))
    assert engine.scheduler.num_preemptions > 0
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 14
        assert_greedy(cfg, tensors, prompt, out["token_ids"], TOLERANCE[dtype])
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_warm_up_captures_the_decode_graphs_ahead_and_changes_no_token(dtype):
    """warm_up() captures the graphs of all decode batch sizes up to max_batch_size before the first
    request; generation afterwards captures nothing more and gives the tokens of a cold engine."""
    kw = dict(block_size=8, num_blocks=64, max_batch_size=6, max_num_batched_tokens=32)
    cfg, tensors, cold = engine_for("A", dtype, **kw)
    prompts = [tokens_for(cfg, n, 70 + i) for i, n in enumerate([9, 3, 14, 6, 11])]
    params = SamplingParams(max_tokens=9, temperature=0.0)
    want = [o["token_ids"] for o in cold.generate(prompts, params)]
    _, _, warm = engine_for("A", dtype, **kw)
    assert warm.warm_up() == {"decode_graphs_captured": 4}            # rows 1, 2, 4, 8
    assert sorted(warm.runner._graphs) == [1, 2, 4, 8]
    assert warm.warm_up() == {"decode_graphs_captured": 0}            # nothing left to do
    assert warm.stats()["allocated_blocks"] == 0                      # padding rows hold no page
    got = [o["token_ids"] for o in warm.generate(prompts, params)]
    assert sorted(warm.runner._graphs) == [1, 2, 4, 8] and warm.runner.graph_replays > 0
    if dtype == "float32":
        assert got == want
    for prompt, tokens in zip(prompts, got):
        assert_greedy(cfg, tensors, prompt, tokens, TOLERANCE[dtype])
    _, _, eager = engine_for("A", dtype, use_cuda_graphs=False, **kw)
    assert eager.warm_up() == {"decode_graphs_captured": 0}
