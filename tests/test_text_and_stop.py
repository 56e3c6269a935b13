"""Text while tokens arrive, and stop strings (src/minigpt_infer/tokenizer.py:49-97,
src/minigpt_infer/engine/engine.py:186-205), with a toy byte-level vocabulary on the CPU double."""

from __future__ import annotations

import pytest

from harness import make_tensors, tiny_config, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, Request, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model
from mini_gpt_inference_b200.engine.text import IncrementalText, cut_at_stop


def test_characters_spread_over_tokens_are_held_until_whole():
    euro = "€".encode()                        # three bytes
    table = {0: b"a", 1: euro[:1], 2: euro[1:2], 3: euro[2:], 4: b"\xff", 5: "é".encode()[:1]}
    text = IncrementalText(table.__getitem__)
    assert [text.add_token(t) for t in (0, 1, 2, 3, 0)] == ["a", "", "", "€", "a"]
    assert text.text == "a€a"
    assert text.add_token(4) == "�"         # a byte that can start nothing is not held back
    assert text.add_token(5) == "" and text.finalize() == "�"
    assert text.finalize() == ""


def test_cut_at_stop():
    assert cut_at_stop("hello world", "world", ["wor"]) == ("", "wor")
    assert cut_at_stop("hello world", "lo world", [" w", "zzz"]) == ("lo", " w")
    assert cut_at_stop("hello world", "d", ["o w"]) == ("", "o w")        # began before this delta
    assert cut_at_stop("hello", "lo", ["x", ""]) == ("lo", None)
    assert cut_at_stop("abcabc", "abc", ["c", "bc"]) == ("", "bc")        # the earliest occurrence


def _engine(token_bytes=None):
    cfg = tiny_config("A")
    tensors = make_tensors(cfg, 5, "float32", sharp=True)
    loaded = load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")
    ecfg = EngineConfig(block_size=8, num_blocks=32, max_batch_size=2, dtype="float32", device="cpu")
    return cfg, LLMEngine(loaded, ecfg, ops=TorchOps(), token_bytes=token_bytes)


def test_stop_strings_need_text_and_end_the_request():
    cfg, plain = _engine()
    prompt = tokens_for(cfg, 5, 1)
    with pytest.raises(ValueError, match="stop strings"):
        plain.add_request(Request("x", prompt, SamplingParams(max_tokens=4, stop=["ab"])))
    ids = plain.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0))[0]["token_ids"]

    def token_bytes(t):                          # token t is the letter chr(97 + t % 26)
        return bytes([97 + t % 26])

    letters = "".join(chr(97 + t % 26) for t in ids)
    stop = letters[4:6]
    first = letters.find(stop)
    cfg, engine = _engine(token_bytes)
    out = engine.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0, stop=[stop]))[0]
    assert out["finish_reason"] == "stop"
    assert out["token_ids"] == ids[: first + 2]          # it ends with the token that completed the stop string
    assert out["text"] == letters[:first]                # and the text ends where the stop string begins
    free = engine.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0))[0]
    assert free["text"] == letters and free["finish_reason"] == "length"
    assert engine.stats()["allocated_blocks"] == 0
