"""The plain implementation itself: held to the logits that the reference's own model gave
(tests/golden/*.json, written by tests/golden/make_golden.py), and each part to its formula
through torch's own functions."""

from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

import plain_gpt
from mini_gpt_inference_b200.config import GPTConfig, lookup
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import random_tensors

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["golden_a", "golden_b"])
def test_plain_matches_the_reference_models_logits(name):
    g = json.loads((GOLDEN / f"{name}.json").read_text())
    cfg = GPTConfig.from_dict(g["config"])
    tensors = random_tensors(DecoderModel(lookup(cfg.architecture).describe(cfg)), g["seed"])
    logits = plain_gpt.forward_logits(g["tokens"], tensors, cfg.n_layer, cfg.n_head,
                                      cfg.layer_norm_epsilon)
    for p in g["positions"]:
        want = torch.tensor(g["logits_first_16"][str(p)], dtype=torch.float64)
        assert torch.allclose(logits[p, :16], want, atol=1e-12, rtol=0)
        assert abs(logits[p].sum().item() - g["logit_row_sums"][str(p)]) < 1e-9
    assert g["max_abs_diff_plain_vs_reference"] < 1e-9
    greedy = plain_gpt.greedy_generate(g["tokens"], tensors, cfg.n_layer, cfg.n_head,
                                       cfg.layer_norm_epsilon, len(g["greedy_tokens"]))
    assert greedy == g["greedy_tokens"]


def test_parts_against_torch_functions():
    torch.manual_seed(0)
    x = torch.randn(9, 24, dtype=torch.float64)
    gain, shift = torch.randn(24, dtype=torch.float64), torch.randn(24, dtype=torch.float64)
    assert torch.allclose(plain_gpt.layer_norm(x, gain, shift, 3e-4),
                          F.layer_norm(x, (24,), gain, shift, 3e-4), atol=1e-12)
    assert torch.allclose(plain_gpt.layer_norm(x, gain, None, 1e-5),
                          F.layer_norm(x, (24,), gain, None, 1e-5), atol=1e-12)
    assert torch.allclose(plain_gpt.gelu_tanh(x), F.gelu(x, approximate="tanh"), atol=1e-12)
    w, b = torch.randn(7, 24, dtype=torch.float64), torch.randn(7, dtype=torch.float64)
    assert torch.allclose(plain_gpt.linear(x, w, b), F.linear(x, w, b), atol=1e-12)


def test_attention_order_of_q_k_v_and_causality():
    torch.manual_seed(1)
    T, C, H = 6, 12, 3
    w = {"qkv.weight": torch.randn(3 * C, C, dtype=torch.float64),
         "qkv.bias": torch.randn(3 * C, dtype=torch.float64),
         "proj.weight": torch.eye(C, dtype=torch.float64)}
    x = torch.randn(T, C, dtype=torch.float64)
    got = plain_gpt.causal_attention(x, w, "", H)
    q, k, v = F.linear(x, w["qkv.weight"], w["qkv.bias"]).split(C, dim=1)
    q, k, v = (t.reshape(T, H, C // H).transpose(0, 1) for t in (q, k, v))
    want = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(0, 1).reshape(T, C)
    assert torch.allclose(got, want, atol=1e-12)
    # a later token never changes an earlier position
    x2 = x.clone()
    x2[-1] += 1.0
    assert torch.allclose(plain_gpt.causal_attention(x2, w, "", H)[:-1], got[:-1], atol=1e-12)
    # a window of one sees only itself: output = v of the same position
    alone = plain_gpt.causal_attention(x, w, "", H, window=1)
    assert torch.allclose(alone, v.transpose(0, 1).reshape(T, C), atol=1e-12)


def test_sampling_distribution_rules():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0], dtype=torch.float64)
    p = plain_gpt.sampling_distribution(logits, 1.0, top_k=2)
    assert (p > 0).tolist() == [True, True, False, False, False]
    assert torch.allclose(p[:2], torch.softmax(logits[:2], 0))
    # top-p always keeps the first and grows with p (tests/test_sampling.py:33-52)
    kept = [int((plain_gpt.sampling_distribution(logits, 1.0, top_p=q) > 0).sum())
            for q in (0.01, 0.5, 0.8, 0.95, 1.0)]
    assert kept[0] == 1 and kept == sorted(kept) and kept[-1] == 5
    cold = plain_gpt.sampling_distribution(logits, 0.0)
    assert cold.argmax() == 0 and cold[0] > 0.999999
