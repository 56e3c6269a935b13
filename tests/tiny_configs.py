"""Two tiny configurations of the architecture that differ in every size and option."""

from __future__ import annotations

from mini_gpt_inference_b200.config import GPTConfig

TINY_A = dict(vocab_size=256, n_positions=64, n_layer=2, n_head=4, n_embd=64, n_inner=256,
              bias=True, layer_norm_epsilon=1e-5)
TINY_B = dict(vocab_size=509, n_positions=128, n_layer=3, n_head=3, n_embd=96, n_inner=200,
              bias=False, layer_norm_epsilon=3e-4)
# The second tiny configuration as the task's own list of configurations words it (MLP 384, eps 1e-5);
# B above differs from A in those two as well.
TINY_C = dict(vocab_size=509, n_positions=128, n_layer=3, n_head=3, n_embd=96, n_inner=384,
              bias=False, layer_norm_epsilon=1e-5)
PAGE_TOKENS = {"A": 16, "B": 8, "C": 8}


def tiny_config(which: str) -> GPTConfig:
    return GPTConfig.from_dict({"A": TINY_A, "B": TINY_B, "C": TINY_C}[which])
