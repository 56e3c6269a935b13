"""Compare the tests' plain implementation with the reference's own model code, once.

Run on the CPU from the repository root, with the reference checkout beside it:

    python tests/golden/make_golden.py /path/to/mini-gpt-inference

It builds the reference's ``ReferenceGPT`` (src/minigpt_infer/reference.py:78-114) and
``GPT`` at two tiny sizes, loads this repository's seeded random tensors into them by
name, and checks that ``tests/plain_gpt.py`` gives the same logits at every position
(64-bit, max abs difference < 1e-9) and the same greedy tokens.  It then stores the
token ids, the seed and the logits of a few positions in ``tests/golden/*.json`` so that
``tests/test_plain_reference.py`` can hold the plain implementation to them without the
reference being present.  The reference fixes the MLP width to 4 x n_embd and eps to
1e-5, so both golden configurations keep those; tiny B's other options are covered by
the formulas alone.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import plain_gpt  # noqa: E402
from mini_gpt_inference_b200.config import GPTConfig, lookup  # noqa: E402
from mini_gpt_inference_b200.parts import DecoderModel  # noqa: E402
from mini_gpt_inference_b200.weights import random_tensors  # noqa: E402

CASES = {
    "golden_a": dict(vocab_size=256, n_positions=64, n_layer=2, n_head=4, n_embd=64, bias=True,
                     seed=11, length=40, new=6),
    "golden_b": dict(vocab_size=509, n_positions=128, n_layer=3, n_head=3, n_embd=96, bias=False,
                     seed=12, length=70, new=6),
}


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "src"))
    from minigpt_infer.config import GPTConfig as RefConfig
    from minigpt_infer.reference import ReferenceGPT

    for name, case in CASES.items():
        case = dict(case)
        seed, length, new = case.pop("seed"), case.pop("length"), case.pop("new")
        cfg = GPTConfig.from_dict(case)
        model = DecoderModel(lookup(cfg.architecture).describe(cfg))
        tensors = random_tensors(model, seed)
        ref = ReferenceGPT(RefConfig(vocab_size=cfg.vocab_size, block_size=cfg.n_positions,
                                     n_layer=cfg.n_layer, n_head=cfg.n_head, n_embd=cfg.n_embd,
                                     bias=cfg.bias)).double().eval()
        state = {k: v.double() for k, v in tensors.items()}
        state["lm_head.weight"] = state["tok_emb.weight"]
        missing, unexpected = ref.load_state_dict(state, strict=False)
        assert not missing and not unexpected, (missing, unexpected)
        gen = torch.Generator().manual_seed(seed + 1000)
        tokens = torch.randint(0, cfg.vocab_size, (length,), generator=gen).tolist()
        with torch.no_grad():
            ref_logits = ref(torch.tensor([tokens]))[0]
            ref_greedy = ref.greedy_generate(torch.tensor([tokens]), new)[0, length:].tolist()
        ours = plain_gpt.forward_logits(tokens, tensors, cfg.n_layer, cfg.n_head,
                                        cfg.layer_norm_epsilon)
        diff = (ours - ref_logits).abs().max().item()
        greedy = plain_gpt.greedy_generate(tokens, tensors, cfg.n_layer, cfg.n_head,
                                           cfg.layer_norm_epsilon, new)
        assert diff < 1e-9, f"{name}: plain implementation differs from the reference by {diff}"
        assert greedy == ref_greedy, (greedy, ref_greedy)
        keep = [0, 1, length // 2, length - 1]
        out = {"config": case, "seed": seed, "tokens": tokens, "positions": keep,
               "max_abs_diff_plain_vs_reference": diff,
               "logits_first_16": {str(p): ref_logits[p, :16].tolist() for p in keep},
               "logit_row_sums": {str(p): ref_logits[p].sum().item() for p in keep},
               "greedy_tokens": ref_greedy}
        path = Path(__file__).parent / f"{name}.json"
        path.write_text(json.dumps(out, indent=1) + "\n")
        print(f"{name}: max |plain - reference| = {diff:.3e}; greedy {ref_greedy}; wrote {path}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
