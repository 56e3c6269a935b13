"""Helpers shared by the tests: model folders in a temporary place, token streams, and the
comparison of engine logits with the plain implementation."""

from __future__ import annotations

import torch

import plain_gpt
from tiny_configs import PAGE_TOKENS, tiny_config

from mini_gpt_inference_b200.config import lookup
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import load_file, random_tensors, write_random_model

# Largest allowed |engine - plain| on logits.  32-bit: rounding of a few hundred 32-bit sums.
# bfloat16: the plain side uses the same bfloat16 weights; what differs is the rounding of
# activations to 8 significant bits between kernels (measured about 1.5e-3 on logits whose
# standard deviation is 0.17; a dropped key, bias or page shows as 3e-2 or more).
TOLERANCE = {"float32": 2e-5, "bfloat16": 8e-3}


def sharpen_attention(tensors: dict, cfg, factor: float = 6.0) -> dict:
    """Scale the query and key projections so that the softmax is peaked: each query then
    leans on one or two keys, and a key that is lost, misplaced or read from the wrong page
    moves the logits by far more than any tolerance."""
    out = dict(tensors)
    for i in range(cfg.n_layer):
        w = out[f"blocks.{i}.attn.qkv.weight"].clone().float()
        w[: 2 * cfg.n_embd] *= factor
        out[f"blocks.{i}.attn.qkv.weight"] = w.to(tensors[f"blocks.{i}.attn.qkv.weight"].dtype)
        name = f"blocks.{i}.attn.qkv.bias"
        if name in out:
            b = out[name].clone().float()
            b[: 2 * cfg.n_embd] *= factor
            out[name] = b.to(tensors[name].dtype)
    return out


def make_tensors(cfg, seed: int, dtype: str, sharp: bool = False) -> dict:
    model = DecoderModel(lookup(cfg.architecture).describe(cfg))
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = random_tensors(model, seed, store)
    return sharpen_attention(tensors, cfg) if sharp else tensors


def make_model_dir(tmp_path, which: str, seed: int, dtype: str):
    cfg = tiny_config(which)
    folder = tmp_path / f"tiny_{which}_{dtype}_{seed}"
    write_random_model(folder, cfg, seed, dtype)
    return folder, cfg, load_file(folder / "model.safetensors")


def tokens_for(cfg, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (length,), generator=gen).tolist()


def plain_logits(cfg, tensors, tokens, rows=None) -> torch.Tensor:
    return plain_gpt.forward_logits(tokens, tensors, cfg.n_layer, cfg.n_head,
                                    cfg.layer_norm_epsilon, rows=rows)


def gpu_runner(cfg, tensors, dtype: str, page_tokens: int, num_pages: int, max_requests: int = 8,
               ops=None):
    from mini_gpt_inference_b200.kernels.ops import default_ops

    loaded = load_model(config=cfg, tensors=tensors, dtype=dtype, device="cuda:0")
    return make_runner(loaded, ops or default_ops("cuda:0"), page_tokens, num_pages, max_requests)


def first_mismatch(got: torch.Tensor, want: torch.Tensor, tol: float):
    """Index of the first row whose logits differ by more than tol, with the difference."""
    diff = (got.double().cpu() - want.double()).abs().amax(dim=-1)
    bad = (diff > tol).nonzero()
    if bad.numel() == 0:
        return None, float(diff.max()) if diff.numel() else 0.0
    i = int(bad[0])
    return i, float(diff[i])


def assert_close(got, want, tol, what: str, places=None) -> None:
    i, d = first_mismatch(got, want, tol)
    if i is not None:
        where = places[i] if places is not None else i
        raise AssertionError(f"{what}: first wrong logits at {where}: |diff| = {d:.3e} > {tol:.1e}")


__all__ = ["TOLERANCE", "PAGE_TOKENS", "tiny_config", "sharpen_attention", "make_tensors",
           "make_model_dir", "tokens_for", "plain_logits", "gpu_runner", "first_mismatch",
           "assert_close"]
