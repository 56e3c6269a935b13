"""Random-weights mode: write a model folder from a configuration and a seed.

The scheme follows the reference's initialisation (src/minigpt_infer/model.py:132-144):
matrices ``N(0, 0.02)``, residual output projections (names ending ``proj.weight``)
``N(0, 0.02 / sqrt(2 * n_layer))``.  The reference zeroes biases and leaves norm gains at
one; here norm gains are ``1 + N(0, 0.1)``, norm shifts ``N(0, 0.1)`` and biases
``N(0, 0.02)``, so that a kernel that drops a bias or an affine term shows up in a test.
Tensors are drawn in sorted name order from one CPU generator, so a seed fixes them.
"""

from __future__ import annotations

import math
from pathlib import Path

import torch

from ..config.registry import lookup
from ..parts.model import DecoderModel
from .safetensors_io import save_file


def random_tensors(model: DecoderModel, seed: int, dtype: torch.dtype = torch.float32
                   ) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    n_layer = max(1, len(model.layers))
    out: dict[str, torch.Tensor] = {}
    specs = model.tensor_specs()
    for name in sorted(specs):
        spec = specs[name]
        if spec.optional_alias_of is not None:
            continue
        if spec.role == "table":
            out[name] = torch.randint(0, 2**15, spec.shape, generator=gen, dtype=torch.int32)
            continue
        noise = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if spec.init == "residual_proj":
            t = noise * (0.02 / math.sqrt(2 * n_layer))
        elif spec.init == "norm_gain":
            t = 1.0 + 0.1 * noise
        elif spec.init == "norm_shift":
            t = 0.1 * noise
        else:  # "normal", "bias"
            t = 0.02 * noise
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str | Path, config, seed: int,
                       dtype: str | torch.dtype = "float32") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``."""
    if isinstance(dtype, str):
        dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    model_dir = Path(model_dir)
    family = lookup(config.architecture)
    model = DecoderModel(family.describe(config))
    config.save(model_dir)
    save_file(random_tensors(model, seed, dtype), model_dir / "model.safetensors",
              metadata={"format": "pt", "seed": str(seed)})
    return model_dir
