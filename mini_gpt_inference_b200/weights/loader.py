"""Bind checkpoint tensors to a model by name, with one error that tells everything.

Names are the reference's state-dict names (``tok_emb.weight``, ``pos_emb.weight``,
``blocks.{i}.ln1.weight`` ... ``ln_f.weight``, ``lm_head.weight``;
src/minigpt_infer/model.py:43-44, 96-97, 107-110, 123-128), so a converted reference
checkpoint loads as it is.  As in src/minigpt_infer/loader.py:35-38, 107-110 the
wrappers' prefixes ``module.`` and ``_orig_mod.`` are stripped; as in
src/minigpt_infer/loader.py:112-118 a mismatch raises one error that lists missing and
unexpected names — here wrong shapes too.  A tied head stored a second time must equal
the embedding (src/minigpt_infer/loader.py:120-126 asserts shared storage).

Storage dtype is kept: bfloat16 stays bfloat16, 32-bit stays 32-bit, integer tables
become int32.  The cast to the compute dtype happens when the model is placed on the
device (``place_on_device``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsError, load_file

_WRAPPER_PREFIXES = ("module.", "_orig_mod.")


class WeightsError(RuntimeError):
    """The checkpoint does not fit the model.  Carries the three lists."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()) -> None:
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


def strip_wrapper_prefixes(tensors: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    out = dict(tensors)
    for prefix in _WRAPPER_PREFIXES:
        if any(k.startswith(prefix) for k in out):
            out = {(k[len(prefix):] if k.startswith(prefix) else k): v for k, v in out.items()}
    return out


_INTEGER_DTYPES = (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64)


def _keep_storage_dtype(t: torch.Tensor, role: str) -> torch.Tensor | str:
    """The tensor as it is kept (bfloat16 stays bfloat16, 32-bit stays 32-bit, integer tables
    become int32), or a string that says what was expected if its stored dtype is none of these:
    nothing is converted silently."""
    if role == "table":
        return t.to(torch.int32) if t.dtype in _INTEGER_DTYPES else "an integer table"
    return t if t.dtype in (torch.bfloat16, torch.float32) else "bfloat16 or float32"


def check_and_bind(tensors: Mapping[str, torch.Tensor],
                   expected: Mapping[str, TensorSpec], where: str = "checkpoint"
                   ) -> dict[str, torch.Tensor]:
    """Match ``tensors`` against ``expected``; raise one WeightsError naming every fault."""
    tensors = strip_wrapper_prefixes(tensors)
    missing, unexpected, wrong_shape, wrong_dtype, unequal = [], [], [], [], []
    bound: dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in tensors:
            if spec.optional_alias_of is None:
                missing.append(name)
            continue
        t = tensors[name]
        if tuple(t.shape) != tuple(spec.shape):
            wrong_shape.append(f"{name}: checkpoint {tuple(t.shape)}, model {tuple(spec.shape)}")
            continue
        if spec.optional_alias_of is not None:
            other = tensors.get(spec.optional_alias_of)
            if other is not None and other.shape == t.shape and not torch.equal(
                    other.to(torch.float32), t.to(torch.float32)):
                unequal.append(f"{name} differs from {spec.optional_alias_of} (they are tied)")
            continue
        kept = _keep_storage_dtype(t, spec.role)
        if isinstance(kept, str):
            wrong_dtype.append(f"{name}: checkpoint {str(t.dtype).replace('torch.', '')}, model wants {kept}")
            continue
        bound[name] = kept
    for name in tensors:
        if name not in expected:
            unexpected.append(name)
    if missing or unexpected or wrong_shape or wrong_dtype or unequal:
        parts = [f"{where} does not match the model:"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            parts.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if wrong_dtype:
            parts.append(f"  wrong dtype ({len(wrong_dtype)}): " + "; ".join(wrong_dtype))
        if unequal:
            parts.append("  tied tensors differ: " + "; ".join(unequal))
        raise WeightsError("\n".join(parts), missing, unexpected, wrong_shape + unequal, wrong_dtype)
    return bound


def load_checkpoint(model_dir: str | Path, expected: Mapping[str, TensorSpec]
                    ) -> dict[str, torch.Tensor]:
    path = Path(model_dir) / "model.safetensors"
    if not path.is_file():
        raise WeightsError(f"no model.safetensors in {model_dir}")
    try:
        tensors = load_file(path)
    except SafetensorsError as exc:
        raise WeightsError(str(exc)) from exc
    return check_and_bind(tensors, expected, where=str(path))


def place_on_device(bound: Mapping[str, torch.Tensor], expected: Mapping[str, TensorSpec],
                    compute_dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """Matrices go to the compute dtype; vectors (norm gains, biases) are held in 32-bit;
    integer tables stay int32."""
    out = {}
    for name, t in bound.items():
        role = expected[name].role
        if role == "table":
            out[name] = t.to(device=device, dtype=torch.int32).contiguous()
        elif role == "vector":
            out[name] = t.to(device=device, dtype=torch.float32).contiguous()
        else:
            out[name] = t.to(device=device, dtype=compute_dtype).contiguous()
    return out
