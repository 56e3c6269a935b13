"""From a model folder to a runnable model with its cache: the one place where the
registry, the loader, the parts and the cache are put together."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.registry import load_config, lookup
from ..parts.model import DecoderModel
from ..weights.loader import check_and_bind, load_checkpoint, place_on_device
from .runner import ModelRunner

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class LoadedModel:
    config: Any
    model: DecoderModel
    dtype: torch.dtype
    device: torch.device


def load_model(model_dir: str | Path | None = None, *, config=None, tensors=None,
               dtype: str = "bfloat16", device="cuda:0") -> LoadedModel:
    """Build the model named by ``model_dir/config.json`` and bind its checkpoint.
    Alternatively pass a typed ``config`` and a dict of CPU ``tensors``."""
    if model_dir is not None:
        family, config = load_config(model_dir)
    else:
        family = lookup(config.architecture)
    model = DecoderModel(family.describe(config))
    expected = model.tensor_specs()
    if model_dir is not None:
        bound = load_checkpoint(model_dir, expected)
    else:
        bound = check_and_bind(tensors, expected, where="given tensors")
    compute = _TORCH_DTYPES[dtype]
    model.bind(place_on_device(bound, expected, compute, device))
    return LoadedModel(config, model, compute, torch.device(device))


def make_runner(loaded: LoadedModel, ops, page_tokens: int, num_pages: int,
                max_requests: int, use_cuda_graphs: bool = True,
                max_step_tokens: int | None = None) -> ModelRunner:
    """``page_tokens`` and ``num_pages``: the geometry of every cache group that names none of its
    own.  ``max_step_tokens``: the most tokens one request brings in a step, if the caller keeps
    to such a bound (cache groups with a window then get smaller pools)."""
    manager = CacheManager(loaded.model.cache_specs(), page_tokens, num_pages, max_requests,
                           window_slack_tokens=max_step_tokens)
    storage = CacheStorage(manager, loaded.dtype, loaded.device)
    return ModelRunner(loaded.model, manager, storage, ops, loaded.dtype, loaded.device,
                       use_cuda_graphs=use_cuda_graphs)
