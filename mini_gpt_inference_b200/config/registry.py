"""One registry from an architecture's name to its configuration and model description.

The reference has a single model class and no registry (src/minigpt_infer/loader.py:88-136
builds ``GPT`` directly).  Here ``config.json`` names the architecture
(``architectures[0]`` or ``model_type``) and everything else — the loader, the
engine, the replay program — asks this registry for it.

A family is a pair: a configuration class with ``from_dict`` and a function that
turns a configuration into a ``ModelSpec`` (a plain description of parts per
layer and of the order in which layers run).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping


class UnknownArchitectureError(KeyError):
    pass


@dataclass(frozen=True)
class ModelFamily:
    name: str
    config_class: Any                      # has from_dict(raw, architecture=...)
    describe: Callable[[Any], Any]         # config -> parts.spec.ModelSpec


MODEL_REGISTRY: dict[str, ModelFamily] = {}

# A config.json without "architectures"/"model_type" is taken to be the reference's own
# field dict (src/minigpt_infer/config.py:10-18 has no architecture name at all).
DEFAULT_ARCHITECTURE = "MiniGPTLMHeadModel"


def register_model(name: str, *aliases: str, config_class: Any):
    """Decorator for a ``describe(config) -> ModelSpec`` function."""

    def wrap(describe: Callable[[Any], Any]):
        family = ModelFamily(name=name, config_class=config_class, describe=describe)
        for key in (name, *aliases):
            MODEL_REGISTRY[key] = family
        return describe

    return wrap


def architecture_name(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    if isinstance(archs, str):
        return archs
    if raw.get("model_type"):
        return str(raw["model_type"])
    return DEFAULT_ARCHITECTURE


def lookup(name: str) -> ModelFamily:
    _ensure_builtin_models()
    try:
        return MODEL_REGISTRY[name]
    except KeyError:
        known = ", ".join(sorted(MODEL_REGISTRY)) or "(none)"
        raise UnknownArchitectureError(
            f"architecture {name!r} is not registered; known: {known}") from None


def family_for(raw: Mapping[str, Any]) -> ModelFamily:
    return lookup(architecture_name(raw))


def load_config(model_dir) -> tuple[ModelFamily, Any]:
    """Read ``model_dir/config.json`` and return (family, typed configuration)."""
    from pathlib import Path

    from .model_config import read_config_json

    raw = read_config_json(Path(model_dir) / "config.json")
    family = family_for(raw)
    return family, family.config_class.from_dict(raw, architecture=family.name)


def _ensure_builtin_models() -> None:
    # Importing the module registers the family; done lazily to avoid an import cycle.
    from ..models import minigpt  # noqa: F401
