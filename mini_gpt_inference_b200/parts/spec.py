"""Plain-data description of a model: which part sits where, and in which order layers run.

A ``ModelSpec`` is what an architecture's ``describe(config)`` returns.  It holds no
tensors and no code: parts are named by registry key (``kind``) with their sizes and
constants as ``params``; ``layer_order`` is a list, so a layer may run twice or use
another layer's cache.  ``parts.build`` turns it into runnable parts.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


ROLES = ("norm", "mixer", "feed_forward")


@dataclass(frozen=True)
class PartSpec:
    kind: str                               # key in the part registry of its role
    params: Mapping[str, Any] = field(default_factory=dict)
    name: str = ""                          # weight-name prefix inside its parent ("ln1", "attn")
    role: str = ""                          # inside a layer: "norm" | "mixer" | "feed_forward"; if empty,
                                            # taken from the part's name in the layer (see LayerSpec)


@dataclass(frozen=True)
class LayerSpec:
    """A layer is a bag of named parts and the name of the arrangement that wires them.  What
    names an arrangement expects is the arrangement's business (``pre_norm`` wants ``norm1``,
    ``mixer``, ``norm2``, ``feed_forward``); a layer with one norm, without a feed-forward or
    with two mixers is another arrangement over another bag, not another schema."""

    prefix: str                             # weight-name prefix of the layer ("blocks.0.")
    parts: Mapping[str, PartSpec]           # name in the layer -> part
    arrangement: str = "pre_norm"           # key in the block-arrangement registry

    def role_of(self, name: str) -> str:
        role = self.parts[name].role
        if not role:
            role = next((r for r in ROLES if name == r or name.startswith(r)), "")
        if role not in ROLES:
            raise ValueError(f"layer {self.prefix!r}: part {name!r} has no role; set PartSpec.role to "
                             f"one of {ROLES} or name it after its role")
        return role


def pre_norm_layer(prefix: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec,
                   feed_forward: PartSpec) -> LayerSpec:
    """The usual block: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``."""
    return LayerSpec(prefix, {"norm1": norm1, "mixer": mixer, "norm2": norm2,
                              "feed_forward": feed_forward}, "pre_norm")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run ``layer`` against the cache of ``cache_layer``."""

    layer: int
    cache_layer: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab_size: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    layer_order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        n = len(self.layers)
        for call in self.layer_order:
            if not (0 <= call.layer < n and 0 <= call.cache_layer < n):
                raise ValueError(f"layer_order entry {call} names a layer outside 0..{n - 1}")


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint."""

    shape: tuple[int, ...]
    role: str = "matrix"        # "matrix": stored in the compute dtype; "vector": kept in 32-bit;
                                # "table": integer table kept as int32
    init: str = "normal"        # random-weights mode: "normal" | "residual_proj" | "norm_gain" |
                                # "norm_shift" | "bias"
    optional_alias_of: str | None = None   # e.g. lm_head.weight may repeat tok_emb.weight
