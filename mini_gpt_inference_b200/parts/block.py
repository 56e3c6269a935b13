"""How a layer's parts are wired.  ``pre_norm``: ``x += mixer(norm1(x)); x += ff(norm2(x))``
(src/minigpt_infer/model.py:112-115)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .base import register_arrangement


@dataclass
class Layer:
    norm1: Any
    mixer: Any
    norm2: Any
    feed_forward: Any
    run: Callable[..., None]

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]


@register_arrangement("pre_norm")
def pre_norm(ctx, layer: Layer, cache, residual32) -> None:
    y = layer.norm1.forward(ctx, residual32)
    layer.mixer.forward(ctx, cache, y, residual32)
    y = layer.norm2.forward(ctx, residual32)
    layer.feed_forward.forward(ctx, y, residual32)
