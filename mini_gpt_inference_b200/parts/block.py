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
    mixer, ff = layer.mixer, layer.feed_forward
    y = (layer.norm1.defer if getattr(mixer, "accepts_deferred_norm", False)
         else layer.norm1.forward)(ctx, residual32)
    mixer.forward(ctx, cache, y, residual32)
    y = (layer.norm2.defer if getattr(ff, "accepts_deferred_norm", False)
         else layer.norm2.forward)(ctx, residual32)
    ff.forward(ctx, y, residual32)
