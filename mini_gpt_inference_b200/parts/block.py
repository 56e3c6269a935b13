"""A layer at run time, and how its parts are wired.

A block arrangement is a function ``run(ctx, layer, cache, residual32)`` registered under a name;
it finds the layer's parts by the names it expects (``layer.norm1`` ...) and says which names
those are in ``requires``, so that a layer that lacks one is refused when the model is built.
Mixers and feed-forwards add their output to the 32-bit residual stream: in place (they return
nothing), or into another tensor that they return (a kernel that fuses the whole part cannot
always write where it reads); an arrangement hands the stream on with ``stream_after`` and
returns the tensor that holds it at the end (or nothing, if that is the one it was given).
``pre_norm``: ``x += mixer(norm1(x)); x += ff(norm2(x))`` (src/minigpt_infer/model.py:112-115).
"""

from __future__ import annotations

from typing import Any, Callable

from .base import register_arrangement


class Layer:
    """The built parts of one layer, by their names in the layer, and the arrangement's function."""

    def __init__(self, parts: dict[str, Any], roles: dict[str, str], run: Callable[..., None],
                 prefix: str = "") -> None:
        self._parts = dict(parts)
        self.roles = dict(roles)
        self.run = run
        self.prefix = prefix
        missing = [n for n in getattr(run, "requires", ()) if n not in self._parts]
        if missing:
            raise ValueError(f"layer {prefix!r}: its arrangement needs parts named {missing}; "
                             f"it has {sorted(self._parts)}")

    def __getattr__(self, name: str):
        try:
            return self.__dict__["_parts"][name]
        except KeyError:
            raise AttributeError(f"layer {self.__dict__.get('prefix', '')!r} has no part {name!r}") from None

    def parts(self) -> list:
        return list(self._parts.values())

    def cache_spec(self):
        """What the layer keeps per request: its mixer's wish.  One cache per layer: of several
        mixers at most one may keep something."""
        specs = [spec for name, part in self._parts.items() if self.roles[name] == "mixer"
                 for spec in [part.cache_spec()] if spec is not None]
        if len(specs) > 1:
            raise ValueError(f"layer {self.prefix!r}: more than one of its mixers keeps a cache")
        return specs[0] if specs else None


def _normed(ctx, norm, consumer, residual32):
    """The norm's result, as a deferred norm if its consumer can fuse it."""
    run = norm.defer if getattr(consumer, "accepts_deferred_norm", False) else norm.forward
    return run(ctx, residual32)


def stream_after(returned, residual32):
    """The tensor that holds the residual stream after a part ran: what the part returned, or, if
    it returned nothing, the tensor it was given (it added in place)."""
    return residual32 if returned is None else returned


def pre_norm(ctx, layer: Layer, cache, residual32):
    x = residual32
    x = stream_after(layer.mixer.forward(ctx, cache, _normed(ctx, layer.norm1, layer.mixer, x), x), x)
    return stream_after(layer.feed_forward.forward(ctx, _normed(ctx, layer.norm2, layer.feed_forward, x), x), x)


pre_norm.requires = ("norm1", "mixer", "norm2", "feed_forward")
register_arrangement("pre_norm")(pre_norm)
