"""Roles a part can play, their interfaces, and one registry per role.

A part is built from a ``PartSpec``'s params alone and never learns which model it is
in.  It names the tensors it wants (``tensor_specs``), receives them (``bind``) and
runs on a ``StepContext``: a flat, ragged batch of tokens that belong to requests, with
the step's metadata on the device.  The residual stream is always 32-bit; what flows
between a norm and the following projection is the compute dtype.

Interfaces (what a new part must provide):

* Norm:             ``forward(ctx, x32) -> y``            y in ctx.act_dtype, same shape
* PositionEncoding: ``table()`` (rows added to the token embedding, or None),
                    ``rotate(ctx, qkv, n_head, n_kv_head, head_dim)`` (in place on the q and
                    k columns of the fused projection; default no-op),
                    ``max_positions`` (None if unbounded)
* Mixer:            built with ``position=`` (the model's position encoding),
                    ``cache_spec()`` (what the layer keeps per request, or None),
                    ``forward(ctx, cache, y, residual32)``  adds its output to residual32 in place
                    and returns None, or returns another tensor that holds the sum
* FeedForward:      ``forward(ctx, y, residual32)``         the same
* Block arrangement: a function ``run(ctx, layer, cache, residual32)`` that wires the layer's
                    named parts and returns the tensor that holds the stream (None: in place).
"""

from __future__ import annotations

from typing import Any, Callable, Mapping

from .spec import PartSpec, TensorSpec


class Part:
    """Common behaviour: name the tensors wanted under a prefix, and take them."""

    kind = ""
    # True if forward() only launches kernels whose arguments do not change from step to step
    # (no host-side reads of the batch): such a part can be captured in a CUDA graph.
    graph_safe = False

    def __init__(self, prefix: str = "") -> None:
        self.prefix = prefix

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def plan_step(self, batch, plan, ops) -> None:
        """Prepare on the host what this part's kernels need for one step besides the batch's own
        integers.  ``batch`` is a ``HostBatch`` (tokens per request, tokens already cached, state
        slots); add int32 arrays to ``plan.arrays[name]`` (they reach ``forward`` as
        ``ctx.extra[name]`` on the device) and to ``plan.signature`` whatever else decides the
        launches.  Called for every step that is not replayed from a captured single-token graph;
        a part that needs a plan in those too sets ``graph_safe = False``.  Default: nothing."""

    def bind(self, tensors: Mapping[str, Any]) -> None:
        """Receive device tensors by full name (only the names of tensor_specs)."""
        for full_name in self.tensor_specs():
            local = full_name[len(self.prefix):].replace(".", "_")
            setattr(self, local, tensors.get(full_name))


class Norm(Part):
    def forward(self, ctx, x32):
        raise NotImplementedError

    def defer(self, ctx, x32, rows=None):
        """The norm as an object that the consuming projection may fuse (see the consumer's
        ``accepts_deferred_norm``).  By default it simply runs."""
        if rows is not None:
            x32 = ctx.ops.gather_rows(x32, rows)
        return self.forward(ctx, x32)


class PositionEncoding(Part):
    max_positions: int | None = None

    def table(self):
        return None

    def rotate(self, ctx, qkv, n_head: int, n_kv_head: int, head_dim: int) -> None:
        return None


class Mixer(Part):
    # True if forward() hands its input only to ctx.ops projections, which understand a
    # deferred norm; then the block passes norm.defer(...) instead of the normalised tensor.
    accepts_deferred_norm = False

    def cache_spec(self):
        return None

    def forward(self, ctx, cache, y, residual32) -> None:
        raise NotImplementedError


class FeedForward(Part):
    accepts_deferred_norm = False

    def forward(self, ctx, y, residual32) -> None:
        raise NotImplementedError


class Registry:
    def __init__(self, role: str) -> None:
        self.role = role
        self._entries: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str):
        def wrap(factory):
            self._entries[kind] = factory
            if isinstance(factory, type) and not getattr(factory, "kind", ""):
                factory.kind = kind
            return factory

        return wrap

    def get(self, kind: str):
        try:
            return self._entries[kind]
        except KeyError:
            known = ", ".join(sorted(self._entries)) or "(none)"
            raise KeyError(f"no {self.role} registered as {kind!r}; known: {known}") from None

    def build(self, spec: PartSpec, prefix: str, **extra):
        factory = self.get(spec.kind)
        return factory(prefix=prefix + (spec.name + "." if spec.name else ""),
                       **dict(spec.params), **extra)

    def __contains__(self, kind: str) -> bool:
        return kind in self._entries


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
ARRANGEMENTS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")

register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_arrangement = ARRANGEMENTS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
