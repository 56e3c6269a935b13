"""A decoder put together from a ``ModelSpec``.

The reference's forward (src/minigpt_infer/model.py:152-187): embed, run the blocks,
final norm, head.  Differences that matter: the order of layers is the spec's list, the
final norm and the head run only on the rows whose logits are wanted (a norm over rows is
row-wise, so selecting first changes nothing), and logits are 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping

from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                   POSITION_ENCODINGS)
from .block import Layer, stream_after
from .spec import ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding, "")
        self.position = POSITION_ENCODINGS.build(spec.position, "")
        self.layers: list[Layer] = []
        for layer_spec in spec.layers:
            p = layer_spec.prefix
            parts, roles = {}, {}
            for name, part_spec in layer_spec.parts.items():
                role = roles[name] = layer_spec.role_of(name)
                if role == "mixer":
                    parts[name] = MIXERS.build(part_spec, p, position=self.position)
                else:
                    parts[name] = (NORMS if role == "norm" else FEED_FORWARDS).build(part_spec, p)
            self.layers.append(Layer(parts, roles, ARRANGEMENTS.get(layer_spec.arrangement), p))
        self.final_norm = NORMS.build(spec.final_norm, "")
        self.head = HEADS.build(spec.head, "", embedding=self.embedding)
        self.layer_order = spec.layer_order

    # ---- tensors ----------------------------------------------------------------------
    def parts(self) -> list[Any]:
        out = [self.embedding, self.position]
        for layer in self.layers:
            out.extend(layer.parts())
        out.extend([self.final_norm, self.head])
        return out

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for part in self.parts():
            for name, spec in part.tensor_specs().items():
                if name in specs:
                    raise ValueError(f"two parts claim the tensor {name!r}")
                specs[name] = spec
        return specs

    def bind(self, tensors: Mapping[str, Any]) -> None:
        for part in self.parts():
            part.bind(tensors)

    @property
    def max_positions(self) -> int | None:
        return self.position.max_positions

    def cache_specs(self) -> list[Any]:
        return [layer.cache_spec() for layer in self.layers]

    # ---- one step ------------------------------------------------------------------------
    def forward(self, ctx):
        """Run ``ctx``'s tokens; return 32-bit logits ``[len(ctx.logit_rows), vocab]``."""
        x = self.embedding.forward(ctx, self.position)
        for call in self.layer_order:
            layer = self.layers[call.layer]
            x = stream_after(layer.run(ctx, layer, ctx.cache_view(call.cache_layer, call.writes_cache), x), x)
        if ctx.logit_rows.numel() == 0:
            return None
        if getattr(self.head, "accepts_deferred_norm", False):
            return self.head.forward(ctx, self.final_norm.defer(ctx, x, ctx.logit_rows))
        rows = ctx.ops.gather_rows(x, ctx.logit_rows)
        return self.head.forward(ctx, self.final_norm.forward(ctx, rows))
