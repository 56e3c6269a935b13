"""Token embedding (plus the position table's rows, if the position encoding has one) and
the output head that shares its matrix.

``x = tok_emb[id] + pos_emb[pos]`` into the 32-bit residual stream
(src/minigpt_infer/model.py:183); ``logits = y @ tok_emb^T`` without bias, 32-bit out
(src/minigpt_infer/model.py:128-130, 187).
"""

from __future__ import annotations

from .base import Part, register_embedding, register_head
from .spec import TensorSpec


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step
    # forward() honours ctx.token_source / ctx.fed_ids (tokens taken from the ids that the step
    # before sampled); an embedding without this flag gets its tokens gathered by a kernel in front.
    takes_token_source = True

    def __init__(self, prefix: str, vocab_size: int, width: int) -> None:
        super().__init__(prefix)
        self.vocab_size, self.width = vocab_size, width
        self.weight = None

    def tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.width), "matrix")}

    def forward(self, ctx, position):
        table = position.table() if position is not None else None
        if getattr(ctx, "token_source", None) is not None:
            # some tokens are still on the device where the step before sampled them
            return ctx.ops.embed(ctx.token_ids, ctx.positions, self.weight, table,
                                 source=ctx.token_source, previous=ctx.fed_ids)
        return ctx.ops.embed(ctx.token_ids, ctx.positions, self.weight, table)


@register_head("tied_head")
class TiedHead(Part):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    """Output projection with the embedding's matrix.  A checkpoint may store it again
    under the head's own name; then it must equal the embedding."""

    def __init__(self, prefix: str, vocab_size: int, width: int, tied_to: str,
                 embedding=None) -> None:
        super().__init__(prefix)
        self.vocab_size, self.width, self.tied_to = vocab_size, width, tied_to
        self.embedding = embedding

    def tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.width), "matrix",
                                                   optional_alias_of=self.tied_to)}

    accepts_deferred_norm = True

    def bind(self, tensors) -> None:
        return None

    def forward(self, ctx, y):
        greedy_out = getattr(ctx, "greedy_out", None)
        if greedy_out is not None:
            # the step also wants each row's greedy choice: the projection may take it on its way
            logits, ctx.greedy_taken = ctx.ops.logits(y, self.embedding.weight, greedy_out,
                                                      getattr(ctx, "greedy_vocab_limit", None))
            return logits
        return ctx.ops.logits(y, self.embedding.weight)
