"""Causal multi-head attention over the paged cache.

One fused projection gives q, k, v in that order, head ``h`` in columns
``[h*D, (h+1)*D)`` of each (src/minigpt_infer/model.py:43, 50-53).  New keys and values
are written to their pages, then every query attends to the keys of its own request at
positions up to its own (scale ``1/sqrt(D)`` unless given; softmax in 32-bit) — always
from the pages, whether a key arrived in this step or an earlier one, so that the result
does not depend on how the tokens were cut into steps.  The reference gathers the pages
into a dense tensor and calls a library attention (src/minigpt_infer/model.py:55-87,
src/minigpt_infer/cache/paged.py:139-165).  The output projection adds into the
residual stream (src/minigpt_infer/model.py:90, 113).

Heads may share keys (``n_kv_head`` divides ``n_head``) and may look back only
``window`` positions; this architecture uses neither, the part takes them as parameters, and
with them the page size and the pool size of its cache group (layers that agree in all of these
share a group).
"""

from __future__ import annotations

import math

from ..cache.spec import PagedKVSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec


@register_mixer("causal_attention")
class CausalAttention(Mixer):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, bias: bool,
                 n_kv_head: int | None = None, scale: float | None = None,
                 window: int | None = None, cache_page_tokens: int | None = None,
                 cache_pages: int | None = None, position=None) -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim = width, n_head, head_dim
        self.n_kv_head = n_head if n_kv_head is None else n_kv_head
        if self.n_head % self.n_kv_head != 0:
            raise ValueError(f"n_head {n_head} is not a multiple of n_kv_head {self.n_kv_head}")
        self.has_bias = bool(bias)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.window = window
        # page size and pool size of this layer's cache group (None: the cache manager's)
        self.cache_page_tokens, self.cache_pages = cache_page_tokens, cache_pages
        self.position = position
        self.qkv_weight = self.qkv_bias = self.proj_weight = self.proj_bias = None

    @property
    def qkv_width(self) -> int:
        return (self.n_head + 2 * self.n_kv_head) * self.head_dim

    def tensor_specs(self):
        p = self.prefix
        specs = {
            p + "qkv.weight": TensorSpec((self.qkv_width, self.width), "matrix"),
            p + "proj.weight": TensorSpec((self.width, self.n_head * self.head_dim), "matrix",
                                          "residual_proj"),
        }
        if self.has_bias:
            specs[p + "qkv.bias"] = TensorSpec((self.qkv_width,), "vector", "bias")
            specs[p + "proj.bias"] = TensorSpec((self.width,), "vector", "bias")
        return specs

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_head, self.head_dim, self.window, self.cache_page_tokens,
                           self.cache_pages)

    accepts_deferred_norm = True

    def _position_rotates(self) -> bool:
        from .base import PositionEncoding

        return (self.position is not None
                and type(self.position).rotate is not PositionEncoding.rotate)

    def plan_step(self, batch, plan, ops) -> None:
        # the kernel set cuts prompt portions into the tiles of its attention kernel, if it has one
        planner = getattr(ops, "plan_prompt_attention", None)
        if planner is not None:
            planner(batch, plan, self.n_head, self.n_kv_head, self.head_dim)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        slots = ctx.slot_mapping[cache.group]
        if not self._position_rotates() and hasattr(ops, "linear_qkv"):
            # nothing happens between the projection and the page write: one fused call
            qkv = ops.linear_qkv(y, self.qkv_weight, self.qkv_bias, self.n_head, self.n_kv_head,
                                 self.head_dim, cache, slots, ctx.act_dtype)
        else:
            qkv = ops.linear(y, self.qkv_weight, self.qkv_bias, "none", ctx.act_dtype)
            if self.position is not None:
                self.position.rotate(ctx, qkv, self.n_head, self.n_kv_head, self.head_dim)
            if cache.writes:
                ops.kv_store(qkv, self.n_head, self.n_kv_head, self.head_dim, cache, slots)
        out = ops.paged_attention(qkv, self.n_head, self.n_kv_head, self.head_dim, self.scale,
                                  cache, ctx)
        ops.linear_residual(out, self.proj_weight, self.proj_bias, residual32)
