"""LayerNorm over the width, statistics in 32-bit.

``y = (x - mean) / sqrt(var + eps) * gain (+ shift)`` with the biased variance, as
``nn.LayerNorm`` in src/minigpt_infer/model.py:107-109, 127 (eps there is the library
default 1e-5; here it is a parameter).  The shift exists only if ``bias``.
"""

from __future__ import annotations

from .base import Norm, register_norm
from .spec import TensorSpec


@register_norm("layernorm")
class LayerNorm(Norm):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, eps: float, bias: bool) -> None:
        super().__init__(prefix)
        self.width, self.eps, self.has_bias = width, float(eps), bool(bias)
        self.weight = None
        self.bias = None

    def tensor_specs(self):
        specs = {self.prefix + "weight": TensorSpec((self.width,), "vector", "norm_gain")}
        if self.has_bias:
            specs[self.prefix + "bias"] = TensorSpec((self.width,), "vector", "norm_shift")
        return specs

    def forward(self, ctx, x32):
        return ctx.ops.layernorm(x32, self.weight, self.bias, self.eps, ctx.act_dtype)

    def defer(self, ctx, x32, rows=None):
        if not hasattr(ctx.ops, "defer_layernorm"):
            return super().defer(ctx, x32, rows)
        return ctx.ops.defer_layernorm(x32, self.weight, self.bias, self.eps, ctx.act_dtype, rows)
