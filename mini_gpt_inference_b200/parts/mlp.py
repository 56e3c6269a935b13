"""Dense feed-forward: ``proj(act(fc(y)))`` added into the residual stream.

The reference's MLP (src/minigpt_infer/model.py:93-101) with its hidden width and its
activation as parameters; ``gelu_tanh(u) = 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))``
is evaluated in 32-bit inside the first projection's epilogue.
"""

from __future__ import annotations

from .base import FeedForward, register_feed_forward
from .spec import TensorSpec

_ACTIVATIONS = {"gelu_tanh": "gelu_tanh", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh"}


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, inner: int, bias: bool,
                 activation: str = "gelu_tanh") -> None:
        super().__init__(prefix)
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel epilogue; known: "
                             + ", ".join(sorted(_ACTIVATIONS)))
        self.width, self.inner, self.has_bias = width, inner, bool(bias)
        self.activation = _ACTIVATIONS[activation]
        self.fc_weight = self.fc_bias = self.proj_weight = self.proj_bias = None

    def tensor_specs(self):
        p = self.prefix
        specs = {
            p + "fc.weight": TensorSpec((self.inner, self.width), "matrix"),
            p + "proj.weight": TensorSpec((self.width, self.inner), "matrix", "residual_proj"),
        }
        if self.has_bias:
            specs[p + "fc.bias"] = TensorSpec((self.inner,), "vector", "bias")
            specs[p + "proj.bias"] = TensorSpec((self.width,), "vector", "bias")
        return specs

    accepts_deferred_norm = True

    def forward(self, ctx, y, residual32):
        whole = getattr(ctx.ops, "mlp_residual", None)
        if whole is not None:
            # the kernel set may run both projections as one kernel; it returns where the sum lies
            return whole(y, self.fc_weight, self.fc_bias, self.proj_weight, self.proj_bias, self.activation,
                         residual32, ctx.act_dtype)
        h = ctx.ops.linear(y, self.fc_weight, self.fc_bias, self.activation, ctx.act_dtype)
        ctx.ops.linear_residual(h, self.proj_weight, self.proj_bias, residual32)
        return None
