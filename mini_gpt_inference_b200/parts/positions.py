"""Position encodings.

``learned_absolute``: a table with one row per position, added to the token embedding
(src/minigpt_infer/model.py:124, 183).  It bounds the context: a position beyond the
table is an error (src/minigpt_infer/model.py:177-182).  It does nothing to q and k.
"""

from __future__ import annotations

from .base import PositionEncoding, register_position_encoding
from .spec import TensorSpec


@register_position_encoding("learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, n_positions: int, width: int) -> None:
        super().__init__(prefix)
        self.n_positions, self.width = n_positions, width
        self.max_positions = n_positions
        self.weight = None

    def tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.n_positions, self.width), "matrix")}

    def table(self):
        return self.weight


@register_position_encoding("none")
class NoPositions(PositionEncoding):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str = "") -> None:
        super().__init__(prefix)
