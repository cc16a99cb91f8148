"""Learned absolute positions: a table with one row a position, added to the embedding.

``x[t] += table[position[t]]`` on the fp32 residual, once a step, before the first layer
(``ModelSpec.embedding_position``).  The table's length is the longest sequence the model takes.
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import POSITION_ENCODINGS, PositionEncoding, StepContext, TensorSpec


@POSITION_ENCODINGS.register("learned")
class LearnedPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, *, name: str, max_positions: int, hidden_size: int, dtype: torch.dtype, device: str, **_: object) -> None:
        self.name = name
        self.max_positions = max_positions
        self.hidden_size = hidden_size
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.max_positions, self.hidden_size))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()

    def embed_hook(self, residual: torch.Tensor, ctx: StepContext) -> None:
        kernels.add_positions(self.table, ctx.positions, residual, ctx.error_flag)
