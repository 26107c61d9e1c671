"""Learned absolute positions: a table with one row per position, added to the residual stream
right after the embedding (no factor).  A position encoding of the whole model
(``ModelSpec.position``), not of a mixer: mixers below it see positions only through what
they add themselves (a window, a penalty on the distance)."""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import POSITIONS, Position


@POSITIONS.register("learned")
class LearnedPositions(Position):
    def __init__(self, spec, prefix, dtype, device, head_dim=None):
        super().__init__(spec, prefix, dtype, device)
        self.rows = int(spec["positions"])
        self.width = int(spec["size"])
        self.tensor = self.prefix + str(spec.get("tensor", "weight"))
        self.table = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.rows, self.width), role="matrix")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors.pop(self.tensor)

    def add_to_stream(self, x32: torch.Tensor, ctx) -> None:
        K.add_position_rows(x32, self.table, ctx.positions)
