"""Position encodings that are added to the residual stream after the embedding.

Interface of a stream position (what the decoder needs):
  ``param_specs(spec, hidden) -> {local name: ParamSpec}``      (class method)
  ``load(tensors, device)``
  ``forward(h [T, hidden] 32-bit, ctx)``: adds to h in place from ``ctx.positions``

``LearnedPosition``: one learned vector per position, times the spec's scale.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import LearnedPositionSpec
from .base import ParamSpec, register_stream_position


class LearnedPosition:
    def __init__(self, spec: LearnedPositionSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.positions < 1:
            raise ValueError("a learned position table needs at least one row")
        self.spec, self.hidden_size, self.dtype = spec, hidden_size, dtype
        self.table: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, spec: LearnedPositionSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        return {"table.weight": ParamSpec((spec.positions, hidden_size), "embedding")}

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        self.table = tensors["table.weight"].to(device=device, dtype=self.dtype).contiguous()

    def forward(self, h: torch.Tensor, ctx) -> None:
        kernels.add_position_rows(ctx.positions, self.table, h, float(self.spec.scale))


register_stream_position("learned", LearnedPosition)
