"""Dense gated feed-forward: down(act(gate x) * up x), no biases
(src/models/gemma3.zig:840-872); the activation and the product are the
epilogue of the gate/up kernel.

Interface of a feed-forward part:
  ``param_specs(spec, hidden) -> {local name: ParamSpec}``      (class method)
  ``load(tensors, dtype, device)``
  ``forward(x [T, hidden], ctx) -> y [T, hidden]`` (or ``[S, T, hidden]`` 32-bit
  partial sums, which the norm that follows adds)
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import DenseFeedForwardSpec, GatedFeedForwardSpec
from .base import ParamSpec, register_feed_forward
from .linear import GatedLinear, Linear


class GatedFeedForward:
    def __init__(self, spec: GatedFeedForwardSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        self.spec, self.hidden_size = spec, hidden_size
        self.gate_up: Optional[GatedLinear] = None
        self.down: Optional[Linear] = None

    @classmethod
    def param_specs(cls, spec: GatedFeedForwardSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        ff = spec.intermediate_size
        return {
            "gate_proj.weight": ParamSpec((ff, hidden_size)),
            "up_proj.weight": ParamSpec((ff, hidden_size)),
            "down_proj.weight": ParamSpec((hidden_size, ff)),
        }

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype).contiguous()
        self.gate_up = GatedLinear(mat("gate_proj.weight"), mat("up_proj.weight"),
                                   self.spec.activation)
        self.down = Linear(mat("down_proj.weight"), role="down")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.down.partial(self.gate_up(x))


register_feed_forward("gated_dense", GatedFeedForward)


class DenseFeedForward:
    """down(act(up x)): no gate.  "relu2" is the squared relu, max(z, 0)^2; "gelu_erf" is
    z / 2 * (1 + erf(z / sqrt 2))."""

    def __init__(self, spec: DenseFeedForwardSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.activation not in ("relu2", "gelu_erf"):
            raise ValueError(f"dense feed-forward: unknown activation {spec.activation!r}")
        self.spec, self.hidden_size = spec, hidden_size
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    @classmethod
    def param_specs(cls, spec: DenseFeedForwardSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        ff = spec.intermediate_size
        return {"up_proj.weight": ParamSpec((ff, hidden_size)),
                "down_proj.weight": ParamSpec((hidden_size, ff))}

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        self.up = Linear(tensors["up_proj.weight"].to(device=device, dtype=dtype).contiguous(),
                         role="up")
        self.down = Linear(tensors["down_proj.weight"].to(device=device, dtype=dtype).contiguous(),
                           role="down")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        z = self.up.activated(x, self.spec.activation)
        return self.down.partial(z)


register_feed_forward("dense", DenseFeedForward)
