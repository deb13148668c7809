"""RMS norm: x * w / sqrt(mean(x^2) + eps), statistics in 32-bit.

The weight is kept in 32-bit; a zero-centred norm stores w and multiplies by
1 + w, which is formed once at load time (the reference does the same when it
warms its norm cache, src/models/gemma3.zig:908-954).

Interface of a norm part (what a block needs):
  ``forward(h, out, rows=None)``      out = norm(h[rows]) for the 32-bit stream h
  ``residual(h, y, nxt, x_out, mult=1)``      h += mult * self(y); x_out = nxt(h) if nxt
  ``after_residual(h, y, x_out, mult=1)``     h += mult * y; x_out = self(h)
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import IdentityNormSpec, LayerNormSpec, NormSpec
from .base import ParamSpec, register_norm


class RMSNorm:
    def __init__(self, spec: NormSpec, width: int, dtype: torch.dtype, device: torch.device):
        self.spec, self.width = spec, width
        self.eps = float(spec.eps)
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, spec: NormSpec, width: int) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((width,), "norm", zero_centered=spec.zero_centered)}

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        w = tensors["weight"].to(device=device, dtype=torch.float32)
        self.weight = (w + 1.0 if self.spec.zero_centered else w).contiguous()

    def forward(self, h: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.norm_residual(h, None, None, self.weight, out, eps_next=self.eps, rows=rows)
        return out

    def residual(self, h: torch.Tensor, y: torch.Tensor, nxt, x_out, mult: float = 1.0) -> None:
        """h += mult * self(y); x_out = nxt(h) if nxt (one launch when nxt is an RMS norm
        and there is no multiplier)."""
        if mult != 1.0:
            kernels.layer_norm_join(h, y, self.weight, None, None, None, None, eps_post=self.eps,
                                    mult=mult, rms=True)
            if nxt is not None:
                nxt.forward(h, x_out)
        elif nxt is None or isinstance(nxt, RMSNorm):
            fused_residual(h, y, self, nxt, x_out)
        elif isinstance(nxt, Identity):
            # the stream itself, rounded, is what follows: one launch
            kernels.layer_norm_join(h, y, self.weight, None, None, None, x_out,
                                    eps_post=self.eps, rms=True)
        else:
            fused_residual(h, y, self, None, None)
            nxt.forward(h, x_out)

    def after_residual(self, h: torch.Tensor, y: torch.Tensor, x_out: torch.Tensor,
                       mult: float = 1.0) -> None:
        """h += mult * y; x_out = self(h)."""
        if mult != 1.0:
            kernels.layer_norm_join(h, y, None, None, self.weight, None, x_out,
                                    eps_next=self.eps, mult=mult, rms=True)
        else:
            fused_residual(h, y, None, self, x_out)


def fused_residual(h: torch.Tensor, y: torch.Tensor, post: Optional[RMSNorm],
                   nxt: Optional[RMSNorm], x_out: Optional[torch.Tensor]) -> None:
    """h += post(y) (or y); x_out = nxt(h): one launch for RMS norms."""
    kernels.norm_residual(
        h, y, post.weight if post is not None else None,
        nxt.weight if nxt is not None else None, x_out if nxt is not None else None,
        eps_post=post.eps if post is not None else 0.0,
        eps_next=nxt.eps if nxt is not None else 0.0)


class LayerNorm:
    """(x - mean) / sqrt(var + eps) * w + b, statistics in 32-bit; the same interface,
    and the same fusion of branch norm, residual sum and next norm into one launch."""

    def __init__(self, spec: LayerNormSpec, width: int, dtype: torch.dtype, device: torch.device):
        self.spec, self.width = spec, width
        self.eps = float(spec.eps)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, spec: LayerNormSpec, width: int) -> Dict[str, ParamSpec]:
        p = {"weight": ParamSpec((width,), "norm")}
        if spec.bias:
            p["bias"] = ParamSpec((width,), "norm_bias")
        return p

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()
        if self.spec.bias:
            self.bias = tensors["bias"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.layer_norm_join(h, None, None, None, self.weight, self.bias, out,
                                eps_next=self.eps, rows=rows)
        return out

    def residual(self, h: torch.Tensor, y: torch.Tensor, nxt, x_out, mult: float = 1.0) -> None:
        """h += mult * self(y); x_out = nxt(h) if nxt (one launch when nxt is a layer norm or
        no norm at all)."""
        if isinstance(nxt, Identity):
            kernels.layer_norm_join(h, y, self.weight, self.bias, None, None, x_out,
                                    eps_post=self.eps, mult=mult)
        elif nxt is None or isinstance(nxt, LayerNorm):
            kernels.layer_norm_join(
                h, y, self.weight, self.bias, nxt.weight if nxt is not None else None,
                nxt.bias if nxt is not None else None, x_out if nxt is not None else None,
                eps_post=self.eps, eps_next=nxt.eps if nxt is not None else 0.0, mult=mult)
        else:
            kernels.layer_norm_join(h, y, self.weight, self.bias, None, None, None,
                                    eps_post=self.eps, mult=mult)
            nxt.forward(h, x_out)

    def after_residual(self, h: torch.Tensor, y: torch.Tensor, x_out: torch.Tensor,
                       mult: float = 1.0) -> None:
        """h += mult * y; x_out = self(h)."""
        kernels.layer_norm_join(h, y, None, None, self.weight, self.bias, x_out,
                                eps_next=self.eps, mult=mult)


class Identity:
    """No norm: the part that follows reads the 32-bit stream itself, rounded to the compute
    dtype.  It has no tensors; the same interface, so that a block can stand before or after
    blocks with norms."""

    def __init__(self, spec: IdentityNormSpec, width: int, dtype: torch.dtype,
                 device: torch.device):
        self.spec, self.width = spec, width

    @classmethod
    def param_specs(cls, spec: IdentityNormSpec, width: int) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        pass

    def forward(self, h: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.layer_norm_join(h, None, None, None, None, None, out, rows=rows)
        return out

    def after_residual(self, h: torch.Tensor, y: torch.Tensor, x_out: torch.Tensor,
                       mult: float = 1.0) -> None:
        """h += mult * y; x_out = h."""
        kernels.layer_norm_join(h, y, None, None, None, None, x_out, mult=mult)


register_norm("identity", Identity)
register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
