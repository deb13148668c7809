"""Rotary position encoding as a table of angles per step.

A position part turns the step's positions into ``(cos, sin)`` tables
``[T, rotary_dim / 2]`` (32-bit); the attention kernels rotate the pairs
(i, i + rotary_dim / 2) of every head with them.  The tables of one spec are
made once per step and shared by all layers that use that spec.  Any encoding
that is a rotation of such pairs fits this interface by giving other tables.
``interleaved`` (pairs (2i, 2i + 1)) is a flag the rotating kernel of a mixer must honour;
``scaling`` blends the frequencies by wavelength and multiplies cos and sin.

angle = (p / factor) * theta^(-2 i / rotary_dim): src/backend/kernels/cpu/rope.zig:11-27,
src/models/gemma3.zig:884-902.  Angles are formed in 64-bit on the device.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import kernels
from ..config.base import RotarySpec
from .base import register_position


class RotaryEmbedding:
    def __init__(self, spec: RotarySpec, head_dim: int):
        self.spec = spec
        self.rotary_dim = spec.rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most "
                             f"head_dim {head_dim}")
        self.interleaved = bool(getattr(spec, "interleaved", False))
        self.scaling = getattr(spec, "scaling", None)
        self._key = ("rotary", float(spec.theta), float(spec.factor), self.rotary_dim, self.scaling)
        self._freqs = None          # 64-bit frequencies on the device, where they are scaled
        self.mult = 1.0

    def frequencies(self):
        """(f [rotary_dim / 2] as Python floats, multiplier of cos and sin) of a spec with
        wavelength scaling: pairs whose wavelength is short against the original context keep
        f_i, long ones turn with f_i / factor, a linear ramp over the pair index between."""
        import math
        sc, dims, base = self.scaling, self.rotary_dim, float(self.spec.theta)
        f = [base ** (-2.0 * i / dims) / float(self.spec.factor) for i in range(dims // 2)]
        if sc is None:
            return f, 1.0
        from ..config.base import BandScalingSpec
        if isinstance(sc, BandScalingSpec):
            # three bands of wavelength: kept, blended, divided by the factor
            out = []
            for fi in f:
                wavelength = 2.0 * math.pi / fi
                if wavelength < sc.original / sc.high:
                    out.append(fi)
                elif wavelength > sc.original / sc.low:
                    out.append(fi / sc.factor)
                else:
                    t = (sc.original / wavelength - sc.low) / (sc.high - sc.low)
                    out.append((1.0 - t) * fi / sc.factor + t * fi)
            return out, 1.0

        def pair_of(turns: float) -> float:
            return dims * math.log(sc.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(sc.fast)), 0)
        hi = min(math.ceil(pair_of(sc.slow)), dims - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            out.append(fi / sc.factor * ramp + fi * (1.0 - ramp))
        return out, 0.1 * math.log(sc.factor) + 1.0

    def prepare(self, device) -> None:
        """Put the scaled frequencies on the device (at load time, so that no step, recorded
        or not, has to copy them there)."""
        if self.scaling is not None:
            f, self.mult = self.frequencies()
            self._freqs = torch.tensor(f, dtype=torch.float64, device=device)

    def tables(self, ctx) -> Tuple[torch.Tensor, torch.Tensor]:
        hit = ctx.rope_tables.get(self._key)
        if hit is None:
            half = self.rotary_dim // 2
            cos = ctx.new(ctx.n_tokens, half, dtype=torch.float32)
            sin = ctx.new(ctx.n_tokens, half, dtype=torch.float32)
            if self.scaling is None:
                kernels.rope_table(ctx.positions, self.rotary_dim, self.spec.theta,
                                   self.spec.factor, cos, sin)
            else:
                if self._freqs is None or self._freqs.device != cos.device:
                    self.prepare(cos.device)
                kernels.rope_table_freqs(ctx.positions, self._freqs, self.mult, cos, sin)
            hit = ctx.rope_tables[self._key] = (cos, sin)
        return hit


register_position("rotary", RotaryEmbedding)
