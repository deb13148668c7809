"""The gated delta rule with a decay per key channel, as a recurrent mixer part.

Per head, with q and k unit vectors (q times head_dim ** -0.5), beta = sigmoid(W_b x) and the
decay g = exp(-exp(A_log) * softplus(W_a2 W_a1 x + dt_bias)) per key channel:

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

(the read-out sees the token's own write).  q, k and v come through a short causal
convolution over time, channel by channel, and silu; query/key head h // (H / G) serves head
h.  The head's o is divided by its root mean square, multiplied by a weight shared by the
heads and by sigmoid(W_g2 W_g1 x), and goes through the output product.

Flow of a step: one stacked product  q | k | v | b | a1 | g1;  a row kernel (sums over the
product's partial sums, convolution, silu, unit norms, beta, the two bottlenecks rounded for
their products); the two small products W_a2 a1 and W_g2 g1 into 32-bit; the scan over the
step's tokens, sequence by sequence; the read-out row kernel; the output product.  A prompt
and a decoded token run the same kernels: the state S [H, dv, d] and the convolution's last
taps - 1 inputs live in 32-bit in the sequence's slot of the cache's fixed-size state
(``StateRequest``), zero when the slot is taken, read at the start of a step and written at
its end.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import ChannelDeltaSpec
from .base import ParamSpec, StateRequest, register_mixer
from .linear import Linear


class ChannelDeltaMixer:
    def __init__(self, spec: ChannelDeltaSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if min(spec.n_heads, spec.n_qk_heads, spec.head_dim, spec.value_dim, spec.conv_taps,
               spec.decay_rank, spec.gate_rank) < 1:
            raise ValueError("the sizes of a delta-rule mixer must be positive")
        if spec.n_heads % spec.n_qk_heads:
            raise ValueError("n_heads must be a multiple of n_qk_heads")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        s = spec
        self.n_qk = s.n_qk_heads * s.head_dim
        self.n_v = s.n_heads * s.value_dim
        self.channels = 2 * self.n_qk + self.n_v              # what the convolution runs over
        self.state_numel = s.n_heads * s.value_dim * s.head_dim          # S of every head
        self.conv_off = self.state_numel
        self.in_proj: Optional[Linear] = None
        self.decay_up: Optional[Linear] = None
        self.gate_up: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.conv_w = self.dt_bias = self.neg_a = self.out_norm = None

    @classmethod
    def param_specs(cls, spec: ChannelDeltaSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        s = spec
        nqk, nv = s.n_qk_heads * s.head_dim, s.n_heads * s.value_dim
        return {
            "q_proj.weight": ParamSpec((nqk, hidden_size)),
            "k_proj.weight": ParamSpec((nqk, hidden_size)),
            "v_proj.weight": ParamSpec((nv, hidden_size)),
            "q_conv.weight": ParamSpec((nqk, s.conv_taps), "float32"),
            "k_conv.weight": ParamSpec((nqk, s.conv_taps), "float32"),
            "v_conv.weight": ParamSpec((nv, s.conv_taps), "float32"),
            "beta_proj.weight": ParamSpec((s.n_heads, hidden_size)),
            "a_log": ParamSpec((s.n_heads,), "float32"),
            "dt_bias": ParamSpec((s.n_heads * s.head_dim,), "float32"),
            "decay_down.weight": ParamSpec((s.decay_rank, hidden_size)),
            "decay_up.weight": ParamSpec((s.n_heads * s.head_dim, s.decay_rank)),
            "gate_down.weight": ParamSpec((s.gate_rank, hidden_size)),
            "gate_up.weight": ParamSpec((nv, s.gate_rank)),
            "out_norm.weight": ParamSpec((s.value_dim,), "norm"),
            "o_proj.weight": ParamSpec((hidden_size, nv)),
        }

    def cache_request(self):
        return StateRequest(self.state_numel + (self.spec.conv_taps - 1) * self.channels)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype)

        def f32(name):
            return tensors[name].to(device=device, dtype=torch.float32).contiguous()
        # one product for  q | k | v | b | a1 | g1
        self.in_proj = Linear(torch.cat([
            mat("q_proj.weight"), mat("k_proj.weight"), mat("v_proj.weight"),
            mat("beta_proj.weight"), mat("decay_down.weight"), mat("gate_down.weight")],
            dim=0).contiguous(), role="qkv")
        self.decay_up = Linear(mat("decay_up.weight").contiguous(), role="decay_up")
        self.gate_up = Linear(mat("gate_up.weight").contiguous(), role="gate_up_proj")
        self.out = Linear(mat("o_proj.weight").contiguous(), role="out_proj")
        self.conv_w = torch.cat([f32("q_conv.weight"), f32("k_conv.weight"),
                                 f32("v_conv.weight")], dim=0).contiguous()
        self.dt_bias = f32("dt_bias").reshape(-1)
        self.neg_a = (-torch.exp(f32("a_log"))).contiguous()
        self.out_norm = f32("out_norm.weight")

    def forward(self, x: torch.Tensor, ctx, cache_entry: int, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a recurrent mixer owns the state of its cache entry")
        s = self.spec
        T = x.shape[0]
        H, G, d, dv = s.n_heads, s.n_qk_heads, s.head_dim, s.value_dim
        state = ctx.cache.state_view(cache_entry).state
        proj = self.in_proj.partial(x, cheap_sum=True)
        part = proj if proj.dim() == 3 else None
        f32 = torch.float32
        qkv = ctx.new(T, self.channels, dtype=f32)
        beta = ctx.new(T, H, dtype=f32)
        low_a, low_g = ctx.new(T, s.decay_rank), ctx.new(T, s.gate_rank)
        kernels.delta_prepare(None if part is not None else proj, part, T, ctx, state,
                              self.conv_off, G, H, d, dv, s.conv_taps, s.decay_rank, s.gate_rank,
                              self.conv_w, s.unit_eps, float(d) ** -0.5, qkv, beta, low_a, low_g)
        a = self.decay_up(low_a, out=ctx.new(T, H * d, dtype=f32))
        gate = self.gate_up(low_g, out=ctx.new(T, self.n_v, dtype=f32))
        o = ctx.new(T, self.n_v, dtype=f32)
        kernels.delta_scan(qkv, beta, a, self.dt_bias, self.neg_a, o, ctx, state, G, H, d, dv)
        y = ctx.new(T, self.n_v)
        kernels.delta_out(o, gate, self.out_norm, s.eps, H, dv, ctx, y)
        return self.out.partial(y)


register_mixer("channel_delta", ChannelDeltaMixer)
