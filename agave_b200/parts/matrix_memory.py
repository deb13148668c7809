"""A matrix memory with exponential gates (the mLSTM of xLSTM) as a recurrent mixer part.

Per head, with q = W_q x * d ** -0.5, k = W_k x, v = W_v x, a log input gate
i = cap * tanh((W_i x + b_i) / cap), a log forget gate f = logsigmoid(cap * tanh((W_f x + b_f)
/ cap)) and a running maximum m that starts at 0:

    m_t = max(f + m_(t-1), i)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T        n_t: the same with k alone
    o   = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps)

Every head's o is divided by its root mean square, multiplied by a weight per channel and by
sigmoid(W_g x), and goes through the output product.

Flow of a step: one stacked product  q | k | v | g | i | f  into 32-bit sums; a row kernel
(q scaled, the two gates capped and taken to logarithms); the scan over the step's tokens,
sequence by sequence, which leaves S^T q, n . q and exp(-m); the read-out row kernel (the
division, norm, weight, gate, rounding); the output product.  A prompt and a decoded token run
the same kernels: S [H, d, dv], n [H, d] and m (a copy per CTA of a head's scan) live in 32-bit
in the sequence's slot of the cache's fixed-size state (``StateRequest``), zero when the slot
is taken (the running maximum's start), read at the start of a step and written at its end.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import MatrixMemorySpec
from .base import ParamSpec, StateRequest, register_mixer
from .linear import Linear


def project_f32(lin: Linear, x: torch.Tensor):
    """(rows, partial sums) of x w^T in 32-bit: partial sums [S, T, N] over ranges of K where
    the tensor cores take the product, else the rows [T, N]; one of the two is None."""
    if kernels.linear_tc_supported(x, lin.weight):
        return None, lin.partial(x, cheap_sum=True)
    out = torch.empty((x.shape[0], lin.out_features), dtype=torch.float32, device=x.device)
    kernels.linear(x, lin.weight, out, op=lin.role)
    return out, None


class MatrixMemoryMixer:
    def __init__(self, spec: MatrixMemorySpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if min(spec.n_heads, spec.head_dim, spec.value_dim) < 1 or spec.gate_cap <= 0:
            raise ValueError("the sizes and the gate cap of a matrix memory must be positive")
        if spec.head_dim > 256:
            raise ValueError("a matrix memory's key heads are at most 256 wide")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        self.state_numel = kernels.mlstm_state_numel(spec.n_heads, spec.head_dim, spec.value_dim)
        self.in_proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.bias_i = self.bias_f = self.out_norm = None

    @classmethod
    def param_specs(cls, spec: MatrixMemorySpec, hidden_size: int) -> Dict[str, ParamSpec]:
        nq, nv = spec.n_heads * spec.head_dim, spec.n_heads * spec.value_dim
        return {
            "q_proj.weight": ParamSpec((nq, hidden_size)),
            "k_proj.weight": ParamSpec((nq, hidden_size)),
            "v_proj.weight": ParamSpec((nv, hidden_size)),
            "g_proj.weight": ParamSpec((nv, hidden_size)),
            "i_proj.weight": ParamSpec((spec.n_heads, hidden_size)),
            "i_proj.bias": ParamSpec((spec.n_heads,), "float32"),
            "f_proj.weight": ParamSpec((spec.n_heads, hidden_size)),
            "f_proj.bias": ParamSpec((spec.n_heads,), "float32"),
            "out_norm.weight": ParamSpec((nv,), "norm"),
            "o_proj.weight": ParamSpec((hidden_size, nv)),
        }

    def cache_request(self):
        return StateRequest(self.state_numel)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype)

        def f32(name):
            return tensors[name].to(device=device, dtype=torch.float32).reshape(-1).contiguous()
        # one product for  q | k | v | g | i | f
        self.in_proj = Linear(torch.cat([
            mat("q_proj.weight"), mat("k_proj.weight"), mat("v_proj.weight"),
            mat("g_proj.weight"), mat("i_proj.weight"), mat("f_proj.weight")],
            dim=0).contiguous(), role="qkv")
        self.out = Linear(mat("o_proj.weight").contiguous(), role="out_proj")
        self.bias_i, self.bias_f = f32("i_proj.bias"), f32("f_proj.bias")
        self.out_norm = f32("out_norm.weight")

    def forward(self, x: torch.Tensor, ctx, cache_entry: int, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a recurrent mixer owns the state of its cache entry")
        s = self.spec
        T = x.shape[0]
        H, d, dv = s.n_heads, s.head_dim, s.value_dim
        state = ctx.cache.state_view(cache_entry).state
        row, part = project_f32(self.in_proj, x)
        f32 = torch.float32
        qkv = ctx.new(T, 2 * H * d + H * dv, dtype=f32)
        gates = ctx.new(T, 2 * H, dtype=f32)
        kernels.mlstm_prepare(row, part, T, H, d, dv, self.bias_i, self.bias_f, float(s.gate_cap),
                              float(d) ** -0.5, qkv, gates)
        num = ctx.new(T, H * dv, dtype=f32)
        den = ctx.new(T, H, 2, dtype=f32)
        kernels.mlstm_scan(qkv, gates, num, den, ctx, state, H, d, dv)
        y = ctx.new(T, H * dv)
        kernels.mlstm_out(num, den, float(s.den_eps), row, part, self.out_norm, float(s.eps), H, d,
                          dv, y)
        return self.out.partial(y)


register_mixer("matrix_memory", MatrixMemoryMixer)
