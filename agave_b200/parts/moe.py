"""Routed feed-forward (mixture of experts) as a feed-forward part.

Every token uses ``top`` of ``n_experts`` small gated feed-forwards
down_e(act(gate_e x) * up_e x).  Router: s = sigmoid(W_r x) in 32-bit; the choice scores
s + correction pick (restricted to the experts of the best ``keep_groups`` of ``n_groups``
equal groups of neighbours, a group scoring the sum of its two largest choice scores), the
plain s weigh, not renormalised; the output is the weighted sum of the chosen experts'.

Flow of a step (all decided on the device, so a step records into a CUDA graph):
router -> plan (the (token, choice) pairs laid out by expert, each expert's run padded to
the row tile) -> gate/up as one grouped product with the activation in its epilogue ->
down as a grouped product whose epilogue multiplies by the pair's weight and scatters to
[choice, token, :].  In bfloat16 the grouped products run on the tensor cores (tcgen05 +
TMA, ``csrc/moe_tcgen05.cu``), in 32-bit and for odd sizes as FFMA dot products
(``csrc/moe.cu``).  That 32-bit tensor is returned as partial sums: the norm that
follows adds the choices in order, as it adds the ranges of K of a dense projection.

The experts' matrices are stacked [E, ...] at load time so that a tile finds its expert
by index.

Options of the spec: a bias on the router's logits (``router_bias``); weights that are the
softmax over the chosen experts' logits, the logits making the choice (``weighting``
"softmax_top"); and a shared expert of the same form that every token uses, its output
multiplied by sigmoid(w_sg . x), one number per token (``shared_size``): it is one more
slice of the partial sums; scores that are the softmax over all the router's outputs, with the
chosen ones renormalised and multiplied by a constant (``weighting`` "softmax_all",
``route_scale``); and identity experts (``n_identity``): router outputs beyond the experts
that have no tensors and whose output is the input itself, times the weight.  A pair that
chose one is left out of the plan, and a small kernel writes its row of the partial sums.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import RoutedFeedForwardSpec
from .base import ParamSpec, register_feed_forward
from .linear import GatedLinear, Linear


class RoutedFeedForward:
    def __init__(self, spec: RoutedFeedForwardSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.n_experts % spec.n_groups:
            raise ValueError("the experts must form equal groups")
        if not 1 <= spec.keep_groups <= spec.n_groups:
            raise ValueError("keep_groups must lie in 1..n_groups")
        if spec.top > spec.keep_groups * (spec.n_experts // spec.n_groups) + \
                int(getattr(spec, "n_identity", 0) or 0):
            raise ValueError("top exceeds the experts of the groups kept")
        self.spec, self.hidden_size, self.dtype = spec, hidden_size, dtype
        self.weighting = getattr(spec, "weighting", "sigmoid")
        self.n_identity = int(getattr(spec, "n_identity", 0) or 0)
        self.route_scale = float(getattr(spec, "route_scale", 1.0))
        if self.n_identity < 0 or (self.n_identity and spec.n_groups != 1):
            raise ValueError("identity experts go with ungrouped routing")
        if self.weighting not in ("sigmoid", "softmax_top", "softmax_all"):
            raise ValueError(f"unknown expert weighting {self.weighting!r}")
        if self.weighting == "softmax_top" and spec.correction:
            raise ValueError("weights by softmax over the chosen logits go without a correction")
        self.has_bias = bool(getattr(spec, "router_bias", False))
        self.shared_size = int(getattr(spec, "shared_size", 0) or 0)
        self.router_bias: Optional[torch.Tensor] = None
        self.shared_gate_up = self.shared_down = self.shared_gate = None
        self.w_router: Optional[torch.Tensor] = None
        self.correction: Optional[torch.Tensor] = None
        self.w_gate = self.w_up = self.w_down = None

    @classmethod
    def param_specs(cls, spec: RoutedFeedForwardSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        ff = spec.intermediate_size
        n_out = spec.n_experts + int(getattr(spec, "n_identity", 0) or 0)
        p = {"router.weight": ParamSpec((n_out, hidden_size))}
        if spec.correction:
            p["router.correction"] = ParamSpec((n_out,), "float32")
        for e in range(spec.n_experts):
            p[f"experts.{e}.gate_proj.weight"] = ParamSpec((ff, hidden_size))
            p[f"experts.{e}.up_proj.weight"] = ParamSpec((ff, hidden_size))
            p[f"experts.{e}.down_proj.weight"] = ParamSpec((hidden_size, ff))
        if getattr(spec, "router_bias", False):
            p["router.bias"] = ParamSpec((spec.n_experts,), "float32")
        sf = int(getattr(spec, "shared_size", 0) or 0)
        if sf:
            p["shared.gate_proj.weight"] = ParamSpec((sf, hidden_size))
            p["shared.up_proj.weight"] = ParamSpec((sf, hidden_size))
            p["shared.down_proj.weight"] = ParamSpec((hidden_size, sf))
            p["shared.gate.weight"] = ParamSpec((1, hidden_size))
        return p

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def stack(name):
            return torch.stack([tensors[f"experts.{e}.{name}.weight"].to(device=device, dtype=dtype)
                                for e in range(self.spec.n_experts)]).contiguous()
        self.w_router = tensors["router.weight"].to(device=device, dtype=dtype).contiguous()
        if self.spec.correction:
            self.correction = tensors["router.correction"].to(
                device=device, dtype=torch.float32).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate_proj"), stack("up_proj"), stack("down_proj")
        if self.has_bias:
            self.router_bias = tensors["router.bias"].to(device=device,
                                                         dtype=torch.float32).contiguous()
        if self.shared_size:
            def mat(name):
                return tensors[name].to(device=device, dtype=dtype).contiguous()
            self.shared_gate_up = GatedLinear(mat("shared.gate_proj.weight"),
                                              mat("shared.up_proj.weight"), self.spec.activation,
                                              role="shared_gate_up")
            self.shared_down = Linear(mat("shared.down_proj.weight"), role="shared_down")
            self.shared_gate = mat("shared.gate.weight").reshape(-1).contiguous()

    def route(self, x: torch.Tensor):
        """(ids [T, top] int32, weights [T, top] 32-bit) of the tokens of x."""
        s = self.spec
        T = x.shape[0]
        ids = torch.empty((T, s.top), dtype=torch.int32, device=x.device)
        wts = torch.empty((T, s.top), dtype=torch.float32, device=x.device)
        kernels.moe_route(x, self.w_router, self.correction, s.n_groups, s.keep_groups, s.top,
                          ids, wts, bias=self.router_bias,
                          softmax_top=self.weighting == "softmax_top",
                          softmax_all=self.weighting == "softmax_all", scale=self.route_scale)
        return ids, wts

    def _shared(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """out [T, H] (32-bit) = sigmoid(w_sg . x) * down(act(gate x) * up x)."""
        self.shared_down(self.shared_gate_up(x), out=out)
        kernels.row_gate(x, self.shared_gate, out)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s = self.spec
        T, H = x.shape
        ids, wts = self.route(x)
        plan = kernels.moe_plan(ids, wts, s.n_experts)
        z = torch.empty((plan.rows, s.intermediate_size), dtype=x.dtype, device=x.device)
        n_sh = 1 if self.shared_size else 0
        y = torch.empty((s.top + n_sh, T, H), dtype=torch.float32, device=x.device)
        if n_sh:
            self._shared(x, y[s.top])
        if self.n_identity:
            kernels.moe_identity(x, ids, wts, s.n_experts, y[:s.top])
        if (kernels.moe_grouped_tc_supported(x, self.w_gate) and
                kernels.moe_grouped_tc_supported(z, self.w_down)):
            # bfloat16 on the tensor cores: the tokens are brought into the plan's order
            # first, so that a tile's rows come as one TMA box
            xs = torch.empty((plan.rows, H), dtype=x.dtype, device=x.device)
            kernels.moe_gather_rows(x, plan, xs)
            kernels.moe_grouped_tc(xs, self.w_gate, z, plan, w2=self.w_up,
                                   activation=s.activation, op="experts_gate_up")
            kernels.moe_grouped_tc(z, self.w_down, y[:s.top].view(s.top * T, H), plan, scatter=True,
                                   op="experts_down")
            return y
        kernels.moe_grouped(x, self.w_gate, z, plan, w2=self.w_up, activation=s.activation,
                            gather=True, op="experts_gate_up")
        kernels.moe_grouped(z, self.w_down, y[:s.top].view(s.top * T, H), plan, scatter=True,
                            op="experts_down")
        return y


register_feed_forward("routed", RoutedFeedForward)
