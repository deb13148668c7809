"""One layer: mixer and feed-forward between norms, over a 32-bit residual stream.

"sandwich" (src/models/gemma3.zig:708-709,824-826,835-836,876-878):
    h += post_mixer_norm(mixer(pre_mixer_norm(h)))
    h += post_ffn_norm(ffn(pre_ffn_norm(h)))
"pre": the same without the two post norms.
"post": the same without the two pre norms: a branch reads the stream itself.
``residual_mult`` m: every branch joins as h += m * (...).  A spec without a feed-forward
gives a layer of the mixer branch alone (and no norms of the second branch).
``token_side``: after the feed-forward (or, without one, after the mixer) the layer takes an
input from the token itself: with e the layer's slice of the token's row of a table the
layers share (``ctx.token_side_rows``), g = gelu_tanh(W_gate h) * e, y = W_proj g and
h += y / rms(y) * w; tensors ``side.gate_proj.weight``, ``side.proj.weight``,
``side.norm.weight``.

The residual sum, the norm of the branch and the norm that feeds the next
branch are one kernel launch, so a block receives its input already normed
(``x``) and returns the input of whatever runs next, normed with that part's
own input norm (``next_norm``; None after the last block).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import BlockSpec, IdentityNormSpec, NormSpec
from .base import ParamSpec, feed_forward_class, mixer_class, norm_class, register_block
from .linear import Linear
from .norm import fused_residual


class Block:
    def __init__(self, spec: BlockSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.arrangement not in ("sandwich", "pre", "post"):
            raise ValueError(f"unknown block arrangement {spec.arrangement!r}")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        N = norm_class(spec.norm.kind)
        self.sandwich = spec.arrangement in ("sandwich", "post")      # branches are normed
        self.mult = float(getattr(spec, "residual_mult", 1.0))
        has_ffn = spec.feed_forward is not None
        # where a branch has no norm before it, the "identity" norm part stands in
        P, pspec = N, spec.norm
        if spec.arrangement == "post":
            pspec = IdentityNormSpec()
            P = norm_class(pspec.kind)
        self.pre_mixer_norm = P(pspec, hidden_size, dtype, device)
        self.pre_ffn_norm = P(pspec, hidden_size, dtype, device) if has_ffn else None
        self.post_mixer_norm = N(spec.norm, hidden_size, dtype, device) if self.sandwich else None
        self.post_ffn_norm = (N(spec.norm, hidden_size, dtype, device)
                              if self.sandwich and has_ffn else None)
        self.mixer = mixer_class(spec.mixer.kind)(spec.mixer, hidden_size, dtype, device)
        self.ffn = (feed_forward_class(spec.feed_forward.kind)(spec.feed_forward, hidden_size,
                                                               dtype, device) if has_ffn else None)
        self.side = getattr(spec, "token_side", None)
        self.side_gate: Optional[Linear] = None
        self.side_proj: Optional[Linear] = None
        self.side_in = self.side_norm = None
        if self.side is not None:
            if self.side.dim < 1 or self.side.offset < 0:
                raise ValueError("a token input needs a positive width and an offset in its table")
            # the gate reads the stream itself; the branch joins through a plain RMS norm
            self.side_in = norm_class("identity")(IdentityNormSpec(), hidden_size, dtype, device)
            self.side_norm = norm_class("rmsnorm")(
                NormSpec(eps=self.side.eps, zero_centered=False), hidden_size, dtype, device)

    @classmethod
    def param_specs(cls, spec: BlockSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        N = norm_class(spec.norm.kind)
        has_ffn = spec.feed_forward is not None
        names = []
        if spec.arrangement != "post":
            names += ["pre_mixer_norm"] + (["pre_ffn_norm"] if has_ffn else [])
        if spec.arrangement != "pre":
            names += ["post_mixer_norm"] + (["post_ffn_norm"] if has_ffn else [])
        out: Dict[str, ParamSpec] = {}
        for n in names:
            for k, v in N.param_specs(spec.norm, hidden_size).items():
                out[f"{n}.{k}"] = v
        for k, v in mixer_class(spec.mixer.kind).param_specs(spec.mixer, hidden_size).items():
            out[f"mixer.{k}"] = v
        if has_ffn:
            F = feed_forward_class(spec.feed_forward.kind)
            for k, v in F.param_specs(spec.feed_forward, hidden_size).items():
                out[f"ffn.{k}"] = v
        side = getattr(spec, "token_side", None)
        if side is not None:
            out["side.gate_proj.weight"] = ParamSpec((side.dim, hidden_size))
            out["side.proj.weight"] = ParamSpec((hidden_size, side.dim))
            out["side.norm.weight"] = ParamSpec((hidden_size,), "norm")
        return out

    @property
    def entry_norm(self):
        """The norm that feeds this block's first branch."""
        return self.pre_mixer_norm

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        """The mixer's fixed-size state alone, for a call that reads another call's keys and
        values and keeps state of its own in a cache entry of its own."""
        ask = getattr(self.mixer, "state_request", None)
        return ask() if ask is not None else None

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def sub(prefix):
            n = len(prefix) + 1
            return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
        for name in ("pre_mixer_norm", "pre_ffn_norm", "post_mixer_norm", "post_ffn_norm"):
            part = getattr(self, name)
            if part is not None:
                part.load(sub(name), device)
        self.mixer.load(sub("mixer"), dtype, device)
        if self.ffn is not None:
            self.ffn.load(sub("ffn"), dtype, device)
        if self.side is not None:
            t = sub("side")
            self.side_gate = Linear(t["gate_proj.weight"].to(device=device, dtype=dtype)
                                    .contiguous(), role="token_side_gate")
            self.side_proj = Linear(t["proj.weight"].to(device=device, dtype=dtype).contiguous(),
                                    role="token_side_proj")
            self.side_norm.load({"weight": t["norm.weight"]}, device)

    def _token_side(self, xs: torch.Tensor, ctx) -> torch.Tensor:
        """W_proj (gelu_tanh(W_gate xs) * e) for the stream xs [T, H] (rounded to the compute
        dtype) and the tokens' slices e of the shared table."""
        rows = getattr(ctx, "token_side_rows", None)
        if rows is None:
            raise ValueError("the layer takes a token input, but the model has no table for it")
        sd = self.side
        e = rows[:, sd.offset:sd.offset + sd.dim]
        z = self.side_gate(xs, out_dtype=torch.float32)
        g = ctx.new(xs.shape[0], sd.dim)
        kernels.gelu_mul_rows(z, e, g)
        return self.side_proj.partial(g)

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx, cache_entry: int,
                writes_cache: bool, next_norm) -> Optional[torch.Tensor]:
        """h: [T, H] 32-bit stream (updated in place); x = pre_mixer_norm(h)."""
        y = self.mixer.forward(x, ctx, cache_entry, writes_cache)
        post = self.post_mixer_norm
        if self.ffn is not None:
            x2 = ctx.new(*x.shape)
            _join(h, y, post, self.pre_ffn_norm, x2, self.mult)
            y = self.ffn.forward(x2, ctx)
            post = self.post_ffn_norm
        x3 = ctx.new(*x.shape) if next_norm is not None else None
        if self.side is None:
            _join(h, y, post, next_norm, x3, self.mult)
            return x3
        xs = ctx.new(*x.shape)
        _join(h, y, post, self.side_in, xs, self.mult)
        _join(h, self._token_side(xs, ctx), self.side_norm, next_norm, x3)
        return x3


register_block("sequential", Block)


def _join(h, y, post, nxt, x_out, mult: float = 1.0) -> None:
    """h += mult * post(y) (or mult * y when there is no post norm); x_out = nxt(h) if nxt."""
    if mult == 1.0:
        # (parts registered from outside may know nothing of a multiplier)
        if post is not None:
            post.residual(h, y, nxt, x_out)
        elif nxt is not None:
            nxt.after_residual(h, y, x_out)
        else:
            fused_residual(h, y, None, None, None)
    elif post is not None:
        post.residual(h, y, nxt, x_out, mult)
    elif nxt is not None:
        nxt.after_residual(h, y, x_out, mult)
    else:
        from .. import kernels
        kernels.layer_norm_join(h, y, None, None, None, None, None, mult=mult)
