"""A plain, slow Bovozen decoder for comparison: whole sequences, no cache, no state kept.

One function per mechanism, each written from the design's equations.  Nothing here is
imported by, or imports, the library under test: the configuration is a dictionary and the
weights a dictionary of tensors under their checkpoint names.

Arithmetic runs in the dtype of the tensors handed in (float64 by default).

Notation: W are matrices stored [out, in]; t, j are positions; a is a head.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


# --------------------------------------------------------------------- inputs
def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    out = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            for k, v in load_file(os.path.join(folder, name)).items():
                out[k] = v.to(dtype) if v.is_floating_point() else v
    return out


# ---------------------------------------------------------------------- norms
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The layers' norm: the weight is stored as its difference from one."""
    return rms(x, eps) * (1.0 + w)


def unit(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


# ----------------------------------------------------------------- attention
def head_slopes(heads: int) -> torch.Tensor:
    """slope_a = 2^(-8 (a + 1) / heads), a = 0 .. heads - 1."""
    a = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -8.0 * a / heads)


def visible(T: int, block: Optional[int]) -> torch.Tensor:
    """[T, T] true where query t sees key j: j <= t, and with blocks of ``block`` positions
    counted from 0 also t // block == j // block."""
    t = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= t
    if block is not None:
        see = see & (torch.div(t, block, rounding_mode="floor")
                     == torch.div(j, block, rounding_mode="floor"))
    return see


def biased_softmax_attention(q, k, v, scale: float, block: Optional[int]) -> torch.Tensor:
    """q [T, A, d], k [T, G, d], v [T, G, dv] -> [T, A, dv].

    weight(t, j) = softmax_j(scale q_t . k_j - slope_a (t - j)) over the visible j."""
    T, A, _ = q.shape
    G = k.shape[1]
    see = visible(T, block)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(q.dtype)
    slopes = head_slopes(A).to(q.dtype)
    out = torch.zeros(T, A, v.shape[2], dtype=q.dtype)
    for a in range(A):
        g = a // (A // G)
        s = (q[:, a] @ k[:, g].T) * scale - slopes[a] * dist
        s = s.masked_fill(~see, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def lean_values(v, v_first, lam):
    """(1 - lam) v + lam v_first."""
    return (1.0 - lam) * v + lam * v_first


def attention_mixer(h, W, p, m, eps, shared: dict) -> torch.Tensor:
    """``shared`` carries the first v_mix layer's values through the layers of one pass."""
    T = h.shape[0]
    A, d, dv = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads") or A
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    q = rms(q, eps) * W[p + "q.norm"]           # over all heads' rows at once
    k = rms(k, eps) * W[p + "k.norm"]
    if m.get("v_mix"):
        if "first" in shared:
            v = lean_values(v, shared["first"], W[p + "vmix"])
        else:
            shared["first"] = v
    block = m["mask"]["size"] if m.get("mask") else None
    o = biased_softmax_attention(q.view(T, A, d), k.view(T, G, d), v.view(T, G, dv),
                                 float(m["scale"]), block)
    return o.reshape(T, A * dv) @ W[p + "o"].T


# ---------------------------------------------------------------- delta rule
def causal_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps] (last column: the current token).  y_t = sum_i w[:, taps-1-i]
    x_{t-i}, zeros before the start; then y * sigmoid(y)."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for i in range(taps):
            if t - i >= 0:
                y[t] += w[:, taps - 1 - i] * x[t - i]
    return y * torch.sigmoid(y)


def channel_decay(low, W_up, dt_bias, A_log, A: int, d: int) -> torch.Tensor:
    """[T, A, d]: exp(-exp(A_log_a) * softplus(W_up low + dt_bias))."""
    pre = low @ W_up.T + dt_bias
    sp = torch.nn.functional.softplus(pre, threshold=1e9)
    return torch.exp(-torch.exp(A_log)[None, :, None] * sp.view(-1, A, d))


def delta_recurrence(q, k, v, beta, decay, S0=None):
    """q, k [T, G, d]; v [T, A, dv]; beta [T, A]; decay [T, A, d] -> (o [T, A, dv], S).

    Per head:  S <- decay * S (row by row);  u = beta (v - S^T k);  S <- S + k u^T;
    o = S^T q."""
    T, A, dv = v.shape
    G, d = k.shape[1], k.shape[2]
    S = torch.zeros(A, d, dv, dtype=v.dtype) if S0 is None else S0.clone()
    o = torch.zeros(T, A, dv, dtype=v.dtype)
    for a in range(A):
        g = a // (A // G)
        for t in range(T):
            S[a] = decay[t, a][:, None] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, g])
            S[a] = S[a] + torch.outer(k[t, g], u)
            o[t, a] = S[a].T @ q[t, g]
    return o, S


def delta_mixer(h, W, p, m, eps) -> torch.Tensor:
    T = h.shape[0]
    A, d, dv = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads") or A
    q = causal_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, A, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    decay = channel_decay(h @ W[p + "a1"].T, W[p + "a2"], W[p + "dt_bias"], W[p + "A_log"], A, d)
    o, _ = delta_recurrence(q, k, v, beta, decay)
    o = rms(o, eps) * W[p + "norm"]
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, A, dv)
    return (o * gate).reshape(T, A * dv) @ W[p + "o"].T


# -------------------------------------------------------------- feed-forward
def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def gated_expert(h, W, p):
    z = h @ W[p + "gate"].T
    return ((z * torch.sigmoid(z)) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W_router, bias, top: int):
    """(ids [T, top], weights [T, top]): the largest biased logits choose; the weights are
    the softmax over the chosen logits alone."""
    z = h @ W_router.T + bias
    val, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(val, dim=-1)


def routed_ff(h, W, p, f):
    ids, wts = route(h, W[p + "router"], W[p + "router.b"], int(f["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(ids.shape[1]):
            out[t] += wts[t, c] * gated_expert(h[t:t + 1], W, f"{p}e{int(ids[t, c])}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * gated_expert(h, W, p + "shared.")
    return out


# --------------------------------------------------------------------- model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int],
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; ``streams`` collects the residual
    stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens)] + W["pos"][:T]
    shared: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_around_zero(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, W, p + "mix.", layer["mixer"], eps, shared)
        elif layer["type"] == "channel_delta":
            x = x + delta_mixer(h, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            h = norm_around_zero(x, W[p + "norm2"], eps)
            x = x + (dense_ff(h, W, p + "mlp.") if f["kind"] == "dense"
                     else routed_ff(h, W, p + "mlp.", f))
        if streams is not None:
            streams.append(x.clone())
    return norm_around_zero(x, W["final.norm"], eps) @ W["embed"].T
