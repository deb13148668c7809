"""Kadavik, written out plainly: one function per mechanism, 64-bit, token by token where the
design is a recurrence.  Nothing here is shared with the library; the tests compare the two.

``cfg`` is the parsed ``config.json`` of a model; ``w`` maps checkpoint names to tensors.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    """x over the root of its mean square, eps under the root, along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


# ------------------------------------------------------------------ positions
def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high = scaling["factor"], scaling["low"], scaling["high"]
            original = scaling["original"]
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x, positions, rot: dict):
    """x [T, heads, dim]: the first rot.dims dimensions of every head turn, pair (i, i + dims/2)."""
    dims = rot["dims"]
    half = dims // 2
    f = torch.tensor(scaled_frequencies(dims, rot["base"], rot.get("scaling")), dtype=F)
    a = positions.to(F)[:, None] * f[None, :]                 # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ convolution
def causal_conv(u, weight):
    """u [T, C], weight [C, taps]: y_t = sum_j weight[:, j] * u_(t - taps + 1 + j), zeros before
    the sequence's first token."""
    T, C = u.shape
    taps = weight.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += weight[:, j] * u[src]
    return y


# ------------------------------------------------------------------ attention
def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def attention_keys_values(h, m: dict, w: Dict[str, torch.Tensor], p: str):
    """(keys as a cache would hold them [T, G, dim], values [T, G, vdim]) of the layer whose
    tensors start with ``p``."""
    T = h.shape[0]
    G = m.get("kv_heads", m["heads"])
    k = causal_conv(h @ w[p + "k"].to(F).T, w[p + "k.conv"].to(F)) if m.get("conv") else \
        h @ w[p + "k"].to(F).T
    v = causal_conv(h @ w[p + "v"].to(F).T, w[p + "v.conv"].to(F)) if m.get("conv") else \
        h @ w[p + "v"].to(F).T
    k = k.view(T, G, m["dim"])
    if m.get("rot") is not None:
        k = rotate(k, torch.arange(T), m["rot"])
    return k, v.view(T, G, m["vdim"])


def attention_mixer(h, m: dict, w: Dict[str, torch.Tensor], p: str, k, v):
    """h [T, width] of one sequence from position 0; k, v: this layer's own or another's."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = h @ w[p + "q"].to(F).T
    if m.get("conv"):
        q = causal_conv(q, w[p + "q.conv"].to(F))
    q = q.view(T, H, d)
    if m.get("rot") is not None:
        q = rotate(q, torch.arange(T), m["rot"])
    mask = m.get("mask")
    size = mask["size"] if mask is not None else None
    keep = (mask.get("keep_first") or 0) if mask is not None else 0
    see = torch.tensor([[visible(i, j, size, keep) for j in range(T)] for i in range(T)])
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = torch.where(see, s, torch.full_like(s, -math.inf))
        out[:, a] = torch.softmax(s, -1) @ v[:, g]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].to(F).T)
    return out @ w[p + "o"].to(F).T


# ------------------------------------------------------------------ matrix memory
def mlstm_mixer(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """The matrix memory with a running maximum that starts at 0, token by token."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].to(F).T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].to(F).T).view(T, H, d)
    v = (h @ w[p + "v"].to(F).T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].to(F).T + w[p + "i.b"].to(F)) / cap)
    gf = torch.nn.functional.logsigmoid(
        cap * torch.tanh((h @ w[p + "f"].to(F).T + w[p + "f.b"].to(F)) / cap))
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F)
        n = torch.zeros(d, dtype=F)
        mx = 0.0
        for t in range(T):
            i_t, f_t = float(gi[t, a]), float(gf[t, a])
            m_new = max(f_t + mx, i_t)
            S = math.exp(f_t + mx - m_new) * S + math.exp(i_t - m_new) * torch.outer(k[t, a], v[t, a])
            n = math.exp(f_t + mx - m_new) * n + math.exp(i_t - m_new) * k[t, a]
            mx = m_new
            den = max(abs(float((n * q[t, a]).sum())), math.exp(-mx)) + 1e-6
            out[t, a] = (S.T @ q[t, a]) / den
    out = rms(out, eps).reshape(T, H * dv) * w[p + "norm"].to(F)
    out = out * torch.sigmoid(h @ w[p + "g"].to(F).T)
    return out @ w[p + "o"].to(F).T


# ------------------------------------------------------------------ feed-forwards
def gated(h, w, p: str, act):
    return (act(h @ w[p + "gate"].to(F).T) * (h @ w[p + "up"].to(F).T)) @ w[p + "down"].to(F).T


def route(h, f: dict, w, p: str):
    """(chosen [T, top], weights [T, top]); indices at or beyond ``experts`` are identities."""
    r = f["router"]
    s = torch.softmax(h @ w[p + "router"].to(F).T, -1)
    choice = s + w[p + "correction"].to(F)
    idx = torch.topk(choice, r["top"], dim=-1).indices
    sc = torch.gather(s, 1, idx)
    return idx, sc / (sc.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def moe(h, f: dict, w, p: str, chosen=None):
    r = f["router"]
    idx, wt = route(h, f, w, p)
    if chosen is not None:                 # experts fixed from outside, weights from the scores
        idx = chosen
        s = torch.softmax(h @ w[p + "router"].to(F).T, -1)
        sc = torch.gather(s, 1, idx)
        wt = sc / (sc.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[t, c])
            if e >= r["experts"]:
                y[t] += wt[t, c] * h[t]
            else:
                y[t] += wt[t, c] * gated(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if f.get("shared") is not None:
        y = y + torch.sigmoid(h @ w[p + "shared.sg"].to(F).T) * gated(h, w, p + "shared.", silu)
    return y


def side_input(x, tokens, layer: int, cfg: dict, w):
    dim = cfg["token_side"]["dim"]
    eps = cfg["norm"]["eps"]
    p = f"l{layer}.side."
    e = w["side.embed"].to(F)[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].to(F).T) * e) @ w[p + "proj"].to(F).T
    return x + rms(y, eps) * w[p + "norm"].to(F)


# ------------------------------------------------------------------ the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, chosen=None, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives
    the stream after every layer.  ``chosen``: {layer: [T, top]} experts to use instead of the
    router's own choice."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F)[tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    kv = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"].to(F), eps)
        if layer["type"] == "mlstm":
            y = mlstm_mixer(h, m, w, p + "mix.", eps)
        else:
            src = m.get("kv_from")
            if src is None:
                kv[i] = attention_keys_values(h, m, w, p + "mix.")
                src = i
            y = attention_mixer(h, m, w, p + "mix.", *kv[src])
        x = x + rms_norm(y, w[p + "norm1b"].to(F), eps)
        f = layer.get("mlp")
        if f is not None:
            h = rms_norm(x, w[p + "norm2"].to(F), eps)
            if f["kind"] == "dense":
                y = gated(h, w, p + "mlp.", gelu_tanh)
            else:
                y = moe(h, f, w, p + "mlp.", None if chosen is None else chosen.get(i))
            x = x + rms_norm(y, w[p + "norm2b"].to(F), eps)
        if cfg.get("token_side") is not None:
            x = side_input(x, tokens, i, cfg, w)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, w["final.norm"].to(F), eps)
    return x @ w["embed"].to(F).T * cfg.get("logit_scale", 1.0)
