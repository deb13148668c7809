"""Typed configuration of the Kadavik decoder, read from its own ``config.json`` keys.

A Kadavik model is a list of layers.  Each entry names its mixer (``type``: ``mlstm`` or
``attention``), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: a
dense one, a mixture of experts, or null for a layer without).  The top level gives the width,
the vocabulary, the embedding's multiplier (``embedding.scale``), the logits' multiplier
(``logit_scale``), the norms' eps (``norm.eps``) and the width of the per-layer token input
(``token_side.dim``; absent: the layers take none).  Every size and every constant that can
differ between two models of the design is read from there.

What the design fixes, and what therefore stands in the lowering below: RMS norms with plain
weights before and after both branches of a layer; after the feed-forward every layer takes an
input from the token itself (a slice of a table the layers share, gated by a projection of the
stream, projected back and RMS-normed); ``mlstm`` is the matrix memory with exponential gates,
capped gate logits, a running maximum that starts at 0 and 1e-6 in the read-out's denominator;
``attention`` projects q, k and v without biases, runs a short causal convolution over time on
each of their channels, rotates the first ``rot.dims`` dimensions of every head in split halves
with frequencies scaled in three bands of wavelength, sees a sliding window of ``mask.size``
keys and, behind it, the sequence's first ``mask.keep_first`` ones, and gates the concatenated
heads with a sigmoid of a projection of its input; a layer with ``kv_from`` attends to another
layer's keys and values with queries of its own; the dense feed-forward is gated with the tanh
GELU; experts are gated with silu, chosen by softmax scores plus a correction, weighted by
their renormalised scores times ``router.scale``, the last ``router.identity`` router outputs
being identity experts, beside a shared expert times a sigmoid gate per token; the head is the
embedding.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import (AttentionSpec, BandScalingSpec, BlockSpec, ConfigError, GatedFeedForwardSpec,
                   LayerCall, MatrixMemorySpec, ModelSpec, NormSpec, RotarySpec,
                   RoutedFeedForwardSpec, TokenSideSpec)

MIXERS = ("mlstm", "attention")
DEN_EPS = 1e-6                   # in the matrix memory's read-out denominator


def _get(d: Any, key: str, where: str, typ=int):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                return int(v)
            raise ConfigError(f"config.json: '{where}{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
        return float(v)
    return v


@dataclass(frozen=True)
class KadavikRotation:
    dims: int
    base: float
    # (factor, low, high, original) of the scaling by bands of wavelength; None: unscaled
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class KadavikMixer:
    """One record for both kinds; the fields a kind does not have stay at their zero."""
    kind: str
    heads: int
    dim: int
    vdim: int
    # mlstm
    gate_cap: float = 0.0
    # attention
    kv_heads: int = 0
    scale: float = 0.0
    conv: int = 0                         # taps of the convolution on q, k, v (0: none)
    window: Optional[int] = None          # mask.size; None: every earlier key is seen
    keep_first: int = 0
    rot: Optional[KadavikRotation] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class KadavikFeedForward:
    kind: str                             # "dense" or "moe"
    ff: int                               # width of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    identity: int = 0
    route_scale: float = 1.0
    shared_ff: int = 0                    # 0: no shared expert


@dataclass(frozen=True)
class KadavikLayer:
    mixer: KadavikMixer
    mlp: Optional[KadavikFeedForward]


def _read_mixer(kind: str, m: dict, where: str) -> KadavikMixer:
    common = dict(kind=kind, heads=_get(m, "heads", where), dim=_get(m, "dim", where),
                  vdim=_get(m, "vdim", where))
    if kind == "mlstm":
        return KadavikMixer(gate_cap=_get(m, "gate_cap", where, float), **common)
    rot = None
    if m.get("rot") is not None:
        r = m["rot"]
        sc = None
        if r.get("scaling") is not None:
            w = where + "rot.scaling."
            sc = tuple(_get(r["scaling"], k, w, float)
                       for k in ("factor", "low", "high", "original"))
        rot = KadavikRotation(dims=_get(r, "dims", where + "rot."),
                              base=_get(r, "base", where + "rot.", float), scaling=sc)
    mask = m.get("mask")
    return KadavikMixer(
        kv_heads=_get(m, "kv_heads", where) if m.get("kv_heads") is not None else common["heads"],
        scale=_get(m, "scale", where, float),
        conv=_get(m, "conv", where) if m.get("conv") is not None else 0,
        window=_get(mask, "size", where + "mask.") if mask is not None else None,
        keep_first=(_get(mask, "keep_first", where + "mask.")
                    if mask is not None and mask.get("keep_first") is not None else 0),
        rot=rot, kv_from=_get(m, "kv_from", where) if m.get("kv_from") is not None else None,
        **common)


def _read_mlp(f: dict, where: str) -> KadavikFeedForward:
    kind = _get(f, "kind", where, typ=None)
    if kind == "dense":
        return KadavikFeedForward("dense", _get(f, "ff", where))
    if kind == "moe":
        router = _get(f, "router", where, typ=None)
        shared = f.get("shared")
        w = where + "router."
        return KadavikFeedForward(
            "moe", _get(_get(f, "expert", where, typ=None), "ff", where + "expert."),
            experts=_get(router, "experts", w), top=_get(router, "top", w),
            identity=_get(router, "identity", w) if router.get("identity") is not None else 0,
            route_scale=_get(router, "scale", w, float) if router.get("scale") is not None else 1.0,
            shared_ff=_get(shared, "ff", where + "shared.") if shared is not None else 0)
    raise ConfigError(f"config.json: '{where}kind' = {kind!r} is not a feed-forward of this "
                      "design (known: dense, moe)")


@dataclass(frozen=True)
class KadavikConfig:
    vocab: int
    width: int
    embed_scale: float
    logit_scale: float
    norm_eps: float
    side_dim: int                         # 0: no per-layer token input
    layers: Tuple[KadavikLayer, ...]
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Kadavik"

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KadavikConfig":
        layers_raw = _get(raw, "layers", "", typ=None)
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where, typ=None)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not a mixer of this "
                                  f"design (known: {', '.join(MIXERS)})")
            mixer = _read_mixer(kind, _get(entry, "mixer", where, typ=None), where + "mixer.")
            mlp = None                     # (no 'mlp' key reads as null: no feed-forward)
            if entry.get("mlp") is not None:
                mlp = _read_mlp(entry["mlp"], where + "mlp.")
            layers.append(KadavikLayer(mixer, mlp))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in eos) if isinstance(eos, list) \
            else (int(eos),)
        bos = raw.get("bos_token_id")
        emb, side = raw.get("embedding"), raw.get("token_side")
        cfg = cls(vocab=_get(raw, "vocab", ""), width=_get(raw, "width", ""),
                  embed_scale=(_get(emb, "scale", "embedding.", float)
                               if emb is not None and emb.get("scale") is not None else 1.0),
                  logit_scale=(_get(raw, "logit_scale", "", float)
                               if raw.get("logit_scale") is not None else 1.0),
                  norm_eps=_get(_get(raw, "norm", "", typ=None), "eps", "norm.", float),
                  side_dim=_get(side, "dim", "token_side.") if side is not None else 0,
                  layers=tuple(layers), bos_token_id=None if bos is None else int(bos),
                  eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        if self.side_dim < 0:
            raise ConfigError("config.json: 'token_side.dim' must be positive")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer."
            for k in ("heads", "dim", "vdim"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"config.json: '{where}{k}' must be positive")
            if m.kind == "mlstm":
                if m.gate_cap <= 0:
                    raise ConfigError(f"config.json: '{where}gate_cap' must be positive")
            else:
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: '{where}heads' ({m.heads}) must be a "
                                      f"multiple of 'kv_heads' ({m.kv_heads})")
                if m.scale <= 0:
                    raise ConfigError(f"config.json: '{where}scale' must be positive")
                if m.conv < 0:
                    raise ConfigError(f"config.json: '{where}conv' cannot be negative")
                if m.window is not None and m.window <= 0:
                    raise ConfigError(f"config.json: '{where}mask.size' must be positive")
                if m.keep_first < 0:
                    raise ConfigError(f"config.json: '{where}mask.keep_first' cannot be negative")
                if m.rot is not None:
                    if m.rot.dims <= 0 or m.rot.dims % 2 or m.rot.dims > m.dim:
                        raise ConfigError(f"config.json: '{where}rot.dims' ({m.rot.dims}) must be "
                                          f"even and at most 'dim' ({m.dim})")
                    if m.rot.base <= 0:
                        raise ConfigError(f"config.json: '{where}rot.base' must be positive")
                    if m.rot.scaling is not None:
                        factor, low, high, original = m.rot.scaling
                        if factor <= 0 or original <= 0 or low <= 0 or high <= low:
                            raise ConfigError(f"config.json: '{where}rot.scaling' needs positive "
                                              "'factor' and 'original' and 0 < 'low' < 'high'")
                if m.kv_from is not None:
                    j = m.kv_from
                    if not 0 <= j < len(self.layers) or j >= i:
                        raise ConfigError(f"config.json: '{where}kv_from' = {j} must name an "
                                          "earlier layer")
                    src = self.layers[j].mixer
                    if src.kind != "attention" or src.kv_from is not None:
                        raise ConfigError(f"config.json: '{where}kv_from' = {j}: that layer has "
                                          "no keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim) or \
                            src.rot != m.rot:
                        raise ConfigError(f"config.json: '{where}kv_from' = {j}: kv_heads, dim, "
                                          "vdim and rot must equal that layer's")
            f = layer.mlp
            if f is not None:
                where = f"layers[{i}].mlp."
                if f.ff <= 0 or f.shared_ff < 0:
                    raise ConfigError(f"config.json: the sizes under '{where}' must be positive")
                if f.kind == "moe":
                    if f.experts < 0 or f.identity < 0 or f.experts + f.identity < 1:
                        raise ConfigError(f"config.json: '{where}router.experts' and 'identity' "
                                          "must not be negative and not both zero")
                    if not 0 < f.top <= f.experts + f.identity:
                        raise ConfigError(f"config.json: '{where}router.top' ({f.top}) must be "
                                          f"between 1 and the router's {f.experts + f.identity} "
                                          "outputs")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer: Dict[str, Any] = {"dim": m.dim, "heads": m.heads, "vdim": m.vdim}
            if m.kind == "mlstm":
                mixer["gate_cap"] = m.gate_cap
            else:
                mixer.update(kv_heads=m.kv_heads, scale=m.scale)
                if m.conv:
                    mixer["conv"] = m.conv
                if m.window is not None:
                    mixer["mask"] = {"keep_first": m.keep_first, "size": m.window}
                if m.rot is not None:
                    rot: Dict[str, Any] = {"base": m.rot.base, "dims": m.rot.dims}
                    if m.rot.scaling is not None:
                        rot["scaling"] = dict(zip(("factor", "low", "high", "original"),
                                                  m.rot.scaling))
                    mixer["rot"] = rot
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"ff": f.ff, "kind": "dense"}
            else:
                mlp = {"expert": {"ff": f.ff}, "kind": "moe",
                       "router": {"experts": f.experts, "identity": f.identity,
                                  "scale": f.route_scale, "top": f.top}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"mixer": mixer, "mlp": mlp, "type": m.kind})
        d: Dict[str, Any] = {"architecture": self.architecture,
                             "embedding": {"scale": self.embed_scale}, "layers": layers,
                             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                             "vocab": self.vocab, "width": self.width}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------------------------- lower
    def _mixer_spec(self, i: int):
        m = self.layers[i].mixer
        if m.kind == "mlstm":
            return MatrixMemorySpec(n_heads=m.heads, head_dim=m.dim, value_dim=m.vdim,
                                    gate_cap=m.gate_cap, eps=self.norm_eps, den_eps=DEN_EPS)
        position = None
        if m.rot is not None:
            sc = None
            if m.rot.scaling is not None:
                factor, low, high, original = m.rot.scaling
                sc = BandScalingSpec(factor=factor, original=original, low=low, high=high)
            position = RotarySpec(theta=m.rot.base, factor=1.0,
                                  rotary_dim=0 if m.rot.dims == m.dim else m.rot.dims, scaling=sc)
        # the layers that borrow this one's keys and values may look further back than it does
        readers = [l.mixer for l in self.layers if l.mixer.kv_from == i]
        wider = any((r.window, r.keep_first if r.window is not None else 0) !=
                    (m.window, m.keep_first if m.window is not None else 0) for r in readers)
        return AttentionSpec(
            n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
            window=m.window, qk_norm=None, position=position, keep_all_keys=wider,
            value_dim=0 if m.vdim == m.dim else m.vdim, own_kv=m.kv_from is None,
            keep_first=m.keep_first if m.window is not None else 0,
            # (a layer of this design always runs the row kernel of the convolution: one tap
            # of weight one is no convolution)
            conv_taps=m.conv, out_gate=True)

    def _ffn_spec(self, i: int):
        f = self.layers[i].mlp
        if f is None:
            return None
        if f.kind == "dense":
            return GatedFeedForwardSpec(intermediate_size=f.ff, activation="gelu_tanh")
        return RoutedFeedForwardSpec(
            n_experts=f.experts, top=f.top, intermediate_size=f.ff, activation="silu",
            n_groups=1, keep_groups=1, correction=True, weighting="softmax_all",
            route_scale=f.route_scale, n_identity=f.identity, shared_size=f.shared_ff)

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(eps=self.norm_eps, zero_centered=False)
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            side = None
            if self.side_dim:
                side = TokenSideSpec(dim=self.side_dim, offset=i * self.side_dim,
                                     eps=self.norm_eps)
            blocks.append(BlockSpec(mixer=self._mixer_spec(i), feed_forward=self._ffn_spec(i),
                                    norm=norm, arrangement="sandwich", token_side=side))
            src = layer.mixer.kv_from
            # a layer without keys and values of its own reads the entry its source writes and
            # keeps the state of its own convolution in the entry of its own number
            schedule.append(LayerCall(block=i, cache=i if src is None else src,
                                      writes_cache=src is None,
                                      state=None if src is None else i))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, embed_scale=self.embed_scale,
            blocks=tuple(blocks), schedule=tuple(schedule), final_norm=norm,
            tie_embeddings=True, max_positions=0, bos_token_id=self.bos_token_id,
            eos_token_ids=self.eos_token_ids, logit_scale=self.logit_scale,
            token_side_width=self.side_dim * len(self.layers))
