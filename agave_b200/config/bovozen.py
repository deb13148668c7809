"""Typed configuration of the Bovozen decoder, read from its own ``config.json`` keys.

A Bovozen model is a list of layers.  Each entry names its mixer (``type``: ``attention`` or
``channel_delta``), the mixer's sizes and constants (``mixer``) and its feed-forward
(``mlp``: a dense one, a mixture of experts, or null for a layer without).  The top level
gives the width, the vocabulary, the number of learned position vectors and the norms' eps.
Every size and every constant that can differ between two models of the design is read from
there; the widths of the recurrent mixer's two bottlenecks, which config.json does not state,
come from the shapes of their tensors.

What the design fixes, and what therefore stands in the lowering below: a learned vector per
position joins the embedding, unscaled; a layer is pre-norm with RMS norms whose weights are
stored around zero; ``attention`` norms q and k over the whole projection with plain weights,
does not rotate, takes slope_a * distance off the scaled score with slope_a =
2 ** (-8 (a + 1) / heads), sees only the keys of its own block of ``mask.size`` positions
(counted from position 0) where a mask is given, and, where ``v_mix`` is set, leans its
values towards those of the first such layer; ``channel_delta`` is the gated delta rule with
a decay per key channel, unit q and k with eps 1e-6 and q times dim ** -0.5; the dense
feed-forward's activation is the erf GELU; experts are gated with silu, chosen by their
biased logits and weighted by the softmax over the chosen logits, beside a shared expert
times a sigmoid gate per token; the head is the embedding.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import (AttentionSpec, BlockSpec, ChannelDeltaSpec, ConfigError, DenseFeedForwardSpec,
                   DistanceSlopeSpec, LayerCall, LearnedPositionSpec, ModelSpec, NormSpec,
                   RoutedFeedForwardSpec, ValueMixSpec)

MIXERS = ("attention", "channel_delta")
SLOPE_EXPONENT = 8.0
UNIT_EPS = 1e-6


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
class BovozenMixer:
    """One record for both kinds; the fields a kind does not have stay at their zero."""
    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    # attention
    scale: float = 0.0
    chunk: Optional[int] = None        # mask.size; None: every earlier key is seen
    v_mix: bool = False
    # channel_delta
    conv: int = 0
    decay_rank: int = 0
    gate_rank: int = 0


@dataclass(frozen=True)
class BovozenFeedForward:
    kind: str                          # "dense" or "moe"
    ff: int                            # width of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0                 # 0: no shared expert


@dataclass(frozen=True)
class BovozenLayer:
    mixer: BovozenMixer
    mlp: Optional[BovozenFeedForward]


def _read_mixer(kind: str, m: dict, where: str, layer: int, shapes) -> BovozenMixer:
    heads = _get(m, "heads", where)
    common = dict(kind=kind, heads=heads, dim=_get(m, "dim", where), vdim=_get(m, "vdim", where),
                  kv_heads=_get(m, "kv_heads", where) if m.get("kv_heads") is not None else heads)
    if kind == "attention":
        mask = m.get("mask")
        return BovozenMixer(scale=_get(m, "scale", where, float),
                            chunk=_get(mask, "size", where + "mask.") if mask is not None else None,
                            v_mix=bool(m.get("v_mix", False)), **common)
    ranks = {}
    for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
        if m.get(key) is not None:
            ranks[key] = _get(m, key, where)
        else:
            shp = shapes(f"l{layer}.mix.{tensor}") if shapes is not None else None
            ranks[key] = int(shp[0]) if shp is not None else 0
    return BovozenMixer(conv=_get(m, "conv", where), **ranks, **common)


def _read_mlp(f: dict, where: str) -> BovozenFeedForward:
    kind = _get(f, "kind", where, typ=None)
    if kind == "dense":
        return BovozenFeedForward("dense", _get(f, "ff", where))
    if kind == "moe":
        router = _get(f, "router", where, typ=None)
        shared = f.get("shared")
        return BovozenFeedForward(
            "moe", _get(_get(f, "expert", where, typ=None), "ff", where + "expert."),
            experts=_get(router, "experts", where + "router."),
            top=_get(router, "top", where + "router."),
            shared_ff=_get(shared, "ff", where + "shared.") if shared is not None else 0)
    raise ConfigError(f"config.json: '{where}kind' = {kind!r} is not a feed-forward of this "
                      "design (known: dense, moe)")


@dataclass(frozen=True)
class BovozenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[BovozenLayer, ...]
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Bovozen"

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], shapes=None) -> "BovozenConfig":
        """``shapes(name)`` gives a stored tensor's shape (or None): the widths of the
        recurrent mixer's bottlenecks come from there.  A raw dictionary may carry them itself
        as ``mixer.decay_rank`` and ``mixer.gate_rank`` (what ``to_dict`` writes)."""
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
            mixer = _read_mixer(kind, _get(entry, "mixer", where, typ=None), where + "mixer.", i,
                                shapes)
            mlp = None                     # (no 'mlp' key reads as null: no feed-forward)
            if entry.get("mlp") is not None:
                mlp = _read_mlp(entry["mlp"], where + "mlp.")
            layers.append(BovozenLayer(mixer, mlp))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in eos) if isinstance(eos, list) \
            else (int(eos),)
        bos = raw.get("bos_token_id")
        if raw.get("max_positions") is None and shapes is not None and shapes("pos") is not None:
            positions = int(shapes("pos")[0])          # as many as the table has rows
        else:
            positions = _get(raw, "max_positions", "")
        cfg = cls(vocab=_get(raw, "vocab", ""), width=_get(raw, "width", ""),
                  max_positions=positions,
                  norm_eps=_get(_get(raw, "norm", "", typ=None), "eps", "norm.", float),
                  layers=tuple(layers), bos_token_id=None if bos is None else int(bos),
                  eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0:
            raise ConfigError("config.json: 'vocab', 'width' and 'max_positions' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        first_mix = None
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer."
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"config.json: '{where}{k}' must be positive")
            if m.heads % m.kv_heads:
                raise ConfigError(f"config.json: '{where}heads' ({m.heads}) must be a multiple of "
                                  f"'kv_heads' ({m.kv_heads})")
            if m.kind == "attention":
                if m.scale <= 0:
                    raise ConfigError(f"config.json: '{where}scale' must be positive")
                if m.chunk is not None and m.chunk <= 0:
                    raise ConfigError(f"config.json: '{where}mask.size' must be positive")
                if m.v_mix:
                    if first_mix is None:
                        first_mix = i
                    else:
                        src = self.layers[first_mix].mixer
                        if (src.kv_heads, src.vdim) != (m.kv_heads, m.vdim):
                            raise ConfigError(f"config.json: '{where}v_mix': kv_heads and vdim "
                                              f"must equal those of layers[{first_mix}], whose "
                                              "values are mixed in")
            else:
                if m.conv <= 0:
                    raise ConfigError(f"config.json: '{where}conv' must be positive")
                if m.decay_rank <= 0 or m.gate_rank <= 0:
                    raise ConfigError(f"layers[{i}]: the widths of the decay's and the gate's "
                                      f"bottlenecks are unknown (no tensors 'l{i}.mix.a1', "
                                      f"'l{i}.mix.g1' and no '{where}decay_rank', "
                                      f"'{where}gate_rank')")
            f = layer.mlp
            if f is not None:
                where = f"layers[{i}].mlp."
                if f.ff <= 0 or f.shared_ff < 0:
                    raise ConfigError(f"config.json: the sizes under '{where}' must be positive")
                if f.kind == "moe" and not 0 < f.top <= f.experts:
                    raise ConfigError(f"config.json: '{where}router.top' ({f.top}) must be "
                                      f"between 1 and 'experts' ({f.experts})")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer: Dict[str, Any] = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads,
                                     "vdim": m.vdim}
            if m.kind == "attention":
                mixer.update(scale=m.scale, v_mix=m.v_mix)
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
            else:
                mixer.update(conv=m.conv, decay_rank=m.decay_rank, gate_rank=m.gate_rank)
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"ff": f.ff, "kind": "dense"}
            else:
                mlp = {"expert": {"ff": f.ff}, "kind": "moe",
                       "router": {"experts": f.experts, "top": f.top}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"mixer": mixer, "mlp": mlp, "type": m.kind})
        d: Dict[str, Any] = {"architecture": self.architecture, "layers": layers,
                             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                             "vocab": self.vocab, "width": self.width}
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------------------------- lower
    def first_mixed(self) -> Optional[int]:
        """The first layer whose values the other ``v_mix`` layers lean towards."""
        for i, layer in enumerate(self.layers):
            if layer.mixer.kind == "attention" and layer.mixer.v_mix:
                return i
        return None

    def _mixer_spec(self, i: int):
        m = self.layers[i].mixer
        if m.kind == "attention":
            first = self.first_mixed()
            mix = None
            if m.v_mix:
                mix = ValueMixSpec(source=None if i == first else first)
            return AttentionSpec(
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                window=None, qk_norm=NormSpec(eps=self.norm_eps, zero_centered=False),
                qk_norm_whole=True, position=None,
                value_dim=0 if m.vdim == m.dim else m.vdim, chunk=m.chunk,
                distance_slope=DistanceSlopeSpec(exponent=SLOPE_EXPONENT,
                                                 reach=self.max_positions),
                value_mix=mix)
        return ChannelDeltaSpec(
            n_heads=m.heads, n_qk_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
            conv_taps=m.conv, decay_rank=m.decay_rank, gate_rank=m.gate_rank, eps=self.norm_eps,
            unit_eps=UNIT_EPS)

    def _ffn_spec(self, i: int):
        f = self.layers[i].mlp
        if f is None:
            return None
        if f.kind == "dense":
            return DenseFeedForwardSpec(intermediate_size=f.ff, activation="gelu_erf")
        return RoutedFeedForwardSpec(
            n_experts=f.experts, top=f.top, intermediate_size=f.ff, activation="silu",
            n_groups=1, keep_groups=1, correction=False, router_bias=True,
            weighting="softmax_top", shared_size=f.shared_ff)

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(eps=self.norm_eps, zero_centered=True)
        blocks = tuple(BlockSpec(mixer=self._mixer_spec(i), feed_forward=self._ffn_spec(i),
                                 norm=norm, arrangement="pre")
                       for i in range(len(self.layers)))
        schedule = tuple(LayerCall(block=i, cache=i, writes_cache=True)
                         for i in range(len(self.layers)))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, embed_scale=1.0, blocks=blocks,
            schedule=schedule, final_norm=norm, tie_embeddings=True,
            max_positions=self.max_positions, bos_token_id=self.bos_token_id,
            eos_token_ids=self.eos_token_ids,
            stream_position=LearnedPositionSpec(positions=self.max_positions, scale=1.0))
