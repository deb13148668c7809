"""Bovozen: the registry entry and the names of its tensors.

The layer structure is data (``BovozenConfig.to_model_spec``): attention over blocks of
positions with a linear bias by distance, a norm over the whole q and k projections and values
that lean towards an earlier layer's; a recurrent mixer (the gated delta rule with a decay per
key channel); a dense erf-GELU feed-forward or routed experts beside a gated shared one; RMS
norms before every branch; learned position vectors; a head tied to the embedding.  What is
left to say here is how the generic decoder's tensor names map to a checkpoint's: ``embed``,
``pos``, ``final.norm`` and per layer ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*`` and
``l<i>.mlp.*`` (experts ``e<j>.{gate,up,down}``, ``router`` and its bias ``router.b``,
``shared.{gate,up,down,sg}``; a convolution is its projection's name with ``.conv``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Tuple

from ..config.bovozen import BovozenConfig
from ..config.registry import register_architecture

_NORMS = {"pre_mixer_norm.weight": "norm1", "pre_ffn_norm.weight": "norm2"}
_MIXER = {
    # attention
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "value_mix": "vmix",
    # the delta rule
    "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv",
    "beta_proj.weight": "b", "a_log": "A_log", "dt_bias": "dt_bias",
    "decay_down.weight": "a1", "decay_up.weight": "a2", "gate_down.weight": "g1",
    "gate_up.weight": "g2", "out_norm.weight": "norm",
}
_FFN = {
    "up_proj.weight": "up", "down_proj.weight": "down",
    "router.weight": "router", "router.bias": "router.b",
    "shared.gate_proj.weight": "shared.gate", "shared.up_proj.weight": "shared.up",
    "shared.down_proj.weight": "shared.down", "shared.gate.weight": "shared.sg",
}
_EXPERT = re.compile(r"^experts\.(\d+)\.(gate|up|down)_proj\.weight$")


@dataclass(frozen=True)
class BovozenWeightNames:
    prefixes: Tuple[str, ...] = ("",)
    # names a checkpoint may carry although the model does not use them: the mixing scalar
    # of an attention layer that mixes nothing
    ignore_prefixes: Tuple[str, ...] = ()

    def checkpoint_name(self, internal: str, prefix: str) -> str:
        if internal == "embed.weight":
            return prefix + "embed"
        if internal == "stream_position.table.weight":
            return prefix + "pos"
        if internal == "final_norm.weight":
            return prefix + "final.norm"
        parts = internal.split(".", 2)
        if parts[0] == "blocks" and len(parts) == 3:
            layer, rest = f"{prefix}l{parts[1]}.", parts[2]
            if rest in _NORMS:
                return layer + _NORMS[rest]
            head, _, leaf = rest.partition(".")
            if head == "mixer" and leaf in _MIXER:
                return f"{layer}mix.{_MIXER[leaf]}"
            if head == "ffn":
                if leaf in _FFN:
                    return f"{layer}mlp.{_FFN[leaf]}"
                m = _EXPERT.match(leaf)
                if m:
                    return f"{layer}mlp.e{m.group(1)}.{m.group(2)}"
        raise KeyError(f"Bovozen has no checkpoint name for '{internal}'")


def _weight_names(config: BovozenConfig) -> BovozenWeightNames:
    unused = tuple(f"l{i}.mix.vmix" for i, layer in enumerate(config.layers)
                   if layer.mixer.kind == "attention" and not layer.mixer.v_mix)
    return BovozenWeightNames(ignore_prefixes=unused)


register_architecture("Bovozen", BovozenConfig, _weight_names, model_types=("bovozen",))
