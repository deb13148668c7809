"""Kadavik: the registry entry and the names of its tensors.

The layer structure is data (``KadavikConfig.to_model_spec``): a matrix memory with
exponential gates or attention with a short convolution on q, k and v, a partial rotation, a
sliding window behind which the first keys stay visible and an output gate; a dense tanh-GELU
feed-forward or routed experts (softmax scores, identity experts) beside a gated shared one;
RMS norms before and after every branch; a per-layer input from the token; a scaled embedding
and a head tied to it.  What is left to say here is how the generic decoder's tensor names map
to a checkpoint's: ``embed``, ``side.embed``, ``final.norm`` and per layer ``l<i>.norm1`` /
``norm1b`` / ``norm2`` / ``norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*`` (experts
``e<j>.{gate,up,down}``, ``router``, ``correction``, ``shared.{gate,up,down,sg}``) and
``l<i>.side.{gate,proj,norm}``; a convolution is its projection's name with ``.conv``, a bias
its projection's with ``.b``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Tuple

from ..config.kadavik import KadavikConfig
from ..config.registry import register_architecture
from ..parts import matrix_memory as _matrix_memory      # registers the mixer

_NORMS = {"pre_mixer_norm.weight": "norm1", "post_mixer_norm.weight": "norm1b",
          "pre_ffn_norm.weight": "norm2", "post_ffn_norm.weight": "norm2b"}
_MIXER = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
    "o_proj.weight": "o",
    # attention
    "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv",
    # the matrix memory
    "i_proj.weight": "i", "i_proj.bias": "i.b", "f_proj.weight": "f", "f_proj.bias": "f.b",
    "out_norm.weight": "norm",
}
_FFN = {
    "gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down",
    "router.weight": "router", "router.correction": "correction",
    "shared.gate_proj.weight": "shared.gate", "shared.up_proj.weight": "shared.up",
    "shared.down_proj.weight": "shared.down", "shared.gate.weight": "shared.sg",
}
_SIDE = {"gate_proj.weight": "gate", "proj.weight": "proj", "norm.weight": "norm"}
_EXPERT = re.compile(r"^experts\.(\d+)\.(gate|up|down)_proj\.weight$")


@dataclass(frozen=True)
class KadavikWeightNames:
    prefixes: Tuple[str, ...] = ("",)
    ignore_prefixes: Tuple[str, ...] = ()

    def checkpoint_name(self, internal: str, prefix: str) -> str:
        if internal == "embed.weight":
            return prefix + "embed"
        if internal == "token_side.weight":
            return prefix + "side.embed"
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
            if head == "side" and leaf in _SIDE:
                return f"{layer}side.{_SIDE[leaf]}"
            if head == "ffn":
                if leaf in _FFN:
                    return f"{layer}mlp.{_FFN[leaf]}"
                m = _EXPERT.match(leaf)
                if m:
                    return f"{layer}mlp.e{m.group(1)}.{m.group(2)}"
        raise KeyError(f"Kadavik has no checkpoint name for '{internal}'")


def _weight_names(config: KadavikConfig) -> KadavikWeightNames:
    return KadavikWeightNames()


register_architecture("Kadavik", KadavikConfig, _weight_names, model_types=("kadavik",))
