"""Ramilorn: the registry entry and the names of its tensors.

The layer structure is data (``RamilornConfig.to_model_spec``): attention with a sink and
a query temperature (some layers attending to an earlier layer's keys and values), a
routed feed-forward, layer norms around every branch, a capped head tied to the
embedding.  What is left to say here is how the generic decoder's tensor names map to a
checkpoint's: ``embed``, ``final.norm``, and per layer ``l<i>.norm1`` / ``norm1b`` /
``norm2`` / ``norm2b`` (a bias is the weight's name with ``.b``), ``l<i>.mix.{q,k,v,o,sink}``,
``l<i>.mlp.router``, ``l<i>.mlp.correction`` and ``l<i>.mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Tuple

from ..config.ramilorn import RamilornConfig
from ..config.registry import register_architecture

_NORMS = {"pre_mixer_norm": "norm1", "post_mixer_norm": "norm1b",
          "pre_ffn_norm": "norm2", "post_ffn_norm": "norm2b"}
_MIXER = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
          "o_proj.weight": "o", "sink": "sink"}
_EXPERT = re.compile(r"^experts\.(\d+)\.(gate|up|down)_proj\.weight$")


def _norm_name(base: str, leaf: str) -> str:
    if leaf == "weight":
        return base
    if leaf == "bias":
        return base + ".b"
    raise KeyError(leaf)


@dataclass(frozen=True)
class RamilornWeightNames:
    prefixes: Tuple[str, ...] = ("",)

    def checkpoint_name(self, internal: str, prefix: str) -> str:
        if internal == "embed.weight":
            return prefix + "embed"
        if internal.startswith("final_norm."):
            return prefix + _norm_name("final.norm", internal.split(".", 1)[1])
        parts = internal.split(".", 2)
        if parts[0] == "blocks" and len(parts) == 3:
            layer, rest = f"{prefix}l{parts[1]}.", parts[2]
            head, _, leaf = rest.partition(".")
            if head in _NORMS:
                return layer + _norm_name(_NORMS[head], leaf)
            if head == "mixer" and leaf in _MIXER:
                return f"{layer}mix.{_MIXER[leaf]}"
            if head == "ffn":
                if leaf == "router.weight":
                    return layer + "mlp.router"
                if leaf == "router.correction":
                    return layer + "mlp.correction"
                m = _EXPERT.match(leaf)
                if m:
                    return f"{layer}mlp.e{m.group(1)}.{m.group(2)}"
        raise KeyError(f"Ramilorn has no checkpoint name for '{internal}'")


def _weight_names(config: RamilornConfig) -> RamilornWeightNames:
    return RamilornWeightNames()


register_architecture("Ramilorn", RamilornConfig, _weight_names, model_types=("ramilorn",))
