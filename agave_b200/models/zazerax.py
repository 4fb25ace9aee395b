"""Zazerax: the registry entry and the names of its tensors.

The layer structure is data (``ZazeraxConfig.to_model_spec``): three kinds of mixer (windowed
attention with a distance bias, and two latent attentions), a dense squared-relu
feed-forward, a layer norm on every branch's output, layers that run another layer's weights
over a cache entry of their own, a head of its own.  What is left to say here is how the
generic decoder's tensor names map to a checkpoint's: ``embed``, ``head``, ``final.norm``
and per layer that owns tensors ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*`` and
``l<i>.mlp.{up,down}``.  Block b of the lowered model is the b-th layer that owns tensors,
so its names carry that layer's number.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

from ..config.registry import register_architecture
from ..config.zazerax import ZazeraxConfig

_NORMS = {"post_mixer_norm.weight": "norm1", "post_ffn_norm.weight": "norm2"}
_MIXER = {
    # windowed attention
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "distance_bias": "rel",
    # latent attention
    "q_down.weight": "dq", "q_down_norm.weight": "dq.norm", "q_up.weight": "uq",
    "kv_down.weight": "dkv", "kv_down_norm.weight": "dkv.norm", "k_up.weight": "uk",
    "v_up.weight": "uv", "gate.weight": "g",
}
_FFN = {"up_proj.weight": "up", "down_proj.weight": "down"}


@dataclass(frozen=True)
class ZazeraxWeightNames:
    owners: Tuple[int, ...]            # layer number of each block
    prefixes: Tuple[str, ...] = ("",)

    def checkpoint_name(self, internal: str, prefix: str) -> str:
        if internal == "embed.weight":
            return prefix + "embed"
        if internal == "lm_head.weight":
            return prefix + "head"
        if internal == "final_norm.weight":
            return prefix + "final.norm"
        parts = internal.split(".", 2)
        if parts[0] == "blocks" and len(parts) == 3 and int(parts[1]) < len(self.owners):
            layer, rest = f"{prefix}l{self.owners[int(parts[1])]}.", parts[2]
            if rest in _NORMS:
                return layer + _NORMS[rest]
            head, _, leaf = rest.partition(".")
            if head == "mixer" and leaf in _MIXER:
                return f"{layer}mix.{_MIXER[leaf]}"
            if head == "ffn" and leaf in _FFN:
                return f"{layer}mlp.{_FFN[leaf]}"
        raise KeyError(f"Zazerax has no checkpoint name for '{internal}'")


def _weight_names(config: ZazeraxConfig) -> ZazeraxWeightNames:
    return ZazeraxWeightNames(owners=config.owners())


register_architecture("Zazerax", ZazeraxConfig, _weight_names, model_types=("zazerax",))
