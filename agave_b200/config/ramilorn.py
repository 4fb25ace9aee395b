"""Typed configuration of the Ramilorn decoder, read from its own ``config.json`` keys.

A Ramilorn model is a list of layers.  Each entry names its mixer type (``attention``),
the mixer's sizes and options (``mixer``) and its feed-forward (``mlp``: a mixture of
experts, or null for a layer without one); the top level gives the width, the vocabulary,
the norms' eps, the multiplier every branch joins the stream with, and the cap of the
logits.  Every size and every constant that can differ between two models of the design is
read from there; nothing is defaulted except what the design itself leaves optional
(``kv_from``, expert groups).

What the design fixes, and what therefore stands in the lowering below: layer norms with
weight and bias before and after every branch; attention without a rotation, with a sink
logit per query head and a query temperature; experts gated with SiLU and a sigmoid router
whose correction only chooses; the head tied to the embedding; no embedding scale.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import (AttentionSpec, BlockSpec, ConfigError, LayerCall, LayerNormSpec, ModelSpec,
                   QueryTemperatureSpec, RoutedFeedForwardSpec)


def _get(d: Dict[str, Any], key: str, where: str, typ=int):
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
class RamilornMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: float
    q_temp_every: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class RamilornMoE:
    experts: int
    top: int
    ff: int
    groups: int
    keep: int


@dataclass(frozen=True)
class RamilornLayer:
    mixer: RamilornMixer
    mlp: Optional[RamilornMoE]


@dataclass(frozen=True)
class RamilornConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float
    layers: Tuple[RamilornLayer, ...]
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Ramilorn"

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "RamilornConfig":
        layers_raw = _get(raw, "layers", "", typ=None)
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where, typ=None)
            if kind != "attention":
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not a mixer of this "
                                  "design (known: attention)")
            m = _get(entry, "mixer", where, typ=None)
            mw = where + "mixer."
            qt = _get(m, "q_temp", mw, typ=None)
            kv_from = m.get("kv_from")
            if kv_from is not None:
                kv_from = _get(m, "kv_from", mw)
            heads = _get(m, "heads", mw)
            mixer = RamilornMixer(
                heads=heads, kv_heads=_get(m, "kv_heads", mw) if m.get("kv_heads") is not None
                else heads, dim=_get(m, "dim", mw), vdim=_get(m, "vdim", mw),
                scale=_get(m, "scale", mw, float), q_temp_coef=_get(qt, "coef", mw + "q_temp.", float),
                q_temp_every=_get(qt, "every", mw + "q_temp."), kv_from=kv_from)
            mlp = None
            if "mlp" not in entry:
                raise ConfigError(f"config.json: required key '{where}mlp' is missing (null: no "
                                  "feed-forward)")
            if entry["mlp"] is not None:
                f = entry["mlp"]
                fw = where + "mlp."
                fk = _get(f, "kind", fw, typ=None)
                if fk != "moe":
                    raise ConfigError(f"config.json: '{fw}kind' = {fk!r} is not a feed-forward of "
                                      "this design (known: moe)")
                r = _get(f, "router", fw, typ=None)
                g = r.get("groups") if isinstance(r, dict) else None
                mlp = RamilornMoE(
                    experts=_get(r, "experts", fw + "router."), top=_get(r, "top", fw + "router."),
                    ff=_get(_get(f, "expert", fw, typ=None), "ff", fw + "expert."),
                    groups=_get(g, "count", fw + "router.groups.") if g is not None else 1,
                    keep=_get(g, "keep", fw + "router.groups.") if g is not None else 1)
            layers.append(RamilornLayer(mixer, mlp))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in eos) if isinstance(eos, list) \
            else (int(eos),)
        bos = raw.get("bos_token_id")
        cfg = cls(vocab=_get(raw, "vocab", ""), width=_get(raw, "width", ""),
                  norm_eps=_get(_get(raw, "norm", "", typ=None), "eps", "norm.", float),
                  residual_mult=_get(raw, "residual_mult", "", float),
                  logit_softcap=_get(raw, "logit_softcap", "", float),
                  layers=tuple(layers), bos_token_id=None if bos is None else int(bos),
                  eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        if self.logit_softcap <= 0:
            raise ConfigError("config.json: 'logit_softcap' must be positive")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer."
            for k in ("heads", "kv_heads", "dim", "vdim", "q_temp_every"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"config.json: '{where}{k}' must be positive")
            if m.heads % m.kv_heads:
                raise ConfigError(f"config.json: '{where}heads' ({m.heads}) must be a multiple of "
                                  f"'kv_heads' ({m.kv_heads})")
            if m.scale <= 0:
                raise ConfigError(f"config.json: '{where}scale' must be positive")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    raise ConfigError(f"config.json: '{where}kv_from' = {m.kv_from} must name an "
                                      "earlier layer")
                src = self.layers[m.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"config.json: '{where}kv_from' = {m.kv_from} names a layer "
                                      "without keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"config.json: '{where}kv_from' = {m.kv_from}: the two "
                                      "layers' kv_heads, dim and vdim must be equal")
            f = layer.mlp
            if f is not None:
                where = f"layers[{i}].mlp."
                if min(f.experts, f.top, f.ff, f.groups, f.keep) <= 0:
                    raise ConfigError(f"config.json: the sizes under '{where}' must be positive")
                if f.experts % f.groups:
                    raise ConfigError(f"config.json: '{where}router.experts' ({f.experts}) must "
                                      f"form {f.groups} equal groups")
                if f.keep > f.groups:
                    raise ConfigError(f"config.json: '{where}router.groups.keep' exceeds 'count'")
                if f.top > f.keep * (f.experts // f.groups):
                    raise ConfigError(f"config.json: '{where}router.top' ({f.top}) exceeds the "
                                      "experts of the groups kept")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer: Dict[str, Any] = {
                "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads,
                "q_temp": {"coef": m.q_temp_coef, "every": m.q_temp_every},
                "scale": m.scale, "vdim": m.vdim}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            f = layer.mlp
            mlp = None if f is None else {
                "expert": {"ff": f.ff}, "kind": "moe",
                "router": {"experts": f.experts, "groups": {"count": f.groups, "keep": f.keep},
                           "top": f.top}}
            layers.append({"mixer": mixer, "mlp": mlp, "type": "attention"})
        d: Dict[str, Any] = {
            "architecture": self.architecture, "layers": layers,
            "logit_softcap": self.logit_softcap, "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------------------------- lower
    def to_model_spec(self) -> ModelSpec:
        norm = LayerNormSpec(eps=self.norm_eps, bias=True)
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            attn = AttentionSpec(
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                window=None, qk_norm=None, position=None,
                value_dim=0 if m.vdim == m.dim else m.vdim, sink=True,
                q_temp=QueryTemperatureSpec(coef=m.q_temp_coef, every=m.q_temp_every),
                own_kv=m.kv_from is None)
            f = layer.mlp
            ffn = None if f is None else RoutedFeedForwardSpec(
                n_experts=f.experts, top=f.top, intermediate_size=f.ff, activation="silu",
                n_groups=f.groups, keep_groups=f.keep, correction=True)
            blocks.append(BlockSpec(mixer=attn, feed_forward=ffn, norm=norm,
                                    arrangement="sandwich", residual_mult=self.residual_mult))
            # a layer without keys and values of its own reads the entry its source writes
            schedule.append(LayerCall(block=i, cache=i if m.kv_from is None else m.kv_from,
                                      writes_cache=m.kv_from is None))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, embed_scale=1.0,
            blocks=tuple(blocks), schedule=tuple(schedule), final_norm=norm,
            tie_embeddings=True, max_positions=0, bos_token_id=self.bos_token_id,
            eos_token_ids=self.eos_token_ids, logit_softcap=self.logit_softcap)
