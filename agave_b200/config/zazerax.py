"""Typed configuration of the Zazerax decoder, read from its own ``config.json`` keys.

A Zazerax model is a list of layers.  Each entry names its mixer (``type``: ``attention``,
``latent_attention`` or ``latent_attention_2``), the mixer's sizes and constants
(``mixer``) and its feed-forward (``mlp``: a dense one, or null for a layer without).  An
entry with ``weights_of: j`` has no tensors of its own: it runs layer j's mixer,
feed-forward and norms over a cache entry of its own.  The top level gives the width, the
vocabulary, the norms' eps and the embedding's multiplier.  Every size and every constant
that can differ between two models of the design is read from there.

What the design fixes, and what therefore stands in the lowering below: a branch reads the
stream itself and its output is layer-normed (weight, no bias) before it joins; the dense
feed-forward's activation is the squared relu; ``attention`` norms q and k over the whole
projection, adds one to its softmax denominator and a learned bias by distance to its
scores, and does not rotate; the latent mixers rotate one part of every query head and a
key part that all heads share, split halves in the first kind and interleaved pairs (with
a query latent and one gate value per head) in the second; the head is a tensor of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import (AttentionSpec, BlockSpec, ConfigError, DenseFeedForwardSpec, DistanceBiasSpec,
                   LatentAttentionSpec, LayerCall, LayerNormSpec, ModelSpec, NormSpec, RotarySpec,
                   WavelengthScalingSpec)

MIXERS = ("attention", "latent_attention", "latent_attention_2")


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
class ZazeraxRotation:
    base: float
    dims: int
    # (factor, original, fast, slow) or None
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class ZazeraxMixer:
    """One record for the three kinds; the fields a kind does not have stay at their zero."""
    kind: str
    heads: int
    dim: int
    vdim: int
    scale: float
    # attention
    kv_heads: int = 0
    window: Optional[int] = None
    bias_max: float = 0.0
    # latent attention
    rot_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0
    rot: Optional[ZazeraxRotation] = None


@dataclass(frozen=True)
class ZazeraxLayer:
    mixer: ZazeraxMixer
    ff: Optional[int]                  # width of the dense feed-forward; None: no feed-forward
    weights_of: Optional[int] = None


def _read_rotation(m: dict, where: str) -> ZazeraxRotation:
    rot = _get(m, "rot", where, typ=None)
    rw = where + "rot."
    sc = rot.get("scaling") if isinstance(rot, dict) else None
    scaling = None
    if sc is not None:
        sw = rw + "scaling."
        scaling = (_get(sc, "factor", sw, float), _get(sc, "original", sw, float),
                   _get(sc, "fast", sw, float), _get(sc, "slow", sw, float))
    return ZazeraxRotation(base=_get(rot, "base", rw, float), dims=_get(rot, "dims", rw),
                           scaling=scaling)


def _read_mixer(kind: str, m: dict, where: str) -> ZazeraxMixer:
    common = dict(kind=kind, heads=_get(m, "heads", where), dim=_get(m, "dim", where),
                  vdim=_get(m, "vdim", where), scale=_get(m, "scale", where, float))
    if kind == "attention":
        mask = m.get("mask")
        window = _get(mask, "size", where + "mask.") if mask is not None else None
        return ZazeraxMixer(kv_heads=_get(m, "kv_heads", where) if m.get("kv_heads") is not None
                            else common["heads"], window=window,
                            bias_max=_get(m, "bias_max", where, float), **common)
    return ZazeraxMixer(rot_dim=_get(m, "rot_dim", where), kv_rank=_get(m, "kv_rank", where),
                        q_rank=_get(m, "q_rank", where) if kind == "latent_attention_2" else 0,
                        rot=_read_rotation(m, where), **common)


@dataclass(frozen=True)
class ZazeraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    layers: Tuple[ZazeraxLayer, ...]
    # rows of each attention layer's distance table, by layer that owns tensors (from the
    # tensor's shape; 0 where unknown)
    bias_rows: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Zazerax"

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], shapes=None) -> "ZazeraxConfig":
        """``shapes(name)`` gives a stored tensor's shape (or None); the distance tables'
        row counts come from there, config.json does not state them.  A raw dictionary may
        carry them itself as ``mixer.bias_rows`` (what ``to_dict`` writes)."""
        layers_raw = _get(raw, "layers", "", typ=None)
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers, rows = [], []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where, typ=None)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not a mixer of this "
                                  f"design (known: {', '.join(MIXERS)})")
            m = _get(entry, "mixer", where, typ=None)
            mixer = _read_mixer(kind, m, where + "mixer.")
            ff = None                      # (no 'mlp' key reads as null: no feed-forward)
            if entry.get("mlp") is not None:
                f = entry["mlp"]
                fk = _get(f, "kind", where + "mlp.", typ=None)
                if fk != "dense":
                    raise ConfigError(f"config.json: '{where}mlp.kind' = {fk!r} is not a "
                                      "feed-forward of this design (known: dense)")
                ff = _get(f, "ff", where + "mlp.")
            wo = entry.get("weights_of")
            if wo is not None:
                wo = _get(entry, "weights_of", where)
            layers.append(ZazeraxLayer(mixer, ff, wo))
            n_rows = 0
            if kind == "attention":
                if m.get("bias_rows") is not None:
                    n_rows = _get(m, "bias_rows", where + "mixer.")
                elif shapes is not None:
                    shp = shapes(f"l{wo if wo is not None else i}.mix.rel")
                    if shp is not None:
                        n_rows = int(shp[0])
            rows.append(n_rows)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in eos) if isinstance(eos, list) \
            else (int(eos),)
        bos = raw.get("bos_token_id")
        cfg = cls(vocab=_get(raw, "vocab", ""), width=_get(raw, "width", ""),
                  norm_eps=_get(_get(raw, "norm", "", typ=None), "eps", "norm.", float),
                  embed_scale=_get(_get(raw, "embedding", "", typ=None), "scale", "embedding.",
                                   float),
                  layers=tuple(layers), bias_rows=tuple(rows),
                  bos_token_id=None if bos is None else int(bos), eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer."
            for k in ("heads", "dim", "vdim"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"config.json: '{where}{k}' must be positive")
            if m.scale <= 0:
                raise ConfigError(f"config.json: '{where}scale' must be positive")
            if m.kind == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: '{where}heads' ({m.heads}) must be a "
                                      f"multiple of 'kv_heads' ({m.kv_heads})")
                if m.window is not None and m.window <= 0:
                    raise ConfigError(f"config.json: '{where}mask.size' must be positive")
                n = self.bias_rows[i]
                if n <= 0:
                    raise ConfigError(f"layers[{i}]: the distance table's rows are unknown "
                                      f"(no tensor 'l{i}.mix.rel' and no '{where}bias_rows')")
                if n < 2 or m.bias_max <= n // 2:
                    raise ConfigError(f"config.json: '{where}bias_max' ({m.bias_max}) must "
                                      f"exceed half the distance table's {n} rows")
            else:
                if m.kv_rank <= 0 or m.rot_dim <= 0 or m.rot_dim % 2:
                    raise ConfigError(f"config.json: '{where}kv_rank' must be positive and "
                                      f"'{where}rot_dim' positive and even")
                if m.kind == "latent_attention_2" and m.q_rank <= 0:
                    raise ConfigError(f"config.json: '{where}q_rank' must be positive")
                if m.rot.dims != m.rot_dim:
                    raise ConfigError(f"config.json: '{where}rot.dims' ({m.rot.dims}) must equal "
                                      f"'{where}rot_dim' ({m.rot_dim})")
                if m.rot.base <= 1:
                    raise ConfigError(f"config.json: '{where}rot.base' must exceed 1")
                if m.rot.scaling is not None and (m.rot.scaling[0] <= 0 or m.rot.scaling[1] <= 0
                                                  or m.rot.scaling[2] <= 0 or m.rot.scaling[3] <= 0):
                    raise ConfigError(f"config.json: the numbers under '{where}rot.scaling' "
                                      "must be positive")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"config.json: 'layers[{i}].mlp.ff' must be positive")
            j = layer.weights_of
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i:
                    raise ConfigError(f"config.json: 'layers[{i}].weights_of' = {j} must name "
                                      "another layer")
                src = self.layers[j]
                if src.weights_of is not None:
                    raise ConfigError(f"config.json: 'layers[{i}].weights_of' = {j} names a layer "
                                      "without tensors of its own")
                if (src.mixer, src.ff) != (layer.mixer, layer.ff):
                    raise ConfigError(f"config.json: 'layers[{i}]' must equal the layer whose "
                                      f"weights it uses (layers[{j}])")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            mixer: Dict[str, Any] = {"dim": m.dim, "heads": m.heads, "scale": m.scale,
                                     "vdim": m.vdim}
            if m.kind == "attention":
                mixer.update(kv_heads=m.kv_heads, bias_max=m.bias_max, bias_rows=self.bias_rows[i])
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
            else:
                rot: Dict[str, Any] = {"base": m.rot.base, "dims": m.rot.dims}
                if m.rot.scaling is not None:
                    f, o, fa, sl = m.rot.scaling
                    rot["scaling"] = {"factor": f, "original": o, "fast": fa, "slow": sl}
                mixer.update(kv_rank=m.kv_rank, rot_dim=m.rot_dim, rot=rot)
                if m.kind == "latent_attention_2":
                    mixer["q_rank"] = m.q_rank
            e: Dict[str, Any] = {"mixer": mixer, "type": m.kind,
                                 "mlp": None if layer.ff is None else {"ff": layer.ff,
                                                                       "kind": "dense"}}
            if layer.weights_of is not None:
                e["weights_of"] = layer.weights_of
            layers.append(e)
        d: Dict[str, Any] = {"architecture": self.architecture,
                             "embedding": {"scale": self.embed_scale}, "layers": layers,
                             "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                             "width": self.width}
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------------------------- lower
    def owners(self) -> Tuple[int, ...]:
        """Layer numbers that have tensors of their own, in order: block b of the lowered
        model is layer ``owners()[b]``."""
        return tuple(i for i, layer in enumerate(self.layers) if layer.weights_of is None)

    def _mixer_spec(self, i: int):
        m = self.layers[i].mixer
        if m.kind == "attention":
            return AttentionSpec(
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                window=m.window, qk_norm=NormSpec(eps=self.norm_eps, zero_centered=False),
                qk_norm_whole=True, position=None,
                value_dim=0 if m.vdim == m.dim else m.vdim, fixed_sink=0.0,
                distance_bias=DistanceBiasSpec(rows=self.bias_rows[i], far=m.bias_max))
        second = m.kind == "latent_attention_2"
        sc = m.rot.scaling
        position = RotarySpec(
            theta=m.rot.base, rotary_dim=m.rot_dim, interleaved=second,
            scaling=None if sc is None else WavelengthScalingSpec(
                factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3]))
        return LatentAttentionSpec(
            n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
            kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, eps=self.norm_eps,
            position=position, gate="head" if second else "element")

    def to_model_spec(self) -> ModelSpec:
        norm = LayerNormSpec(eps=self.norm_eps, bias=False)
        owners = self.owners()
        block_of = {layer: b for b, layer in enumerate(owners)}
        blocks = []
        for i in owners:
            layer = self.layers[i]
            ffn = None if layer.ff is None else DenseFeedForwardSpec(
                intermediate_size=layer.ff, activation="relu2")
            blocks.append(BlockSpec(mixer=self._mixer_spec(i), feed_forward=ffn, norm=norm,
                                    arrangement="post"))
        # every layer has a cache entry of its own; a layer that borrows weights runs the
        # owner's block over it
        schedule = tuple(
            LayerCall(block=block_of[i if layer.weights_of is None else layer.weights_of],
                      cache=i, writes_cache=True)
            for i, layer in enumerate(self.layers))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, embed_scale=self.embed_scale,
            blocks=tuple(blocks), schedule=schedule, final_norm=norm, tie_embeddings=False,
            max_positions=0, bos_token_id=self.bos_token_id, eos_token_ids=self.eos_token_ids)
