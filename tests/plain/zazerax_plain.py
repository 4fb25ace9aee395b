"""A plain, slow Zazerax decoder for comparison: whole sequences, no cache.

One function per mechanism, each written from the design's equations.  Nothing here is
imported by, or imports, the library under test: the configuration is a dictionary and the
weights a dictionary of tensors under their checkpoint names.

Arithmetic runs in the dtype of the tensors handed in (float64 by default).

Notation: W are matrices stored [out, in]; t, j are positions; a is a query head.
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
def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w, var = mean of the squared deviations."""
    d = x - x.mean(dim=-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------ rotations
def rotary_frequencies(rot: dict) -> (torch.Tensor, float):
    """(f [dims / 2] in 64-bit, multiplier of cos and sin).

    f_i = base^(-2 i / dims); with ``scaling`` the frequencies between the two wavelength
    bounds are blended with f_i / factor by a linear ramp over the pair index."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, interleaved: bool) -> torch.Tensor:
    """x [T, ..., dims] rotated by position.  Pairs are (i, i + dims/2), or (2i, 2i + 1) when
    ``interleaved``; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    f, mult = rotary_frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * mult).to(x.dtype), (torch.sin(a) * mult).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    half = x.shape[-1] // 2
    out = torch.empty_like(x)
    if interleaved:
        u, v = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = u * cos - v * sin
        out[..., 1::2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:]
        out[..., :half] = u * cos - v * sin
        out[..., half:] = v * cos + u * sin
    return out


# ------------------------------------------------------------------ attention
def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of the distance table for distance n >= 0: the first rows / 2 distances have a
    row each, the rest share rows that grow logarithmically up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half)
                                                * (rows - half))))


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      window: Optional[int] = None, bias: Optional[torch.Tensor] = None,
                      far: float = 0.0, one_in_denominator: bool = False) -> torch.Tensor:
    """q [T, A, d], k [T, G, d], v [T, G, dv] -> [T, A, dv].

    s[t, j] = scale * q_t . k_j (+ bias[bucket(t - j), a]) for the visible j <= t
    (t - j < window); p = exp(s) / (sum exp(s) (+ 1))."""
    T, A, _ = q.shape
    rep = A // k.shape[1]
    out = torch.zeros(T, A, v.shape[2], dtype=q.dtype)
    if bias is not None:
        row_of = torch.tensor([distance_bucket(n, bias.shape[0], far) for n in range(T)])
    for a in range(A):
        g = a // rep
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, g] @ q[t, a]) * scale
            if bias is not None:
                # keys lo..t lie at distances t - lo .. 0
                s = s + bias[row_of[:t - lo + 1].flip(0), a]
            m = s.max()
            if one_in_denominator:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            den = e.sum()
            if one_in_denominator:
                den = den + math.exp(-float(m))
            out[t, a] = (e / den) @ v[lo:t + 1, g]
    return out


def windowed_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict,
                             eps: float) -> torch.Tensor:
    """Grouped heads, q and k normed over the whole projection, distance bias, window, one in
    the denominator."""
    T = h.shape[0]
    A, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[pre + "q"].T, w[pre + "q.norm"], eps).view(T, A, d)
    k = rms_norm(h @ w[pre + "k"].T, w[pre + "k.norm"], eps).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    o = softmax_attention(q, k, v, m["scale"], window=m["mask"]["size"], bias=w[pre + "rel"],
                          far=float(m["bias_max"]), one_in_denominator=True)
    return o.reshape(T, A * dv) @ w[pre + "o"].T


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict,
                           eps: float, second: bool) -> torch.Tensor:
    """Keys and values rebuilt from a normed latent; one rotated key part for all heads.
    ``second``: queries through a normed latent too, interleaved pairs, a gate per head."""
    T = h.shape[0]
    A, d, r, dv, c_dim = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    if second:
        q = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps) @ w[pre + "uq"].T
    else:
        q = h @ w[pre + "q"].T
    q = q.view(T, A, d + r)
    ckr = h @ w[pre + "dkv"].T
    c = rms_norm(ckr[:, :c_dim], w[pre + "dkv.norm"], eps)
    k_rot = rotate(ckr[:, c_dim:], pos, m["rot"], interleaved=second)            # [T, r]
    q_rot = rotate(q[..., d:], pos, m["rot"], interleaved=second)                # [T, A, r]
    k_plain = (c @ w[pre + "uk"].T).view(T, A, d)
    v = (c @ w[pre + "uv"].T).view(T, A, dv)
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot[:, None, :].expand(T, A, r)], dim=-1)
    o = softmax_attention(qq, kk, v, m["scale"])
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    if second:
        o = o * gate[:, :, None]
    else:
        o = o * gate.view(T, A, dv)
    return o.reshape(T, A * dv) @ w[pre + "o"].T


# --------------------------------------------------------------- feed-forward
def squared_relu_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    z = torch.relu(h @ w[pre + "up"].T)
    return (z * z) @ w[pre + "down"].T


# ---------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int],
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``streams`` collects the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        pre = f"l{src}."
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            y = windowed_attention_mixer(x, w, pre + "mix.", m, eps)
        elif kind in ("latent_attention", "latent_attention_2"):
            y = latent_attention_mixer(x, w, pre + "mix.", m, eps, kind == "latent_attention_2")
        else:
            raise ValueError(kind)
        x = x + layer_norm(y, w[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(squared_relu_feed_forward(x, w, pre + "mlp."), w[pre + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
