"""A plain, slow Ramilorn decoder for comparison: whole sequences, no cache.

One function per mechanism, each written from the design's equations.  Nothing
here is imported by, or imports, the library under test: the configuration is a
dictionary and the weights a dictionary of tensors under their checkpoint
names (read with the ``safetensors`` package).

Arithmetic runs in the dtype of the tensors handed in (float64 by default).

Notation: W are matrices stored [out, in]; t, j are positions; a is a query
head and g = a // (A / G) its key/value head.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

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


# ---------------------------------------------------------------------- parts
def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def query_temperature(n: int, coef: float, every: int, dtype) -> torch.Tensor:
    """tau[t] = 1 + coef * ln(floor((t + 1) / every) + 1)."""
    t = torch.arange(n)
    steps = torch.div(t + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log((steps + 1).to(dtype))


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sink: torch.Tensor,
                   scale: float) -> torch.Tensor:
    """q [T, A, d], k [T, G, d], v [T, G, dv], sink [A] -> [T, A, dv].

    s[t, j] = scale * q_t . k_j for j <= t;
    p[t, j] = exp(s[t, j]) / (exp(sink_a) + sum_{i <= t} exp(s[t, i])).
    The sink adds to the denominator only."""
    T, A, _ = q.shape
    G = k.shape[1]
    rep = A // G
    out = torch.zeros(T, A, v.shape[2], dtype=q.dtype)
    for a in range(A):
        g = a // rep
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, a]) * scale
            m = torch.maximum(s.max(), sink[a])
            e = torch.exp(s - m)
            den = e.sum() + torch.exp(sink[a] - m)
            out[t, a] = (e / den) @ v[:t + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict,
                    kv: Optional[tuple]):
    """The mixer of one layer on h [T, H]; returns (y [T, H], (k, v)).

    ``kv`` given: the layer has no key/value projections and attends to those."""
    T = h.shape[0]
    A, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, A, d)
    if kv is None:
        k = (h @ w[pre + "k"].T).view(T, G, d)
        v = (h @ w[pre + "v"].T).view(T, G, dv)
    else:
        k, v = kv
    tau = query_temperature(T, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]), h.dtype)
    q = q * tau.view(T, 1, 1)
    o = sink_attention(q, k, v, w[pre + "sink"], float(m["scale"]))
    return o.reshape(T, A * dv) @ w[pre + "o"].T, (k, v)


def route(x: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict):
    """Per token of x [T, H]: (chosen expert ids [T, top], their weights [T, top]).

    s = sigmoid(W_r x); c = s + correction picks, s weighs.  Experts lie in
    ``count`` equal groups of neighbours; a group's score is the sum of its two
    largest c; only the ``keep`` best groups stay eligible; the ``top`` largest
    c among the eligible win; the weights are their s, as they are."""
    E, top = int(r["experts"]), int(r["top"])
    grp = r.get("groups") or {"count": 1, "keep": 1}
    n_g, keep = int(grp["count"]), int(grp["keep"])
    s = torch.sigmoid(x @ w_router.T)
    c = s + correction
    per = E // n_g
    cg = c.view(-1, n_g, per)
    g_score = cg.topk(min(2, per), dim=-1).values.sum(dim=-1)
    best = g_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(x.shape[0], n_g, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed.unsqueeze(-1).expand(-1, -1, per).reshape(-1, E), c,
                         torch.full_like(c, -math.inf))
    ids = masked.topk(top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def expert(x: torch.Tensor, w: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    """W_down (silu(W_gate x) * (W_up x))."""
    g = x @ w[pre + "gate"].T
    u = x @ w[pre + "up"].T
    return (g * torch.sigmoid(g) * u) @ w[pre + "down"].T


def moe(x: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mlp: dict,
        ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``ids`` [T, top] given: those experts are used instead of the router's own choice
    (their weights are still this router's scores): for comparisons in reduced precision,
    where a close call may fall the other way."""
    own, wt = route(x, w[pre + "router"], w[pre + "correction"], mlp["router"])
    if ids is None:
        ids = own
    else:
        wt = torch.gather(torch.sigmoid(x @ w[pre + "router"].T), 1, ids.long())
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, a in zip(ids[t].tolist(), wt[t]):
            y[t] += a * expert(x[t:t + 1], w, f"{pre}e{e}.")[0]
    return y


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ---------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            streams: Optional[List[torch.Tensor]] = None,
            experts: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, V] of one sequence; ``streams`` collects the stream after each layer;
    ``experts`` {layer: ids [T, top]} fixes the experts of those layers (see ``moe``)."""
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg["residual_mult"])

    def norm(x, name):
        return layer_norm(x, w[name], w[name + ".b"], eps)

    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(f"unknown layer type {layer['type']!r}")
        m = layer["mixer"]
        src = m.get("kv_from")
        y, kept[i] = attention_mixer(norm(x, p + "norm1"), w, p + "mix.", m,
                                     kept[src] if src is not None else None)
        x = x + mult * norm(y, p + "norm1b")
        if layer.get("mlp") is not None:
            y = moe(norm(x, p + "norm2"), w, p + "mlp.", layer["mlp"],
                    None if experts is None else experts.get(i))
            x = x + mult * norm(y, p + "norm2b")
        if streams is not None:
            streams.append(x.clone())
    z = norm(x, "final.norm") @ w["embed"].T
    return soft_cap(z, float(cfg["logit_softcap"]))
