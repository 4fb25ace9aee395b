"""Latent attention as a mixer part: keys and values rebuilt from a cached latent.

Per position the cache holds one row c | kr: the RMS-normed key/value latent c (``kv_rank``
values) and one rotated key part kr (``rot_dim`` values) that every head shares.  With
A heads, d = ``head_dim`` unrotated and r = ``rot_dim`` rotated query/key dimensions:

    score_a(t, j) = scale * (q_a[:d] . (W_uk c_j)_a + rot_t(q_a[d:]) . kr_j),   j <= t
    out_a(t)      = sum_j softmax_j(score_a(t, .)) (W_uv c_j)_a

and the concatenated heads, times sigmoid(W_g x) (element by element, or one value per head),
go through W_o.  The queries come from x directly (W_q) or, with ``q_rank``, through a normed
latent of their own (W_uq rmsnorm(W_dq x)).

Two ways to compute the same sums.  A prompt step rebuilds keys and values for its tokens
(the products W_uk c and W_uv c) and runs ordinary multi-head attention over the step's own
tensors.  A decode step never rebuilds them: W_uk is absorbed into the query
(q'_a = W_uk,a^T q_a[:d], ``kv_rank`` wide), every head attends to the cache rows
themselves, whose leading ``kv_rank`` values also serve as values, and W_uv is applied to
the ``kv_rank``-wide result; the cache is read once for all heads.

One stacked product gives Q | c | kr | g from x; one kernel norms c (and a query latent),
rotates kr (and the queries' rotated parts) and stores the cache row.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import LatentAttentionSpec
from ..engine.batch import PREFILL
from .base import KVRequest, ParamSpec, position_class, register_mixer
from .linear import Linear


class LatentAttentionMixer:
    def __init__(self, spec: LatentAttentionSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.position is None or (spec.position.rotary_dim or spec.rot_dim) != spec.rot_dim:
            raise ValueError("latent attention rotates exactly its rot_dim part")
        if spec.gate not in (None, "element", "head"):
            raise ValueError(f"unknown gate {spec.gate!r}")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        self.position = position_class(spec.position.kind)(spec.position, spec.rot_dim)
        self.interleaved = bool(spec.position.interleaved)
        self.q_latent = spec.q_rank > 0
        self.q_width = spec.q_rank if self.q_latent else spec.n_heads * (spec.head_dim + spec.rot_dim)
        self.gate_width = {None: 0, "element": spec.n_heads * spec.value_dim,
                           "head": spec.n_heads}[spec.gate]
        self.down: Optional[Linear] = None        # Q | c | kr | g from x
        self.q_up: Optional[Linear] = None
        self.k_up: Optional[Linear] = None        # k_plain from c (prompts)
        self.v_up_prompt: Optional[Linear] = None # v from c (prompts)
        self.k_absorb: Optional[torch.Tensor] = None   # [A, kv_rank, d]: W_uk per head, transposed
        self.v_up: Optional[torch.Tensor] = None       # [A, value_dim, kv_rank]
        self.out: Optional[Linear] = None
        self.w_q_norm = self.w_c_norm = None

    @classmethod
    def param_specs(cls, spec: LatentAttentionSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        A, d, r, dv, R = spec.n_heads, spec.head_dim, spec.rot_dim, spec.value_dim, spec.kv_rank
        p: Dict[str, ParamSpec] = {}
        if spec.q_rank > 0:
            p["q_down.weight"] = ParamSpec((spec.q_rank, hidden_size))
            p["q_down_norm.weight"] = ParamSpec((spec.q_rank,), "norm")
            p["q_up.weight"] = ParamSpec((A * (d + r), spec.q_rank))
        else:
            p["q_proj.weight"] = ParamSpec((A * (d + r), hidden_size))
        p["kv_down.weight"] = ParamSpec((R + r, hidden_size))
        p["kv_down_norm.weight"] = ParamSpec((R,), "norm")
        p["k_up.weight"] = ParamSpec((A * d, R))
        p["v_up.weight"] = ParamSpec((A * dv, R))
        if spec.gate == "element":
            p["gate.weight"] = ParamSpec((A * dv, hidden_size))
        elif spec.gate == "head":
            p["gate.weight"] = ParamSpec((A, hidden_size))
        p["o_proj.weight"] = ParamSpec((hidden_size, A * dv))
        return p

    def cache_request(self):
        s = self.spec
        return KVRequest(1, s.kv_rank + s.rot_dim, None, value_dim=s.kv_rank, values_in_keys=True)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        s = self.spec
        A, d, dv, R = s.n_heads, s.head_dim, s.value_dim, s.kv_rank

        def mat(name):
            return tensors[name].to(device=device, dtype=dtype)
        first = mat("q_down.weight") if self.q_latent else mat("q_proj.weight")
        stack = [first, mat("kv_down.weight")] + ([mat("gate.weight")] if s.gate else [])
        self.down = Linear(torch.cat(stack, dim=0).contiguous(), role="qkv")
        if self.q_latent:
            self.q_up = Linear(mat("q_up.weight").contiguous(), role="q_up")
            self.w_q_norm = tensors["q_down_norm.weight"].to(device=device,
                                                             dtype=torch.float32).contiguous()
        self.w_c_norm = tensors["kv_down_norm.weight"].to(device=device,
                                                          dtype=torch.float32).contiguous()
        uk, uv = mat("k_up.weight"), mat("v_up.weight")
        # (two products, so that the values come out dense: the prompt attention kernels
        # want keys and values at one row stride)
        self.k_up = Linear(uk.contiguous(), role="kv_up")
        self.v_up_prompt = Linear(uv.contiguous(), role="kv_up")
        self.k_absorb = uk.view(A, d, R).transpose(1, 2).contiguous()
        self.v_up = uv.view(A, dv, R).contiguous()
        self.out = Linear(mat("o_proj.weight").contiguous(), role="out_proj")
        if hasattr(self.position, "prepare"):
            self.position.prepare(device)

    def forward(self, x: torch.Tensor, ctx, cache_entry: int, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a latent-attention layer writes its own cache entry")
        s = self.spec
        A, d, r, dv, R = s.n_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        hw, G, Q = d + r, self.gate_width, self.q_width
        T = x.shape[0]
        cos, sin = self.position.tables(ctx)
        view = ctx.cache.kv_view(cache_entry)
        proj = self.down.partial(x, cheap_sum=True)
        part = proj if proj.dim() == 3 else None
        row = proj if part is None else ctx.new(T, Q + R + r + G)
        kernels.latent_prepare(row, Q, self.q_latent, A, d, r, R, G, self.w_q_norm, self.w_c_norm,
                               s.eps, cos, sin, self.interleaved, ctx.positions, view, ctx,
                               partial=part)
        if self.q_latent:
            q = self.q_up(row[:, :Q])
            kernels.rotate_heads(q, A, hw, r, cos, sin, self.interleaved)
        else:
            q = row[:, :Q]
        c, kr = row[:, Q:Q + R], row[:, Q + R:Q + R + r]
        out = ctx.new(T, A * dv)
        if ctx.mode == PREFILL:
            k = ctx.new(T, A * hw)
            kernels.assemble_keys(self.k_up(c), kr, k, A, d, r)
            kernels.attention_prefill(q, k, self.v_up_prompt(c), out, ctx, A, A, hw, s.scale, 0,
                                      value_dim=dv, op="latent_attention")
        else:
            # the key up-projection goes into the query (the rotated part passes through);
            # the heads attend to the cache rows themselves
            D = R + r
            ql = ctx.new(T, A, D)
            kernels.heads_linear(q.unflatten(1, (A, hw)), self.k_absorb, ql, tail=r, op="q_absorb")
            if D % 16 == 0 and D <= 512:
                # the split kernel with the whole row as the value: one kv head, every query
                # head in its group; the r values behind the latent's weighted sum are unused
                lat = ctx.new(T, A, D)
                kernels.attention_decode(ql.view(T, A * D), lat.view(T, A * D), view, ctx, A, 1, D,
                                         s.scale, 0, op="latent_attention")
                lat = lat[:, :, :R]
            else:
                lat = ctx.new(T, A, R)
                kernels.attention_decode(ql.view(T, A * D), lat.view(T, A * R), view, ctx, A, 1, D,
                                         s.scale, 0, value_dim=R, values_in_keys=True,
                                         op="latent_attention")
            # (the output gate rides on the value up-projection)
            kernels.heads_linear(lat, self.v_up, out.view(T, A, dv), op="v_up",
                                 gate=row[:, Q + R + r:] if G else None)
        if G and ctx.mode == PREFILL:
            kernels.gate_sigmoid(out, row[:, Q + R + r:])
        return self.out.partial(out)


register_mixer("latent_attention", LatentAttentionMixer)
