"""Ramilorn on the GPU against the plain implementation (tests/plain/ramilorn_plain.py):
each mechanism alone, then whole models of four small configurations through the engine:
whole prompts, the last tokens one by one, unequal batches against each request alone,
slots and pages used again, lengths round page borders, long decoding across steps of the
query temperature, greedy generation, and trace replay as a separate process.

32-bit runs are compared sharply, row by row, with the plain model's own routing.  In
bfloat16 a router's choice flips where two choice scores are closer than the rounding of its
input (with random weights and several experts per token that is a few rows in a hundred
per layer), which moves that row's logits, and in a short sequence every later row's, by
far more than rounding does.  So in bfloat16 a request that runs alone is compared with the
plain model *under the experts the library chose* (recorded from its router part; the
router itself is compared on its own, on inputs without close calls), and batches and
trace replay are compared with the same request run alone through the library.
"""
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from plain import ramilorn_plain as P
from ramilorn_util import CONFIGS, folder_for, plain_logits, tokens
from util import ROOT

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel_err(got, ref):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def rows_agree(got, ref, dtype, what=""):
    """Logit rows against reference rows: max error over the row's greatest logit.

    32-bit: every row within 3e-4.  bfloat16: the test models' weights are strong, so that
    faults show, and five or six layers of bfloat16 rounding then come to several hundredths
    of the greatest logit; besides, the norm *after* a branch divides by the branch's own
    spread, so where a token's attention output is nearly nothing (the sink took the weight)
    its rounding noise is blown up.  So: every row within 0.5, and all but one row in fifty
    (at least one) within 0.1."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    err = (got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)
    worst = f"{what}: row {err.argmax().item()} of {len(err)} off by {err.max().item():.2e}"
    if dtype == "float32":
        assert err.max().item() <= 3e-4, worst
    else:
        assert err.max().item() <= 0.5, worst
        over = int((err > 0.1).sum().item())
        assert over <= max(1, len(err) // 50), f"{what}: {over} of {len(err)} rows off; " + worst


class chosen_experts:
    """Records, while it is open, the experts every routed layer of an engine chooses:
    ``.ids()`` gives {layer: [tokens seen, top]} in the order the tokens came."""

    def __init__(self, eng):
        self.eng, self.seen, self.saved = eng, {}, []

    def __enter__(self):
        # (a recorded prompt step replays without calling the parts: off while recording)
        self.graphs, self.eng.runner.use_graphs = self.eng.runner.use_graphs, False
        for call in self.eng.model.spec.schedule:
            ffn = self.eng.model.blocks[call.block].ffn
            if ffn is None:
                continue
            route = ffn.route
            self.saved.append((ffn, route))

            def recording(x, _route=route, _layer=call.block):
                ids, wts = _route(x)
                self.seen.setdefault(_layer, []).append(ids.cpu())
                return ids, wts
            ffn.route = recording
        return self

    def __exit__(self, *exc):
        self.eng.runner.use_graphs = self.graphs
        for ffn, route in self.saved:
            ffn.route = route

    def ids(self):
        return {k: torch.cat(v) for k, v in self.seen.items()}

    def ids_of(self, steps, request):
        """The same for one request of a batch: ``steps`` lists, step by step, the
        (request, tokens brought) pairs in batch order."""
        out = {}
        for layer, calls in self.seen.items():
            rows = []
            for call, step in zip(calls, steps):
                o = 0
                for r, n in step:
                    if r == request:
                        rows.append(call[o:o + n])
                    o += n
            out[layer] = torch.cat(rows)
        return out


def reference(eng, folder, toks, dtype, run):
    """The plain logits of one request: ``run()`` drives the engine over exactly these
    tokens, in order; in bfloat16 the plain model then uses the experts recorded."""
    if dtype == "float32":
        got = run()
        return got, plain_logits(folder, toks)
    with chosen_experts(eng) as rec:
        got = run()
    return got, plain_logits(folder, toks, experts=rec.ids())


# ======================================================================= mechanisms
@pytest.mark.parametrize("H", [40, 192, 1000, 5000])
def test_layer_norm_family(H):
    from agave_b200 import kernels
    g = torch.Generator().manual_seed(H)
    R = 7
    h0 = torch.randn(R, H, generator=g) * 3 + 1.5
    y = torch.randn(3, R, H, generator=g)
    w1, b1, w2, b2 = (torch.randn(H, generator=g) for _ in range(4))
    eps1, eps2, mult = 1e-3, 2e-5, 0.35
    # plain: h += mult * N(sum y); x = N(h)
    branch = P.layer_norm(y.double().sum(0), w1.double(), b1.double(), eps1)
    h_ref = h0.double() + mult * branch
    x_ref = P.layer_norm(h_ref, w2.double(), b2.double(), eps2)
    for xd in (torch.float32, torch.bfloat16):
        h = h0.to(DEV).clone()
        x = torch.empty(R, H, dtype=xd, device=DEV)
        kernels.layer_norm_join(h, y.to(DEV), w1.to(DEV), b1.to(DEV), w2.to(DEV), b2.to(DEV), x,
                                eps_post=eps1, eps_next=eps2, mult=mult)
        assert rel_err(h, h_ref) < 2e-6
        assert rel_err(x, x_ref) < (2e-5 if xd == torch.float32 else 1e-2)
    # the plain norm of gathered rows, and a bfloat16 branch without norms
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32, device=DEV)
    x = torch.empty(4, H, dtype=torch.float32, device=DEV)
    kernels.layer_norm_join(h0.to(DEV), None, None, None, w2.to(DEV), b2.to(DEV), x, eps_next=eps2,
                            rows=rows)
    assert rel_err(x, P.layer_norm(h0.double()[rows.cpu().long()], w2.double(), b2.double(), eps2)) < 2e-5
    h = h0.to(DEV).clone()
    yb = y[0].to(torch.bfloat16)
    kernels.layer_norm_join(h, yb.to(DEV), None, None, None, None, None, mult=mult)
    assert rel_err(h, h0.double() + mult * yb.double()) < 2e-6


def test_layer_norm_of_a_constant_row_is_its_bias():
    # the variance comes from the deviations: a large constant row must not leave
    # rounding noise divided by sqrt(eps)
    from agave_b200 import kernels
    H = 96
    h = torch.full((2, H), 1000.25, device=DEV)
    w = torch.ones(H, device=DEV)
    b = torch.linspace(-1, 1, H, device=DEV)
    x = torch.empty(2, H, device=DEV)
    kernels.layer_norm_join(h, None, None, None, w, b, x, eps_next=1e-6)
    assert (x - b).abs().max().item() < 1e-3


ROUTERS = [  # experts, groups, keep, top
    (8, 4, 2, 3), (6, 1, 1, 1), (4, 4, 3, 2), (12, 3, 2, 2), (10, 5, 3, 4), (64, 8, 4, 6),
    (5, 1, 1, 5),
]


@pytest.mark.parametrize("E, G, keep, top", ROUTERS)
@pytest.mark.parametrize("negative", [False, True])
def test_router_choice(E, G, keep, top, negative):
    from agave_b200 import kernels
    g = torch.Generator().manual_seed(E * 100 + top)
    T, H = 300, 48
    x = torch.randn(T, H, generator=g)
    wr = torch.randn(E, H, generator=g) * (2.0 / H ** 0.5)
    # all choice scores negative: a dropped group must not look better than a kept one
    corr = torch.randn(E, generator=g) * 0.3 - (2.5 if negative else 0.0)
    r = {"experts": E, "top": top, "groups": {"count": G, "keep": keep}}
    ids_ref, wt_ref = P.route(x.double(), wr.double(), corr.double(), r)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(x.to(DEV), wr.to(DEV), corr.to(DEV), G, keep, top, ids, wts)
    got = ids.cpu().long()
    # rows whose decision is a close call in 32-bit are left out (there are next to none)
    same = (got.sort(dim=1).values == ids_ref.sort(dim=1).values).all(dim=1)
    assert same.float().mean().item() > 0.99
    order = (got == ids_ref).all(dim=1)
    assert order[same].float().mean().item() > 0.98          # best first, as the plain top-k
    sel = same & order
    assert torch.allclose(wts.cpu().double()[sel], wt_ref[sel], atol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E, G, keep, top", [(8, 4, 2, 3), (6, 1, 1, 1), (12, 3, 2, 2)])
@pytest.mark.parametrize("T", [1, 5, 200])
def test_routed_feed_forward(dtype, E, G, keep, top, T):
    from agave_b200.config import RoutedFeedForwardSpec
    from agave_b200.parts import RoutedFeedForward
    td = TD[dtype]
    H, ff = 72, 40
    g = torch.Generator().manual_seed(T + E)
    spec = RoutedFeedForwardSpec(n_experts=E, top=top, intermediate_size=ff, n_groups=G,
                                 keep_groups=keep)
    t = {"router.weight": torch.randn(E, H, generator=g) * (2.0 / H ** 0.5),
         "router.correction": torch.randn(E, generator=g) * 0.3}
    w = {"router": t["router.weight"], "correction": t["router.correction"]}
    for e in range(E):
        for n, shape, std in (("gate", (ff, H), H ** -0.5), ("up", (ff, H), H ** -0.5),
                              ("down", (H, ff), ff ** -0.5)):
            t[f"experts.{e}.{n}_proj.weight"] = torch.randn(*shape, generator=g) * std
            w[f"e{e}.{n}"] = t[f"experts.{e}.{n}_proj.weight"]
    t = {k: (v.to(td) if v.dim() == 2 else v) for k, v in t.items()}
    w = {k: (v.to(td) if v.dim() == 2 else v).double() for k, v in w.items()}
    part = RoutedFeedForward(spec, H, td, torch.device(DEV))
    part.load(t, td, torch.device(DEV))
    x = (torch.randn(T, H, generator=g)).to(td)
    y = part.forward(x.to(DEV), None)
    assert y.shape == (top, T, H) and y.dtype == torch.float32
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": G, "keep": keep}}}
    ref = P.moe(x.double(), w, "", mlp)
    got = y.sum(0).double().cpu()
    err = (got - ref).abs().amax(dim=1) / ref.abs().amax()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (err > tol).sum().item() <= (0 if dtype == "float32" else max(1, T // 20)), err.max()


@pytest.mark.parametrize("T", [3, 130, 700])
@pytest.mark.parametrize("H, ff, E, top", [(200, 328, 5, 2), (64, 136, 3, 3), (264, 64, 16, 4)])
def test_experts_on_the_tensor_cores(T, H, ff, E, top):
    """bfloat16 with sizes that span several weight tiles and leave tails of K and N: the
    tcgen05 grouped products against the plain experts under the library's own routing, and
    against the dot-product form bit for bit in what they choose."""
    from agave_b200 import kernels
    from agave_b200.config import RoutedFeedForwardSpec
    from agave_b200.parts import RoutedFeedForward
    td = torch.bfloat16
    g = torch.Generator().manual_seed(T + H)
    spec = RoutedFeedForwardSpec(n_experts=E, top=top, intermediate_size=ff)
    t = {"router.weight": (torch.randn(E, H, generator=g) * (2.0 / H ** 0.5)).to(td),
         "router.correction": torch.randn(E, generator=g) * 0.3}
    for e in range(E):
        t[f"experts.{e}.gate_proj.weight"] = (torch.randn(ff, H, generator=g) * H ** -0.5).to(td)
        t[f"experts.{e}.up_proj.weight"] = (torch.randn(ff, H, generator=g) * H ** -0.5).to(td)
        t[f"experts.{e}.down_proj.weight"] = (torch.randn(H, ff, generator=g) * ff ** -0.5).to(td)
    part = RoutedFeedForward(spec, H, td, torch.device(DEV))
    part.load(t, td, torch.device(DEV))
    x = torch.randn(T, H, generator=g).to(td).to(DEV)
    assert kernels.moe_grouped_tc_supported(x, part.w_gate)
    y = part.forward(x, None).sum(0).double().cpu()
    assert kernels.moe_tc_status() == 0
    ids, wts = part.route(x)
    ids, wts = ids.cpu().long(), wts.cpu().double()
    ref = torch.zeros(T, H, dtype=torch.float64)
    w = {f"e{e}.{n}": t[f"experts.{e}.{n}_proj.weight"].double() for e in range(E)
         for n in ("gate", "up", "down")}
    for e in range(E):
        rows, slot = (ids == e).nonzero(as_tuple=True)
        if len(rows):
            ref[rows] += wts[rows, slot][:, None] * P.expert(x.double().cpu()[rows], w, f"e{e}.")
    assert rel_err(y, ref) < 1.5e-2
    # the dot-product form of the same step
    plan = kernels.moe_plan(*part.route(x), E)
    z = torch.empty(plan.rows, ff, dtype=td, device=DEV)
    y2 = torch.empty(top, T, H, dtype=torch.float32, device=DEV)
    kernels.moe_grouped(x, part.w_gate, z, plan, w2=part.w_up, activation="silu", gather=True)
    kernels.moe_grouped(z, part.w_down, y2.view(top * T, H), plan, scatter=True)
    assert rel_err(y2.sum(0), ref) < 1.5e-2


def _sink_case(T, A, G, d, dv, seed, spike=None):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, A, d, generator=g)
    k = torch.randn(T, G, d, generator=g)
    v = torch.randn(T, G, dv, generator=g)
    sink = torch.randn(A, generator=g) + 2.0           # strong enough to show if left out
    if spike is not None:
        # one far key stands out for the last query: its score tops every other by far
        j, t, m = spike
        k[j] = 0
        k[j, :, 0] = m
        q[t] = 0
        q[t, :, 0] = m
    return q, k, v, sink


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, A, G, d, dv", [
    (50, 4, 2, 16, 16), (70, 6, 6, 32, 48), (33, 4, 2, 48, 24),        # general kernel
    (130, 4, 1, 64, 64), (260, 4, 1, 64, 64), (300, 2, 1, 128, 128),   # tensor-core kernels
    (400, 4, 2, 80, 80),
])
def test_prompt_attention_with_sinks(dtype, T, A, G, d, dv):
    from agave_b200 import kernels
    from agave_b200.engine.batch import PREFILL, StepContext
    td = TD[dtype]
    scale = 0.9 / d ** 0.5
    q, k, v, sink = _sink_case(T, A, G, d, dv, T, spike=(3, T - 1, (32 / scale) ** 0.5))
    q, k, v = q.to(td), k.to(td), v.to(td)
    ref = P.sink_attention(q.double(), k.double(), v.double(), sink.double(), scale)
    # two sequences in one step: the case twice, the second cut short
    T2 = T // 2
    qkv = torch.cat([torch.cat([q, q[:T2]]).reshape(T + T2, -1),
                     torch.cat([k, k[:T2]]).reshape(T + T2, -1),
                     torch.cat([v, v[:T2]]).reshape(T + T2, -1)], dim=1).to(DEV).contiguous()
    qv, kv_, vv = qkv[:, :A * d], qkv[:, A * d:(A + G) * d], qkv[:, (A + G) * d:]
    i32 = dict(dtype=torch.int32, device=DEV)
    ctx = StepContext(mode=PREFILL, n_tokens=T + T2, batch=2, tokens=None,
                      positions=torch.cat([torch.arange(T), torch.arange(T2)]).to(**i32),
                      seq_index=torch.cat([torch.zeros(T), torch.ones(T2)]).to(**i32),
                      cu_seqlens=torch.tensor([0, T, T + T2], **i32), slots=None, lens=None,
                      max_len=T, max_new=T, cache=None, dtype=td, device=torch.device(DEV))
    out = torch.empty(T + T2, A * dv, dtype=td, device=DEV)
    kernels.attention_prefill(qv, kv_, vv, out, ctx, A, G, d, scale, 0, value_dim=dv,
                              sinks=sink.to(DEV))
    assert kernels.attention_tc_status() == 0
    tol = 3e-5 if dtype == "float32" else 2e-2
    assert rel_err(out[:T].view(T, A, dv), ref) < tol
    assert rel_err(out[T:].view(T2, A, dv), ref[:T2]) < tol
    # the far key: the last query's output is that key's value, less the sink's share
    if dtype == "float32":
        share = 1 / (1 + torch.exp(sink.double() - 32.0))
        want = v.double()[3].repeat_interleave(A // G, dim=0) * share[:, None]
        assert (out[T - 1].view(A, dv).double().cpu() - want).abs().max() < 1e-2


class _OneLayerCache:
    """A cache of one entry filled by hand, as a decode step finds it."""

    def __init__(self, lens, G, d, dv, td, shuffle_seed):
        from agave_b200.cache import Cache
        from agave_b200.parts.base import KVRequest
        self.cache = Cache([KVRequest(G, d, None, 0 if dv == d else dv)], 16384, 8192, len(lens) + 2,
                           td, torch.device(DEV))
        # slots taken in another order than the batch, after one was freed again
        spare = self.cache.acquire()
        self.slots = [self.cache.acquire() for _ in lens]
        self.cache.release(spare)
        for s, n in zip(self.slots, lens):
            self.cache.reserve(s, n)
        self.cache.flush()

    def fill(self, b, k, v):
        view = self.cache.kv_view(0)
        table = view.page_table[self.slots[b]].cpu()
        for p in range(k.shape[0]):
            page = int(table[p // view.page])
            view.k_pool[page, p % view.page] = k[p].to(view.k_pool.dtype).to(DEV)
            view.v_pool[page, p % view.page] = v[p].to(view.v_pool.dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("A, G, d, dv", [(4, 2, 16, 16), (6, 6, 32, 48), (4, 1, 64, 64),
                                         (2, 1, 128, 128), (8, 2, 80, 80)])
def test_decode_attention_with_sinks(dtype, A, G, d, dv):
    """One query per sequence against the paged cache: lengths of one key, round page and
    chunk borders, and thousands of keys with one far key that decides the result."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import DECODE, StepContext
    td = TD[dtype]
    lens = [1, 2, 63, 64, 65, 129, 700, 3000]
    scale = 0.9 / d ** 0.5
    oc = _OneLayerCache(lens, G, d, dv, td, 0)
    qs, refs = [], []
    sink = None
    for b, n in enumerate(lens):
        q, k, v, sink0 = _sink_case(n, A, G, d, dv, 1000 + n, spike=(min(5, n - 1), n - 1, (32 / scale) ** 0.5))
        sink = sink0 if sink is None else sink            # one layer: one set of sinks
        q, k, v = q.to(td), k.to(td), v.to(td)
        oc.fill(b, k, v)
        qs.append(q[n - 1])
        last = _last_row(q.double()[n - 1], k.double(), v.double(), sink.double(), scale)
        if n <= 129:
            # (the last row of the plain causal attention over the whole sequence)
            full = P.sink_attention(q.double(), k.double(), v.double(), sink.double(), scale)
            assert torch.allclose(full[n - 1], last, atol=1e-12)
        refs.append(last)
    B = len(lens)
    i32 = dict(dtype=torch.int32, device=DEV)
    ctx = StepContext(mode=DECODE, n_tokens=B, batch=B, tokens=None,
                      positions=torch.tensor([n - 1 for n in lens], **i32),
                      seq_index=torch.arange(B, **i32), cu_seqlens=torch.arange(B + 1, **i32),
                      slots=torch.tensor(oc.slots, **i32), lens=torch.tensor(lens, **i32),
                      max_len=max(lens), max_new=1, cache=oc.cache, dtype=td,
                      device=torch.device(DEV))
    qd = torch.stack(qs).reshape(B, A * d).to(DEV)
    out = torch.empty(B, A * dv, dtype=td, device=DEV)
    kernels.attention_decode(qd, out, oc.cache.kv_view(0), ctx, A, G, d, scale, 0, value_dim=dv,
                             sinks=sink.to(DEV))
    assert kernels.attention_decode_status() == 0
    tol = 3e-5 if dtype == "float32" else 2e-2
    for b in range(B):
        assert rel_err(out[b].view(A, dv), refs[b]) < tol, (b, lens[b])


def _last_row(q, k, v, sink, scale):
    """The plain attention of one query over all keys given (vectorised over keys)."""
    A, G = q.shape[0], k.shape[1]
    out = torch.zeros(A, v.shape[2], dtype=torch.float64)
    for a in range(A):
        g = a // (A // G)
        s = (k[:, g] @ q[a]) * scale
        m = torch.maximum(s.max(), sink[a])
        e = torch.exp(s - m)
        out[a] = (e / (e.sum() + torch.exp(sink[a] - m))) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("A, G, d, dv", [(4, 2, 16, 16), (3, 3, 32, 48), (4, 1, 64, 64)])
def test_query_temperature_and_cache_store(dtype, A, G, d, dv):
    """q | k | v rows through the store kernel: q heads take the temperature of their
    position (steps at multiples of the period), k and v reach the cache rows of their
    positions unchanged, also when the value heads have a size of their own."""
    from agave_b200 import kernels
    td = TD[dtype]
    coef, every = 0.37, 4
    lens = [11, 70]
    T = sum(lens)
    g = torch.Generator().manual_seed(d)
    width = (A + G) * d + G * dv
    part = torch.randn(3, T, width, generator=g)             # three partial sums
    full = part.double().sum(0)
    oc = _OneLayerCache(lens, G, d, dv, td, 1)
    view = oc.cache.kv_view(0)
    i32 = dict(dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(n) for n in lens])
    seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)])
    qkv = torch.empty(T, width, dtype=td, device=DEV)
    kernels.qk_norm_rope_store(qkv, A, G, d, None, None, 0.0, None, None, 0, pos.to(**i32),
                               view.k_pool, view.v_pool, view.page_table,
                               torch.tensor(oc.slots, **i32), torch.tensor(lens, **i32),
                               seq.to(**i32), view.page, view.cap, partial=part.to(DEV),
                               value_dim=dv, q_temp=(coef, every))
    tau = torch.cat([P.query_temperature(n, coef, every, torch.float64) for n in lens])
    want = full.clone()
    want[:, :A * d] *= tau[:, None]
    tol = 1e-6 if dtype == "float32" else 8e-3
    assert rel_err(qkv, want) < tol
    assert tau[2] == 1.0 and tau[3] > 1.0 and tau[7] > tau[6]       # the steps are where they belong
    t0 = 0
    for b, n in enumerate(lens):
        table = view.page_table[oc.slots[b]].cpu()
        for p in (0, n - 1, min(n - 1, 63), min(n - 1, 64)):
            page = int(table[p // view.page])
            krow = view.k_pool[page, p % view.page].reshape(-1)
            vrow = view.v_pool[page, p % view.page].reshape(-1)
            assert rel_err(krow, full[t0 + p, A * d:(A + G) * d]) < tol
            assert rel_err(vrow, full[t0 + p, (A + G) * d:]) < tol
        t0 += n
    # queries alone (a layer without keys and values of its own)
    q_only = torch.empty(T, A * d, dtype=td, device=DEV)
    kernels.qk_norm_rope_store(q_only, A, 0, d, None, None, 0.0, None, None, 0, pos.to(**i32),
                               partial=part[:, :, :A * d].contiguous().to(DEV), value_dim=dv,
                               q_temp=(coef, every))
    assert rel_err(q_only, want[:, :A * d]) < tol


def test_soft_cap():
    from agave_b200 import kernels
    z = torch.linspace(-200, 200, 4001, device=DEV).reshape(1, -1).contiguous()
    ref = P.soft_cap(z.double().cpu(), 30.0)
    kernels.soft_cap(z, 30.0)
    assert rel_err(z, ref) < 1e-6


# ======================================================================= whole models
_ENGINES = {}


def engine_for(name, dtype, max_tokens=8192):
    key = (name, dtype)
    if key not in _ENGINES:
        from agave_b200.engine.api import Engine
        folder = folder_for(name, TD[dtype])
        _ENGINES[key] = (Engine(folder, dtype=dtype, max_tokens=max_tokens), folder)
    return _ENGINES[key]


def vocab(name):
    return CONFIGS[name]["vocab"]


NAMES = sorted(CONFIGS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_alone(name, dtype):
    eng, folder = engine_for(name, dtype)
    for n, seed in ((1, 1), (2, 2), (9, 3), (40, 4), (230, 5)):
        toks = tokens(n, vocab(name), seed)

        def run():
            s = eng.acquire()
            got = eng.step([(s, toks)], [list(range(n))])
            eng.release(s)
            return got
        got, ref = reference(eng, folder, toks, dtype, run)
        rows_agree(got, ref, dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(name):
    """32-bit: the residual stream after each layer against the plain model's, so that a
    fault names its layer."""
    eng, folder = engine_for(name, "float32")
    from agave_b200.engine.batch import PREFILL
    toks = tokens(25, vocab(name), 9)
    streams = []
    plain_logits(folder, toks, streams)
    model = eng.model
    spec = model.spec
    for upto in range(1, len(spec.schedule) + 1):
        import dataclasses
        s = eng.acquire()
        ctx = eng.runner.context([(s, toks)])
        keep = model.spec
        model.spec = dataclasses.replace(keep, schedule=keep.schedule[:upto])
        try:
            h = model.hidden_states(ctx)
        finally:
            model.spec = keep
        eng.runner.cache.trim(s)
        eng.release(s)
        assert rel_err(h, streams[upto - 1]) < 2e-5, f"layer {upto - 1}"


def alone(eng, toks, cut):
    """A request by itself: ``cut`` tokens as the prompt, the rest one by one; all rows."""
    s = eng.acquire()
    got = [eng.step([(s, toks[:cut])], [list(range(cut))])]
    for p in range(cut, len(toks)):
        got.append(eng.step([(s, [toks[p]])], [[0]]))
    eng.release(s)
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_tokens_one_by_one(name, dtype):
    """The prompt's end, then 40 tokens decoded through the cache, against the whole
    sequence at once: decoding crosses a page border and steps of the temperature."""
    eng, folder = engine_for(name, dtype)
    for n, cut in ((100, 60), (41, 1), (200, 127)):
        toks = tokens(n, vocab(name), 11 + n)
        got, ref = reference(eng, folder, toks, dtype, lambda: alone(eng, toks, cut))
        rows_agree(got, ref, dtype, f"{name} {n}/{cut}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_slots_used_again(name, dtype):
    """Three requests of unequal lengths start together and are decoded together, the
    shorter ones ending earlier; then other requests take the freed slots and pages.
    Every row is compared with the plain model run on that request alone (in bfloat16 under
    the experts the batch run chose for that request's tokens)."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    for round_, lens in enumerate([(130, 3, 64), (1, 65, 20), (63, 70, 5)]):
        seqs = [tokens(n + 6 + 3 * i, V, 50 + 10 * round_ + i) for i, n in enumerate(lens)]
        rec = chosen_experts(eng)
        rec.__enter__()
        steps = [[(i, n) for i, n in enumerate(lens)]]
        slots = [eng.acquire() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)],
                       [list(range(n)) for n in lens])
        o = 0
        for i, n in enumerate(lens):
            got[i].append(out[o:o + n])
            o += n
        at = list(lens)
        while any(a < len(s) for a, s in zip(at, seqs)):
            live = [i for i in range(len(seqs)) if at[i] < len(seqs[i])]
            steps.append([(i, 1) for i in live])
            out = eng.step([(slots[i], [seqs[i][at[i]]]) for i in live], [[0]] * len(live))
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                at[i] += 1
                if at[i] == len(seqs[i]):
                    eng.release(slots[i])
        rec.__exit__()
        for i in range(len(seqs)):
            ref = plain_logits(folder, seqs[i], experts=None if dtype == "float32"
                               else rec.ids_of(steps, i))
            rows_agree(torch.cat(got[i]), ref, dtype, f"{name} round {round_} request {i}")


@pytest.mark.parametrize("name", ["R1", "R3"])
def test_lengths_round_page_borders(name):
    """32-bit: prompts that end just before, on and just after a page border, each
    followed by three decoded tokens."""
    eng, folder = engine_for(name, "float32")
    for n in (63, 64, 65, 127, 128, 129):
        toks = tokens(n + 3, vocab(name), n)
        ref = plain_logits(folder, toks)
        s = eng.acquire()
        got = [eng.step([(s, toks[:n])], [[0, n - 1]])]
        for p in range(n, n + 3):
            got.append(eng.step([(s, [toks[p]])], [[0]]))
        eng.release(s)
        rows_agree(torch.cat(got), ref[[0, n - 1, n, n + 1, n + 2]], "float32", f"{name} {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R2", "R3"])
def test_long_decoding(name, dtype):
    """300 tokens decoded after a prompt of 5: several pages, many temperature steps."""
    eng, folder = engine_for(name, dtype)
    toks = tokens(305, vocab(name), 77)
    got, ref = reference(eng, folder, toks, dtype, lambda: alone(eng, toks, 5))
    rows_agree(got, ref, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name, dtype):
    """``Engine.generate`` (scheduler, CUDA graphs, the arg max in the head's epilogue): every
    generated token is the plain model's best, or within rounding of it."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    prompts = [tokens(n, V, 300 + n) for n in (4, 37, 70, 9, 130)]
    outs = eng.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    slack = 2e-3 if dtype == "float32" else 8e-2
    misses = 0
    for p, g in zip(prompts, outs):
        assert len(g) == 12
        ref = plain_logits(folder, p + g)
        for k, t in enumerate(g):
            row = ref[len(p) - 1 + k]
            if float(row.max() - row[t]) > slack * float(row.abs().max()):
                misses += 1
    assert misses <= (0 if dtype == "float32" else 3), misses


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_in_batches_of_the_slot_limit(dtype):
    """More prompts than slots: the scheduler cuts them into batches and uses slots again;
    the tokens are the same as with room for all."""
    from agave_b200.engine.api import Engine
    folder = folder_for("R1", TD[dtype])
    V = vocab("R1")
    prompts = [tokens(n, V, 900 + n) for n in (5, 66, 17, 3, 40, 21, 8)]
    wide = Engine(folder, dtype=dtype, max_tokens=4096)
    narrow = Engine(folder, dtype=dtype, max_tokens=4096, max_batch=3)
    a = wide.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    b = narrow.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    same = sum(x == y for x, y in zip(a, b))
    assert same >= (len(prompts) if dtype == "float32" else len(prompts) - 2)


def test_sampling_runs_on_this_architecture():
    eng, _ = engine_for("R1", "bfloat16")
    V = vocab("R1")
    outs = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], max_new_tokens=8, temperature=0.8,
                        top_k=20, top_p=0.9, seed=5, stop_token_ids=[])
    again = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], max_new_tokens=8, temperature=0.8,
                         top_k=20, top_p=0.9, seed=5, stop_token_ids=[])
    assert outs == again and all(len(o) == 8 and all(0 <= t < V for t in o) for o in outs)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype):
    name = "R3"
    folder = folder_for(name, TD[dtype])
    V = vocab(name)
    a, b = tokens(210, V, 5), tokens(33, V, 6)
    if dtype == "float32":
        refs = {"a": plain_logits(folder, a), "b": plain_logits(folder, b)}
    else:
        eng, _ = engine_for(name, dtype)
        refs = {"a": alone(eng, a, 200).cpu(), "b": alone(eng, b, 30).cpu()}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:200], "want": [0, 100, 199]},
                                     {"id": "b", "tokens": b[:30], "want": [29]}], "end": []}]
    for k in range(10):
        ent, end = [{"id": "a", "tokens": [a[200 + k]], "want": [0]}], []
        if k < 3:
            ent.append({"id": "b", "tokens": [b[30 + k]], "want": [0] if k != 1 else []})
            if k == 2:
                end.append("b")
        if k == 9:
            end.append("a")
        steps.append({"step": k + 1, "entries": ent, "end": end})
    out = tempfile.mkdtemp(prefix="ramilorn_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", out, "--max-tokens", "512"],
                       input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(4, V))
    rows_agree(got0, torch.cat([refs["a"][[0, 100, 199]], refs["b"][[29]]]), dtype, "step 0")
    rows = []
    want = []
    for k in range(10):
        g = torch.from_numpy(np.fromfile(os.path.join(out, f"{k + 1}.f32"), dtype="<f4").reshape(-1, V))
        rows.append(g)
        want.append(refs["a"][200 + k:201 + k])
        if k in (0, 2):
            want.append(refs["b"][30 + k:31 + k])
    rows_agree(torch.cat(rows), torch.cat(want), dtype, "decoded")
    import shutil
    shutil.rmtree(out, ignore_errors=True)


def test_trace_replay_counts_tokens_not_pages():
    """--max-tokens counts the tokens live requests hold, without the padding of the
    cache's pages: a dozen requests of two or three tokens each fit a budget of 36."""
    name = "R1"
    folder = folder_for(name, torch.float32)
    V = vocab(name)
    seqs = {f"q{i}": tokens(3, V, 700 + i) for i in range(12)}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": s[:2], "want": [1]}
                                     for k, s in seqs.items()], "end": []},
             {"step": 1, "entries": [{"id": k, "tokens": s[2:], "want": [0]}
                                     for k, s in seqs.items()], "end": list(seqs)}]
    out = tempfile.mkdtemp(prefix="ramilorn_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", "float32", "--out", out, "--max-tokens", "36"],
                       input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    refs = [plain_logits(folder, s) for s in seqs.values()]
    for step, row in ((0, 1), (1, 2)):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")
                               .reshape(12, V))
        rows_agree(got, torch.stack([ref[row] for ref in refs]), "float32", f"step {step}")
    import shutil
    shutil.rmtree(out, ignore_errors=True)


def test_command_line_on_this_architecture():
    """``python -m agave_b200`` picks the model class from config.json: greedy tokens equal the
    plain model's, --model-info names the architecture, --profile lists the routed
    feed-forward's operations, --random-weights draws a model from config.json alone."""
    name = "R3"
    folder = folder_for(name, torch.float32)
    V = vocab(name)
    prompt = tokens(9, V, 31)

    def run(*args):
        env = dict(os.environ)
        env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
        return subprocess.run([sys.executable, "-m", "agave_b200", *args], capture_output=True,
                              text=True, timeout=900, env=env, cwd=ROOT)
    toks = ",".join(str(t) for t in prompt)
    r = run(folder, "--tokens", toks, "-n", "6", "--json", "--dtype", "float32")
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])["output_ids"]
    assert len(out) == 6
    ref = plain_logits(folder, prompt + out)
    for k, t in enumerate(out):
        row = ref[len(prompt) - 1 + k]
        assert float(row.max() - row[t]) <= 2e-3 * float(row.abs().max()), (k, t)
    r = run(folder, "--model-info", "--json")
    assert r.returncode == 0 and "Ramilorn" in r.stdout, r.stderr[-2000:]
    r = run(folder, "--tokens", toks, "-n", "3", "--profile", "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr[-2000:]
    for op in ("norm", "qkv", "attention", "out_proj", "router", "experts_gate_up", "experts_down",
               "lm_head", "soft_cap", "TOTAL"):
        assert op in r.stderr, (op, r.stderr[-1500:])
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        outs = []
        for seed in ("3", "3", "4"):
            r = run(d, "--random-weights", seed, "--tokens", toks, "-n", "5", "--json")
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(json.loads(r.stdout.strip().splitlines()[-1])["output_ids"])
        assert outs[0] == outs[1] and len(outs[0]) == 5
