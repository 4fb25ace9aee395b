"""Zazerax on the GPU against the plain implementation (tests/plain/zazerax_plain.py): each
mechanism alone, then whole models of three small configurations through the engine: the
stream after every layer, whole prompts, the last tokens one by one, unequal batches against
each request alone, slots and pages used again, lengths round page borders and window edges,
long decoding, greedy generation through the scheduler, and trace replay as a process.

Where random weights would hide a fault, the inputs are made so that it shows: a key just
inside and one just outside a window (or far back among hundreds) are given scores that
stand out, so an output that includes or misses the wrong one is far off.
"""
import json
import math
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from plain import zazerax_plain as P
from util import ROOT
from zazerax_util import CONFIGS, folder_for, plain_logits, tokens

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
    """Logit rows against reference rows: max error over the row's greatest logit.  32-bit:
    every row within 3e-4.  bfloat16: the test models' weights are strong, so that faults
    show, and the norm after a branch divides by the branch's own spread, which blows the
    rounding of a small branch up; so every row within 0.5 and all but one row in fifty (at
    least one) within 0.12."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    err = (got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)
    worst = f"{what}: row {err.argmax().item()} of {len(err)} off by {err.max().item():.2e}"
    if dtype == "float32":
        assert err.max().item() <= 3e-4, worst
    else:
        assert err.max().item() <= 0.5, worst
        over = int((err > 0.12).sum().item())
        assert over <= max(1, len(err) // 50), f"{what}: {over} of {len(err)} rows off; " + worst


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * std


# ------------------------------------------------------------ small mechanisms
@pytest.mark.parametrize("H", [40, 256, 1000])
@pytest.mark.parametrize("T", [3, 100])
def test_a_branch_that_reads_the_stream_itself(H, T):
    """The join without a next norm: h += N(y) and x = h rounded; and x = h[rows] alone."""
    from agave_b200 import kernels
    h0, y, w = rnd(T, H, seed=1), rnd(T, H, seed=2, std=3.0), rnd(H, seed=3) * 0.2 + 1.0
    for xd in (torch.float32, torch.bfloat16):
        h = h0.float().to(DEV)
        x = torch.empty(T, H, dtype=xd, device=DEV)
        kernels.layer_norm_join(h, y.float().to(DEV), w.float().to(DEV), None, None, None, x,
                                eps_post=1e-5)
        ref = h0 + P.layer_norm(y, w, 1e-5)
        assert rel_err(h, ref) < 1e-5
        assert rel_err(x, ref) < (1e-5 if xd == torch.float32 else 6e-3)
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
        x2 = torch.empty(2, H, dtype=xd, device=DEV)
        kernels.layer_norm_join(h, None, None, None, None, None, x2, rows=rows)
        assert torch.equal(x2.float(), h[[T - 1, 0]].to(xd).float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_squared_relu_and_products_by_head(dtype):
    from agave_b200 import kernels
    td = TD[dtype]
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    T, A, dv = 7, 3, 10
    o, g = rnd(T, A * dv, seed=1).to(td), rnd(T, A * dv + A, seed=2, std=2.0).to(td)
    for width in (A * dv, A):                       # a gate value per element, per head
        out = o.clone().to(DEV)
        gd = g.to(DEV)[:, A * dv - width + A:] if width == A else g.to(DEV)[:, :A * dv]
        kernels.gate_sigmoid(out, gd)
        gate = torch.sigmoid(gd.double().cpu())
        ref = o.double() * (gate if width == A * dv else gate.repeat_interleave(dv, dim=1))
        assert rel_err(out, ref) < tol
    z = rnd(50, 33, seed=3).to(td).to(DEV)
    ref = torch.relu(z.double().cpu()) ** 2
    kernels.relu2(z)
    assert rel_err(z, ref) < tol
    for T, A, N, K, tail in ((1, 2, 20, 12, 6), (9, 3, 5, 70, 0), (17, 8, 48, 32, 16)):
        x, w = rnd(T, A, K + tail, seed=4).to(td), rnd(A, N, K, seed=5, std=K ** -0.5).to(td)
        out = torch.zeros(T, A, N + tail + 3, dtype=td, device=DEV)
        kernels.heads_linear(x.to(DEV), w.to(DEV), out[:, :, :N + tail], tail=tail)
        ref = torch.einsum("ank,tak->tan", w.double(), x.double()[:, :, :K])
        assert rel_err(out[:, :, :N], ref) < tol
        assert torch.equal(out[:, :, N:N + tail].cpu(), x[:, :, K:])
        assert float(out[:, :, N + tail:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 5, 100, 300])
@pytest.mark.parametrize("N, K", [(40, 72), (384, 256), (1024, 512)])
def test_product_with_the_squared_relu_on_it(dtype, T, N, K):
    """The dense feed-forward's first half: act(x w^T) in one kernel, in every form the
    product takes (dot products, one-shot and cluster tiles, the prompt kernel)."""
    from agave_b200 import kernels
    td = TD[dtype]
    x, w = rnd(T, K, seed=1).to(td), rnd(N, K, seed=2, std=K ** -0.5).to(td)
    out = torch.empty(T, N, dtype=td, device=DEV)
    kernels.linear_activated(x.to(DEV), w.to(DEV), out, "relu2")
    ref = torch.relu(x.double() @ w.double().T) ** 2
    assert rel_err(out, ref) < (1e-5 if dtype == "float32" else 1.5e-2)
    assert kernels.linear_tc_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_on_the_products_by_head(dtype):
    from agave_b200 import kernels
    td = TD[dtype]
    T, A, N, K = 6, 5, 12, 40
    x, w = rnd(T, A, K, seed=4).to(td), rnd(A, N, K, seed=5, std=K ** -0.5).to(td)
    ref = torch.einsum("ank,tak->tan", w.double(), x.double())
    for width in (A, A * N):
        g = rnd(T, width, seed=6, std=2.0).to(td)
        out = torch.empty(T, A, N, dtype=td, device=DEV)
        kernels.heads_linear(x.to(DEV), w.to(DEV), out, gate=g.to(DEV))
        gate = torch.sigmoid(g.double())
        want = ref * (gate[:, :, None] if width == A else gate.view(T, A, N))
        assert rel_err(out, want) < (1e-5 if dtype == "float32" else 1.5e-2)


def test_scaled_rotation_tables():
    from agave_b200.config.base import RotarySpec, WavelengthScalingSpec
    from agave_b200.parts.rope import RotaryEmbedding
    pos = torch.tensor([0, 1, 17, 500, 4095], dtype=torch.int32, device=DEV)

    class Ctx:
        positions, n_tokens, rope_tables = pos, 5, {}

        def new(self, *shape, dtype=None):
            return torch.empty(shape, dtype=dtype, device=DEV)
    for rot in ({"base": 1000.0, "dims": 6, "scaling": {"factor": 4.0, "original": 64,
                                                        "fast": 16.0, "slow": 2.0}},
                {"base": 20000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 128,
                                                          "fast": 32.0, "slow": 1.0}},
                {"base": 300.0, "dims": 4}):
        sc = rot.get("scaling")
        part = RotaryEmbedding(RotarySpec(
            theta=rot["base"], rotary_dim=rot["dims"], scaling=None if sc is None else
            WavelengthScalingSpec(sc["factor"], sc["original"], sc["fast"], sc["slow"])),
            rot["dims"])
        part.prepare(torch.device(DEV))
        ctx = Ctx()
        ctx.rope_tables = {}
        cos, sin = part.tables(ctx)
        f, mult = P.rotary_frequencies(rot)
        a = pos.cpu().double()[:, None] * f[None, :]
        assert (cos.cpu().double() - torch.cos(a) * mult).abs().max() < 2e-7
        assert (sin.cpu().double() - torch.sin(a) * mult).abs().max() < 2e-7


class _Cache:
    """A cache of one entry and a step context over it, as a mixer finds them."""

    def __init__(self, request, lens, td):
        from agave_b200.cache import Cache
        self.cache = Cache([request], 16384, 8192, len(lens) + 2, td, torch.device(DEV))
        spare = self.cache.acquire()          # slots in another order than the batch
        self.slots = [self.cache.acquire() for _ in lens]
        self.cache.release(spare)
        for s, n in zip(self.slots, lens):
            self.cache.reserve(s, n)
        self.cache.flush()
        self.lens, self.td = lens, td

    def context(self, mode, new):
        """``new``: tokens each sequence brings (its last ones)."""
        from agave_b200.engine.batch import StepContext
        i32 = dict(dtype=torch.int32, device=DEV)
        B = len(self.lens)
        pos, seq, cu = [], [], [0]
        for b, (n, k) in enumerate(zip(self.lens, new)):
            pos += list(range(n - k, n))
            seq += [b] * k
            cu.append(cu[-1] + k)
        return StepContext(mode=mode, n_tokens=len(pos), batch=B, tokens=None,
                           positions=torch.tensor(pos, **i32), seq_index=torch.tensor(seq, **i32),
                           cu_seqlens=torch.tensor(cu, **i32),
                           slots=torch.tensor(self.slots, **i32),
                           lens=torch.tensor(self.lens, **i32), max_len=max(self.lens),
                           max_new=max(new), cache=self.cache, dtype=self.td,
                           device=torch.device(DEV))

    def row(self, b, p, pool):
        view = self.cache.kv_view(0)
        r = p % view.cap
        page = int(view.page_table[self.slots[b], r // view.page])
        return pool[page, r % view.page]

    def fill(self, b, k, v=None):
        """Positions 0..len-1 by hand (a ring keeps the last ``cap``)."""
        view = self.cache.kv_view(0)
        n = k.shape[0]
        for p in range(max(0, n - view.cap), n):
            self.row(b, p, view.k_pool).copy_(k[p].to(self.td))
            if v is not None:
                self.row(b, p, view.v_pool).copy_(v[p].to(self.td))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("partial", [False, True])
def test_norm_over_the_whole_projection_and_its_cache_rows(dtype, partial):
    """q and k normed over all heads at once, v untouched, k and v in the cache rows of the
    tokens' positions; a prompt longer than the ring keeps its last rows only."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import PREFILL
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    A, G, d, dv, window = 4, 2, 10, 14, 7
    nq, nk, nv = A * d, G * d, G * dv
    lens = [5, 70, 130]
    oc = _Cache(KVRequest(G, d, window, dv), lens, td)
    ctx = oc.context(PREFILL, lens)
    T = sum(lens)
    row = rnd(T, nq + nk + nv, seed=3, std=2.0)
    wq, wk = rnd(nq, seed=4) * 0.3 + 1.0, rnd(nk, seed=5) * 0.3 + 1.0
    out = torch.empty(T, nq + nk + nv, dtype=td, device=DEV)
    if partial:
        parts = torch.stack([row * 0.25, row * 0.75]).float().to(DEV)
        ref_in = parts.double().sum(0).cpu()
        kernels.proj_norm_store(out, nq, nk, nv, wq.float().to(DEV), wk.float().to(DEV), 1e-5,
                                ctx.positions, oc.cache.kv_view(0), ctx, partial=parts)
    else:
        out.copy_(row.to(td))
        ref_in = out.double().cpu()
        kernels.proj_norm_store(out, nq, nk, nv, wq.float().to(DEV), wk.float().to(DEV), 1e-5,
                                ctx.positions, oc.cache.kv_view(0), ctx)
    ref = torch.cat([P.rms_norm(ref_in[:, :nq], wq, 1e-5),
                     P.rms_norm(ref_in[:, nq:nq + nk], wk, 1e-5), ref_in[:, nq + nk:]], dim=1)
    tol = 1e-5 if dtype == "float32" else 6e-3
    assert rel_err(out, ref) < tol
    view = oc.cache.kv_view(0)
    assert view.cap == 64
    t0 = 0
    for b, n in enumerate(lens):
        for p in (0, n - 65, n - 64, n - 1):
            if 0 <= p and p >= n - view.cap:
                k_row = oc.row(b, p, view.k_pool).reshape(-1)
                v_row = oc.row(b, p, view.v_pool).reshape(-1)
                assert torch.equal(k_row, out[t0 + p, nq:nq + nk])
                assert torch.equal(v_row, out[t0 + p, nq + nk:])
        t0 += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("second", [False, True])
def test_latent_rows(dtype, second):
    """The latent normed, the shared key part and the queries' last dimensions rotated in
    the kind's pair layout, the gate passed through, and latent | key part in the cache."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import PREFILL
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    A, d, r, R, G = 3, 12, 6, 20, 5
    Q = 24 if second else A * (d + r)
    lens = [3, 66]
    oc = _Cache(KVRequest(1, R + r, None, value_dim=R, values_in_keys=True), lens, td)
    ctx = oc.context(PREFILL, lens)
    T = sum(lens)
    rot = {"base": 50.0, "dims": r}
    f, _ = P.rotary_frequencies(rot)
    a = ctx.positions.cpu().double()[:, None] * f[None, :]
    cos, sin = torch.cos(a).float().to(DEV), torch.sin(a).float().to(DEV)
    row = rnd(T, Q + R + r + G, seed=8, std=1.5).to(td)
    wq, wc = rnd(Q, seed=1) * 0.2 + 1.0, rnd(R, seed=2) * 0.2 + 1.0
    out = row.clone().to(DEV)
    kernels.latent_prepare(out, Q, second, A, d, r, R, G, wq.float().to(DEV) if second else None,
                           wc.float().to(DEV), 1e-5, cos, sin, second, ctx.positions,
                           oc.cache.kv_view(0), ctx)
    x = row.double()
    pos = ctx.positions.cpu()
    if second:
        ref_q = P.rms_norm(x[:, :Q], wq, 1e-5)
    else:
        q = x[:, :Q].view(T, A, d + r)
        ref_q = torch.cat([q[..., :d], P.rotate(q[..., d:], pos, rot, False)], dim=-1).reshape(T, Q)
    ref = torch.cat([ref_q, P.rms_norm(x[:, Q:Q + R], wc, 1e-5),
                     P.rotate(x[:, Q + R:Q + R + r], pos, rot, second), x[:, Q + R + r:]], dim=1)
    tol = 1e-5 if dtype == "float32" else 6e-3
    assert rel_err(out, ref) < tol
    view = oc.cache.kv_view(0)
    assert view.v_pool.data_ptr() == view.k_pool.data_ptr()
    t0 = 0
    for b, n in enumerate(lens):
        for p in (0, n - 1, min(64, n - 1)):
            assert torch.equal(oc.row(b, p, view.k_pool).reshape(-1), out[t0 + p, Q:Q + R + r])
        t0 += n
    if second:
        # the queries of the second kind are rotated after their up-projection
        hq = rnd(T, A * (d + r), seed=9).to(td)
        got = hq.clone().to(DEV)
        kernels.rotate_heads(got, A, d + r, r, cos, sin, True)
        q = hq.double().view(T, A, d + r)
        want = torch.cat([q[..., :d], P.rotate(q[..., d:], pos, rot, True)], dim=-1).reshape(T, -1)
        assert rel_err(got, want) < tol


# ------------------------------------------- windowed attention with a distance bias
def _windowed_case(T, A, G, d, dv, window, rows, seed, spikes=()):
    """q, k, v, bias with the last query's scores at chosen distances made to stand out:
    ``spikes`` = (distance, strength); the keys there point along the last query of head 0."""
    q, k, v = rnd(T, A, d, seed=seed), rnd(T, G, d, seed=seed + 1), rnd(T, G, dv, seed=seed + 2)
    bias = rnd(rows, A, seed=seed + 3)
    u = q[T - 1, 0] / q[T - 1, 0].norm()
    for dist, strength in spikes:
        if T - 1 - dist >= 0:
            k[T - 1 - dist, 0] = u * strength
    return q, k, v, bias


WINDOWED = [
    # T, A, G, d, dv, window, rows, far
    (9, 4, 2, 10, 14, 7, 6, 30.0),          # odd sizes: the one-warp kernels
    (200, 4, 1, 64, 64, 100, 12, 500.0),    # tensor-core sizes, a window that crosses pages
    (130, 3, 3, 16, 16, 64, 8, 100.0),      # a window of exactly one page
    (70, 2, 2, 24, 8, 1, 4, 40.0),          # a window of one: every token sees itself only
    (300, 6, 2, 48, 48, 129, 16, 1000.0),   # a window one longer than two pages
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, A, G, d, dv, window, rows, far", WINDOWED)
def test_prompt_attention_with_window_bias_and_one_in_the_denominator(dtype, T, A, G, d, dv,
                                                                      window, rows, far):
    """Whole prompts: the key at the window's last place counts, the one behind it does not,
    though its score is the greatest of all."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import PREFILL
    from agave_b200.parts.attention import AttentionMixer
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    scale = 1.0 / d ** 0.5
    strong = 12.0 / scale / d ** 0.5
    q, k, v, bias = _windowed_case(T, A, G, d, dv, window, rows, 5,
                                   spikes=((window - 1, strong), (window, 1.5 * strong)))
    q, k, v = q.to(td), k.to(td), v.to(td)
    ref = P.softmax_attention(q.double(), k.double(), v.double(), scale, window=window,
                              bias=bias, far=far, one_in_denominator=True)
    idx = torch.tensor(AttentionMixer.distance_rows(rows, far, min(window, math.ceil(far) + 1)))
    table = bias[idx].float().t().contiguous().to(DEV)
    lens = [T, 3]
    oc = _Cache(KVRequest(G, d, window, dv), lens, td)
    ctx = oc.context(PREFILL, lens)
    pad = lambda x: torch.cat([x.reshape(T, -1), x.reshape(T, -1)[:3]]).to(DEV)
    out = torch.empty(T + 3, A * dv, dtype=td, device=DEV)
    kernels.attention_prefill(pad(q), pad(k), pad(v), out, ctx, A, G, d, scale, window,
                              value_dim=dv, sinks=torch.zeros(A, device=DEV), dist_bias=table)
    tol = 3e-5 if dtype == "float32" else 2e-2
    assert rel_err(out[:T].view(T, A, dv), ref) < tol
    assert rel_err(out[T:].view(3, A, dv), ref[:3]) < tol       # the second sequence starts anew
    # the spiked key inside the window carries the last row of head 0; without the right edge
    # the one outside would
    if window > 1 and T > window:
        inside = v[T - window, 0].double()
        assert (ref[T - 1, 0] - inside).abs().max() < 0.05 * inside.abs().max() + 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, A, G, d, dv, window, rows, far", WINDOWED)
def test_decode_attention_with_window_bias_and_one_in_the_denominator(dtype, T, A, G, d, dv,
                                                                      window, rows, far):
    """One query per sequence against the ring: lengths below, at and above the window and
    round page borders, the same spikes at the window's edge."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import DECODE
    from agave_b200.parts.attention import AttentionMixer
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    scale = 1.0 / d ** 0.5
    strong = 12.0 / scale / d ** 0.5
    lens = sorted({1, 2, max(1, window - 1), window, window + 1, 63, 64, 65, 129, T, 2 * T + 1})
    oc = _Cache(KVRequest(G, d, window, dv), lens, td)
    idx = torch.tensor(AttentionMixer.distance_rows(rows, far, min(window, math.ceil(far) + 1)))
    qs, refs, bias = [], [], None
    for b, n in enumerate(lens):
        q, k, v, bias0 = _windowed_case(n, A, G, d, dv, window, rows, 40 + n,
                                        spikes=((window - 1, strong), (window, 1.5 * strong)))
        bias = bias0 if bias is None else bias
        q, k, v = q.to(td), k.to(td), v.to(td)
        oc.fill(b, k.to(DEV), v.to(DEV))
        lo = max(0, n - window)
        ref = P.softmax_attention(q.double()[lo:], k.double()[lo:], v.double()[lo:], scale,
                                  window=window, bias=bias, far=far, one_in_denominator=True)
        qs.append(q[n - 1])
        refs.append(ref[-1])
    ctx = oc.context(DECODE, [1] * len(lens))
    table = bias[idx].float().t().contiguous().to(DEV)
    B = len(lens)
    out = torch.empty(B, A * dv, dtype=td, device=DEV)
    kernels.attention_decode(torch.stack(qs).reshape(B, A * d).to(DEV), out, oc.cache.kv_view(0),
                             ctx, A, G, d, scale, window, value_dim=dv,
                             sinks=torch.zeros(A, device=DEV), dist_bias=table)
    assert kernels.attention_decode_status() == 0
    tol = 3e-5 if dtype == "float32" else 2e-2
    for b in range(B):
        assert rel_err(out[b].view(A, dv), refs[b]) < tol, (b, lens[b])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, A, d, dv", [(150, 2, 160, 96), (230, 2, 192, 128), (70, 3, 64, 80),
                                         (40, 2, 18, 10), (260, 2, 128, 128)])
def test_prompt_attention_with_value_heads_of_their_own_size(dtype, T, A, d, dv):
    """As many key/value heads as query heads, keys and values of different widths (what a
    latent attention's prompt step rebuilds), in every width the tensor-core forms pad to."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import PREFILL
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    scale = 1.3 / d ** 0.5
    q, k, v = (rnd(T, A, d, seed=1).to(td), rnd(T, A, d, seed=2).to(td), rnd(T, A, dv, seed=3).to(td))
    ref = P.softmax_attention(q.double(), k.double(), v.double(), scale)
    oc = _Cache(KVRequest(A, d, None, dv), [T], td)
    ctx = oc.context(PREFILL, [T])
    out = torch.empty(T, A * dv, dtype=td, device=DEV)
    kernels.attention_prefill(q.reshape(T, -1).to(DEV), k.reshape(T, -1).to(DEV),
                              v.reshape(T, -1).to(DEV), out, ctx, A, A, d, scale, 0, value_dim=dv)
    assert rel_err(out.view(T, A, dv), ref) < (3e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_decides_without_a_window(dtype):
    """No window, a distance table whose last row stands for everything beyond ``far``: key 3
    of 1,500 carries the last query (prompt kernel and decode kernel)."""
    from agave_b200 import kernels
    from agave_b200.engine.batch import DECODE, PREFILL
    from agave_b200.parts.attention import AttentionMixer
    from agave_b200.parts.base import KVRequest
    td = TD[dtype]
    T, A, G, d, rows, far = 1500, 4, 2, 32, 10, 200.0
    scale = 1.0 / d ** 0.5
    q, k, v, bias = _windowed_case(T, A, G, d, d, 0, rows, 3,
                                   spikes=((T - 4, 14.0 / scale / d ** 0.5),))
    q, k, v = q.to(td), k.to(td), v.to(td)
    s = torch.einsum("ad,jgd->ajg", q.double()[-1], k.double())
    table_rows = torch.tensor([P.distance_bucket(T - 1 - j, rows, far) for j in range(T)])
    ref = torch.zeros(A, d, dtype=torch.float64)
    for a in range(A):
        sc = s[a, :, a // (A // G)] * scale + bias[table_rows, a]
        w = torch.softmax(sc, 0)
        ref[a] = w @ v.double()[:, a // (A // G)]
    assert (ref[0] - v.double()[3, 0]).abs().max() < 0.05 * v.double()[3, 0].abs().max() + 0.05
    idx = torch.tensor(AttentionMixer.distance_rows(rows, far, math.ceil(far) + 1))
    table = bias[idx].float().t().contiguous().to(DEV)
    oc = _Cache(KVRequest(G, d, None, 0), [T], td)
    oc.fill(0, k.to(DEV), v.to(DEV))
    tol = 3e-5 if dtype == "float32" else 2e-2
    ctx = oc.context(PREFILL, [T])
    out = torch.empty(T, A * d, dtype=td, device=DEV)
    flat = lambda x: x.reshape(T, -1).to(DEV)
    kernels.attention_prefill(flat(q), flat(k), flat(v), out, ctx, A, G, d, scale, 0,
                              dist_bias=table)
    assert rel_err(out[-1].view(A, d), ref) < tol
    ctx = oc.context(DECODE, [1])
    out = torch.empty(1, A * d, dtype=td, device=DEV)
    kernels.attention_decode(flat(q)[-1:], out, oc.cache.kv_view(0), ctx, A, G, d, scale, 0,
                             dist_bias=table)
    assert rel_err(out[0].view(A, d), ref) < tol


# ------------------------------------------------------------------ whole models
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


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(name):
    """32-bit: the residual stream after each layer run against the plain model's, so that a
    fault names its layer."""
    import dataclasses
    eng, folder = engine_for(name, "float32")
    toks = tokens(25, vocab(name), 9)
    streams = []
    plain_logits(folder, toks, streams)
    model = eng.model
    for upto in range(1, len(model.spec.schedule) + 1):
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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_alone(name, dtype):
    """Every row of prompts of 1, 2, a window's and a page's length, and of 300 tokens (the
    tensor-core prompt kernels from 193 on)."""
    eng, folder = engine_for(name, dtype)
    for n in (1, 2, 7, 8, 64, 65, 300):
        toks = tokens(n, vocab(name), 20 + n)
        s = eng.acquire()
        got = eng.step([(s, toks)], [list(range(n))])
        eng.release(s)
        rows_agree(got, plain_logits(folder, toks), dtype, f"{name} {n} tokens")


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
    """The prompt's end, then the rest decoded through the cache, against the whole sequence
    at once: decoding starts after one token, inside the first window, at a page border, and
    runs a window past a long prompt."""
    eng, folder = engine_for(name, dtype)
    for n, cut in ((100, 60), (41, 1), (200, 127), (140, 64), (12, 2)):
        toks = tokens(n, vocab(name), 11 + n)
        rows_agree(alone(eng, toks, cut), plain_logits(folder, toks), dtype, f"{name} {n}/{cut}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_slots_used_again(name, dtype):
    """Requests of unequal lengths start together and are decoded together, the shorter ones
    ending earlier; then other requests take the freed slots and pages.  Every row against
    the plain model run on that request alone."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    for round_, lens in enumerate([(130, 3, 64, 1), (1, 65, 20), (63, 70, 5)]):
        seqs = [tokens(n + 6 + 3 * i, V, 50 + 10 * round_ + i) for i, n in enumerate(lens)]
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
            out = eng.step([(slots[i], [seqs[i][at[i]]]) for i in live], [[0]] * len(live))
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                at[i] += 1
                if at[i] == len(seqs[i]):
                    eng.release(slots[i])
        for i in range(len(seqs)):
            rows_agree(torch.cat(got[i]), plain_logits(folder, seqs[i]), dtype,
                       f"{name} round {round_} request {i}")


@pytest.mark.parametrize("name", NAMES)
def test_lengths_round_page_borders_and_window_edges(name):
    """32-bit: prompts that end just before, on and just after a page border and the
    windows' lengths, each followed by three decoded tokens."""
    eng, folder = engine_for(name, "float32")
    windows = {l["mixer"]["mask"]["size"] for l in CONFIGS[name]["layers"] if l["type"] == "attention"}
    edges = {63, 64, 65, 127, 128, 129}
    for w in windows:
        edges |= {max(1, w - 1), w, w + 1}
    for n in sorted(edges):
        toks = tokens(n + 3, vocab(name), n)
        ref = plain_logits(folder, toks)
        s = eng.acquire()
        got = [eng.step([(s, toks[:n])], [[0, n - 1]])]
        for p in range(n, n + 3):
            got.append(eng.step([(s, [toks[p]])], [[0]]))
        eng.release(s)
        rows_agree(torch.cat(got), ref[[0, n - 1, n, n + 1, n + 2]], "float32", f"{name} {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Z1", "Z2"])
def test_long_decoding(name, dtype):
    """300 tokens decoded after a prompt of 5: several pages, the rings wrap more than once."""
    eng, folder = engine_for(name, dtype)
    toks = tokens(305, vocab(name), 77)
    rows_agree(alone(eng, toks, 5), plain_logits(folder, toks), dtype, name)


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
    folder = folder_for("Z1", TD[dtype])
    V = vocab("Z1")
    prompts = [tokens(n, V, 900 + n) for n in (5, 66, 17, 3, 40, 21, 8)]
    wide = Engine(folder, dtype=dtype, max_tokens=4096)
    narrow = Engine(folder, dtype=dtype, max_tokens=4096, max_batch=3)
    a = wide.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    b = narrow.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    same = sum(x == y for x, y in zip(a, b))
    assert same >= (len(prompts) if dtype == "float32" else len(prompts) - 2)


def test_sampling_runs_on_this_architecture():
    eng, _ = engine_for("Z1", "bfloat16")
    V = vocab("Z1")
    kw = dict(max_new_tokens=8, temperature=0.8, top_k=20, top_p=0.9, seed=5, stop_token_ids=[])
    outs = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    again = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    assert outs == again and all(len(o) == 8 and all(0 <= t < V for t in o) for o in outs)


def test_random_weights_from_a_configuration():
    """``Engine.from_config`` with the rows of the distance tables written into the
    configuration: a model with drawn weights steps and generates."""
    import copy
    from agave_b200.engine.api import Engine
    from zazerax_util import BIAS_ROWS
    raw = copy.deepcopy(CONFIGS["Z1"])
    for i, layer in enumerate(raw["layers"]):
        if layer["type"] == "attention":
            layer["mixer"]["bias_rows"] = BIAS_ROWS["Z1"][layer.get("weights_of", i)]
    eng = Engine.from_config(raw, seed=3, max_tokens=1024)
    outs = eng.generate([tokens(9, raw["vocab"], 1)], max_new_tokens=5, stop_token_ids=[])
    assert len(outs[0]) == 5
    info = eng.model_info()
    assert info["architecture"] == "Zazerax" and info["weight_bytes"] > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype):
    name = "Z2"
    folder = folder_for(name, TD[dtype])
    V = vocab(name)
    a, b = tokens(210, V, 5), tokens(33, V, 6)
    refs = {"a": plain_logits(folder, a), "b": plain_logits(folder, b)}
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
    out = tempfile.mkdtemp(prefix="zazerax_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", out, "--max-tokens", "512"],
                       input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(4, V))
    rows_agree(got0, torch.cat([refs["a"][[0, 100, 199]], refs["b"][[29]]]), dtype, "step 0")
    rows, want = [], []
    for k in range(10):
        g = torch.from_numpy(np.fromfile(os.path.join(out, f"{k + 1}.f32"), dtype="<f4").reshape(-1, V))
        rows.append(g)
        want.append(refs["a"][200 + k:201 + k])
        if k in (0, 2):
            want.append(refs["b"][30 + k:31 + k])
    rows_agree(torch.cat(rows), torch.cat(want), dtype, "decoded")
    shutil.rmtree(out, ignore_errors=True)


def test_command_line_on_this_architecture():
    """``python -m agave_b200`` picks the model class from config.json: greedy tokens equal the
    plain model's, --model-info names the architecture, --profile lists this design's
    operations, --random-weights draws a model from a config.json that states the distance
    tables' rows."""
    import copy
    from zazerax_util import BIAS_ROWS
    name = "Z2"
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
    assert r.returncode == 0 and "Zazerax" in r.stdout, r.stderr[-2000:]
    r = run(folder, "--tokens", toks, "-n", "3", "--profile", "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr[-2000:]
    for op in ("norm", "qkv", "attention", "latent_attention", "q_absorb", "v_up", "out_proj", "up",
               "down", "lm_head", "TOTAL"):
        assert op in r.stderr, (op, r.stderr[-1500:])
    raw = copy.deepcopy(CONFIGS[name])
    for i, layer in enumerate(raw["layers"]):
        if layer["type"] == "attention":
            layer["mixer"]["bias_rows"] = BIAS_ROWS[name][layer.get("weights_of", i)]
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(raw, f)
        outs = []
        for seed in ("3", "3", "4"):
            r = run(d, "--random-weights", seed, "--tokens", toks, "-n", "5", "--json")
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(json.loads(r.stdout.strip().splitlines()[-1])["output_ids"])
        assert outs[0] == outs[1] and len(outs[0]) == 5


def test_trace_replay_counts_tokens_not_pages():
    """--max-tokens counts the tokens live requests hold, without the padding of the cache's
    pages: a dozen requests of two or three tokens each fit a budget of 36."""
    name = "Z1"
    folder = folder_for(name, torch.float32)
    V = vocab(name)
    seqs = {f"q{i}": tokens(3, V, 700 + i) for i in range(12)}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": s[:2], "want": [1]}
                                     for k, s in seqs.items()], "end": []},
             {"step": 1, "entries": [{"id": k, "tokens": s[2:], "want": [0]}
                                     for k, s in seqs.items()], "end": list(seqs)}]
    out = tempfile.mkdtemp(prefix="zazerax_trace_")
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
    shutil.rmtree(out, ignore_errors=True)


@pytest.mark.parametrize("name, room", [("Z1", 60), ("Z2", 90), ("Z3", 64)])
def test_a_cache_shorter_than_a_page_or_a_window(name, room):
    """32-bit: a cache of one or two pages.  A window that still fits a sequence keeps its
    edge although its group is no ring; a window no sequence can outgrow is none."""
    from agave_b200.engine.api import Engine
    folder = folder_for(name, torch.float32)
    eng = Engine(folder, dtype="float32", max_tokens=room, ctx_size=room, max_batch=1)
    toks = tokens(room, vocab(name), 5)
    rows_agree(alone(eng, toks, room - 15), plain_logits(folder, toks), "float32", name)
