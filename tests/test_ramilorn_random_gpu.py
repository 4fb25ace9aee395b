"""Ramilorn configurations drawn from seeds, through the engine against the plain model:
widths and head sizes that are no multiples of 8 or 16 (the kernels' general forms) beside
ones that are (the tensor-core forms), value heads of another size than the keys', every
ratio of query to kv heads, layers without feed-forward, chains of shared keys and values,
expert counts, groups and choices of all kinds.  Each configuration runs a request cut into
a prompt and decoded tokens, and an unequal batch, in 32-bit (row by row) and in bfloat16
(under the experts the library chose)."""
import json
import os
import random
import tempfile

import pytest
import torch

from ramilorn_util import config, make_tensors, mixer, moe, plain_logits, tokens
from test_ramilorn_gpu import TD, alone, chosen_experts, rows_agree

pytestmark = pytest.mark.gpu


def draw(seed):
    r = random.Random(seed)
    width = r.choice([40, 52, 64, 88, 100, 128, 136, 200, 256])
    vocab = r.choice([90, 131, 257, 500, 1000])
    n_layers = r.randint(1, 6)
    fast = r.random() < 0.4                     # sizes the tensor-core kernels take
    kinds = []
    for _ in range(r.randint(1, 2)):            # one or two kinds of attention layer
        kvh = r.choice([1, 2, 3])
        heads = kvh * r.choice([1, 2, 4])
        dim = r.choice([64, 128]) if fast else r.choice([8, 12, 16, 20, 24, 32, 40, 48, 80, 96])
        vdim = dim if r.random() < 0.6 else r.choice([8, 16, 24, 40, 64])
        kinds.append(dict(heads=heads, kv_heads=kvh, dim=dim, vdim=vdim,
                          scale=r.choice([0.5, 1.0, 1.7]) / dim ** 0.5,
                          coef=r.choice([0.0, 0.2, 0.45]), every=r.choice([1, 3, 7, 16, 50])))
    experts = r.choice([2, 4, 6, 8, 12, 16])
    count = r.choice([g for g in (1, 2, 3, 4, 6, 8) if experts % g == 0])
    keep = r.randint(1, count)
    top = r.randint(1, min(4, keep * (experts // count)))
    ff = r.choice([16, 24, 36, 64, 100])
    layers, owners = [], {}
    for i in range(n_layers):
        k = r.randrange(len(kinds))
        m = kinds[k]
        src = owners.get(k)
        share = src is not None and r.random() < 0.5
        if not share:
            owners[k] = i
        layers.append((mixer(**m, kv_from=src if share else None),
                       None if r.random() < 0.15 else moe(experts, top, ff, count, keep)))
    return config(width, vocab, layers, eps=r.choice([1e-6, 1e-5, 1e-3]),
                  mult=r.choice([0.25, 0.5, 1.0, 1.3]), cap=r.choice([8.0, 30.0, 50.0]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(12)))
def test_drawn_configuration(seed, dtype):
    from safetensors.torch import save_file
    from agave_b200.engine.api import Engine
    cfg = draw(seed)
    V = cfg["vocab"]
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in make_tensors(cfg, seed, TD[dtype]).items()},
                  os.path.join(d, "model.safetensors"))
        eng = Engine(d, dtype=dtype, max_tokens=4096)
        # a request alone: a prompt, then tokens one by one
        n, cut = 70 + 13 * (seed % 5), 40 + 9 * (seed % 4)
        toks = tokens(n, V, 40 + seed)
        with chosen_experts(eng) as rec:
            got = alone(eng, toks, cut)
        ref = plain_logits(d, toks, experts=rec.ids() if dtype == "bfloat16" else None)
        rows_agree(got, ref, dtype, f"seed {seed} alone")
        # an unequal batch, decoded together for four steps
        lens = (1, 66, 19)
        seqs = [tokens(m + 4, V, 90 + seed + i) for i, m in enumerate(lens)]
        with chosen_experts(eng) as rec:
            slots = [eng.acquire() for _ in seqs]
            steps = [[(i, m) for i, m in enumerate(lens)]]
            out = [eng.step([(sl, s[:m]) for sl, s, m in zip(slots, seqs, lens)],
                            [list(range(m)) for m in lens])]
            for k in range(4):
                steps.append([(i, 1) for i in range(len(seqs))])
                out.append(eng.step([(sl, [s[m + k]]) for sl, s, m in zip(slots, seqs, lens)],
                                    [[0]] * len(seqs)))
            for sl in slots:
                eng.release(sl)
        for i, m in enumerate(lens):
            o = sum(lens[:i])
            rows = torch.cat([out[0][o:o + m]] + [out[1 + k][i:i + 1] for k in range(4)])
            ref = plain_logits(d, seqs[i], experts=rec.ids_of(steps, i)
                               if dtype == "bfloat16" else None)
            rows_agree(rows, ref, dtype, f"seed {seed} batch request {i}")
        del eng
