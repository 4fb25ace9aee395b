"""Zazerax configurations drawn from seeds: random sizes (odd ones and those the tensor-core
kernels take), random order of the three mixers, layers without a feed-forward, layers that
run another layer's weights (also a later layer's), windows from one token to longer than the
prompt, distance tables whose far end lies inside and outside the window, scaled and unscaled
rotations for both latent kinds.  Each model runs a cut request, an unequal batch that is
decoded together, and greedy generation, in both precisions, against the plain model."""
import random
import shutil

import pytest
import torch

from test_zazerax_gpu import TD, alone, rows_agree
from zazerax_util import config, latent, plain_logits, tokens, windowed, write_folder

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    wide = seed % 2 == 1                       # every second model has tensor-core sizes
    mult = 8 if wide else 2
    width = rng.choice([64, 128, 192]) if wide else 2 * rng.randint(17, 60)
    vocab = rng.randint(60, 400)

    def one_mixer():
        kind = rng.choice(["attention", "latent", "latent2"])
        heads = rng.choice([1, 2, 3, 4, 6, 8])
        if kind == "attention":
            kv = rng.choice([g for g in (1, 2, 3, 4, 6, 8) if heads % g == 0])
            dim = mult * rng.randint(2, 8) if not wide else rng.choice([16, 32, 48, 64, 80])
            vdim = dim if rng.random() < 0.5 else mult * rng.randint(2, 8)
            window = rng.choice([1, 2, 5, 33, 64, 65, 100, 128, 500])
            rows = 2 * rng.randint(2, 10)
            far = rng.choice([rows // 2 + 1.5, 20.0, 64.0, 300.0, 1000.0])
            far = max(far, rows // 2 + 1.0)
            return windowed(heads, kv, dim, vdim, 1.3 / dim ** 0.5, window, far, rows)
        rot = 2 * rng.randint(1, 8) if not wide else rng.choice([16, 32])
        dim = mult * rng.randint(1, 6) if not wide else rng.choice([16, 32, 48])
        rank = mult * rng.randint(2, 12) if not wide else rng.choice([32, 48, 96, 112])
        vdim = mult * rng.randint(1, 8)
        scaling = None
        if rng.random() < 0.6:
            scaling = (rng.choice([2.0, 4.0, 8.0]), rng.choice([16, 64, 256]),
                       rng.choice([8.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))
        base = rng.choice([100.0, 10000.0, 500000.0])
        q_rank = None if kind == "latent" else mult * rng.randint(2, 16)
        return latent(heads, dim, rot, vdim, rank, 1.3 / (dim + rot) ** 0.5, base, scaling, q_rank)

    n = rng.randint(2, 6)
    layers = []
    for i in range(n):
        owners = [j for j, l in enumerate(layers) if l[0] != "weights_of"]
        if owners and rng.random() < 0.3:
            layers.append(("weights_of", rng.choice(owners)))
        else:
            ff = None if rng.random() < 0.25 else (mult * rng.randint(3, 20))
            layers.append((one_mixer(), ff))
    return config(width, vocab, layers, eps=rng.choice([1e-6, 1e-5, 1e-3]),
                  embed_scale=rng.choice([0.5, 1.0, 3.0]))


def move_a_borrower_first(cfg, rows):
    """The same model with its first borrowing layer moved to the front, so that it names a
    later layer."""
    layers = cfg["layers"]
    for i, l in enumerate(layers):
        if "weights_of" in l:
            order = [i] + [j for j in range(len(layers)) if j != i]
            where = {old: new for new, old in enumerate(order)}
            out = []
            for old in order:
                e = dict(layers[old])
                if "weights_of" in e:
                    e["weights_of"] = where[e["weights_of"]]
                out.append(e)
            return dict(cfg, layers=out), {where[k]: v for k, v in rows.items()}
    return cfg, rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_a_drawn_configuration(seed, dtype):
    from agave_b200.engine.api import Engine
    cfg, rows = draw(seed)
    if seed % 3 == 2:
        cfg, rows = move_a_borrower_first(cfg, rows)
    folder = write_folder(cfg, rows, seed, TD[dtype], prefix=f"zazerax_draw{seed}_")
    try:
        eng = Engine(folder, dtype=dtype, max_tokens=4096)
        V = cfg["vocab"]
        # a cut request: most of it at once, the rest token by token
        toks = tokens(150 + 7 * seed, V, seed)
        rows_agree(alone(eng, toks, len(toks) - 20), plain_logits(folder, toks), dtype,
                   f"seed {seed} alone")
        # an unequal batch decoded together; the shorter request ends first
        seqs = [tokens(n, V, 100 + seed + n) for n in (70 + seed, 9, 1 + seed)]
        lens = [len(s) - 4 - 2 * i for i, s in enumerate(seqs)]
        lens = [max(1, n) for n in lens]
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
        for sl in slots:
            eng.release(sl)
        for i, s in enumerate(seqs):
            rows_agree(torch.cat(got[i]), plain_logits(folder, s), dtype,
                       f"seed {seed} request {i}")
        # greedy generation through the scheduler
        prompts = [tokens(n, V, 500 + seed + n) for n in (3, 40)]
        outs = eng.generate(prompts, max_new_tokens=6, stop_token_ids=[])
        slack = 2e-3 if dtype == "float32" else 8e-2
        misses = 0
        for p, g in zip(prompts, outs):
            ref = plain_logits(folder, p + g)
            for k, t in enumerate(g):
                row = ref[len(p) - 1 + k]
                misses += float(row.max() - row[t]) > slack * float(row.abs().max())
        assert misses <= (0 if dtype == "float32" else 2), misses
    finally:
        shutil.rmtree(folder, ignore_errors=True)
