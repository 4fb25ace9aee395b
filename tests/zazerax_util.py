"""Small Zazerax configurations and a writer of model folders for the tests.

The writer makes every tensor under its checkpoint name from the configuration dictionary
alone (it does not ask the library which names it expects), with scales chosen so that
faults show: scores of order one to two, distance tables of order one, gates spread round
zero.
"""
import atexit
import json
import os
import shutil
import tempfile

import torch


def rotation(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        factor, original, fast, slow = scaling
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, scaling=None, q_rank=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": rotation(base, rot_dim, scaling),
         "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if q_rank is not None:
        m["q_rank"] = q_rank
    return ("latent_attention" if q_rank is None else "latent_attention_2"), m


def windowed(heads, kv_heads, dim, vdim, scale, window, bias_max, rows):
    m = {"bias_max": bias_max, "dim": dim, "heads": heads, "kv_heads": kv_heads,
         "mask": {"size": window}, "scale": scale, "vdim": vdim}
    return "attention", m, rows


def config(width, vocab, layers, eps=1e-5, embed_scale=2.0):
    """``layers``: (mixer tuple, ff or None) or ("weights_of", j)."""
    out, rows = [], {}
    for i, entry in enumerate(layers):
        if entry[0] == "weights_of":
            j = entry[1]
            e = dict(out[j])
            e["weights_of"] = j
            out.append(e)
            continue
        mix, ff = entry
        kind, m = mix[0], mix[1]
        if kind == "attention":
            rows[i] = mix[2]
        out.append({"mixer": m, "mlp": None if ff is None else {"ff": ff, "kind": "dense"},
                    "type": kind})
    cfg = {"architecture": "Zazerax", "embedding": {"scale": embed_scale}, "layers": out,
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    return cfg, rows


# Z1: small odd sizes (every kernel's general form): three kinds of mixer, a layer without a
# feed-forward, borrowed weights of two kinds, a window shorter than a page, scaled
# frequencies whose ramp lies inside the pairs.
Z1 = config(72, 210, [
    (latent(3, 12, 6, 10, 20, 0.35, 1000.0, scaling=(4.0, 64, 16.0, 2.0)), 40),
    (windowed(4, 2, 10, 14, 0.45, 7, 30, 6), None),
    (latent(2, 8, 4, 6, 18, 0.4, 300.0, q_rank=24), 56),
    ("weights_of", 1),
    ("weights_of", 0),
], eps=1e-5, embed_scale=2.5)

# Z2: the sizes that take the tensor-core kernels (head sizes 64, cache rows of 128 and 64
# values, a window that crosses pages), four query heads per kv head.
Z2 = config(128, 320, [
    (latent(4, 32, 32, 64, 96, 0.19, 20000.0, scaling=(8.0, 128, 32.0, 1.0)), 192),
    (windowed(4, 1, 64, 64, 0.19, 100, 500, 12), 128),
    (latent(8, 48, 16, 32, 48, 0.18, 100000.0, q_rank=64), 128),
    ("weights_of", 0),
    ("weights_of", 1),
    ("weights_of", 2),
], eps=1e-6, embed_scale=1.0)

# Z3: values the other two make unequal are equal here or 1: as many kv heads as query
# heads, a window of exactly one page, a window of one, one latent head, value heads wider
# than the keys, a second latent kind with scaled frequencies, no borrowed weights.
Z3 = config(96, 150, [
    (windowed(3, 3, 16, 16, 0.35, 64, 100, 8), 64),
    (latent(1, 16, 16, 48, 32, 0.25, 500.0), None),
    (windowed(2, 2, 24, 8, 0.3, 1, 40, 4), 48),
    (latent(6, 8, 8, 24, 40, 0.35, 10000.0, scaling=(2.0, 32, 8.0, 1.0), q_rank=16), 80),
], eps=3e-6, embed_scale=4.0)

CONFIGS = {"Z1": Z1[0], "Z2": Z2[0], "Z3": Z3[0]}
BIAS_ROWS = {"Z1": Z1[1], "Z2": Z2[1], "Z3": Z3[1]}


def make_tensors(cfg, rows, seed, dtype):
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    H, V = cfg["width"], cfg["vocab"]
    es = cfg["embedding"]["scale"]
    t = {"embed": rnd(V, H, std=1.0 / es), "final.norm": rnd(H, std=0.2, mean=1.0),
         "head": rnd(V, H, std=1.0 / H ** 0.5)}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p = f"l{i}."
        m = layer["mixer"]
        t[p + "norm1"] = rnd(H, std=0.2, mean=0.7)
        A, d, dv = m["heads"], m["dim"], m["vdim"]
        lin = 1.0 / H ** 0.5                                   # unit outputs from a unit stream
        if layer["type"] == "attention":
            G = m["kv_heads"]
            t[p + "mix.q"] = rnd(A * d, H, std=lin)
            t[p + "mix.k"] = rnd(G * d, H, std=lin)
            t[p + "mix.v"] = rnd(G * dv, H, std=lin)
            t[p + "mix.q.norm"] = rnd(A * d, std=0.3, mean=1.2)
            t[p + "mix.k.norm"] = rnd(G * d, std=0.3, mean=1.2)
            t[p + "mix.rel"] = rnd(rows[i], A, std=1.0)
        else:
            r, R = m["rot_dim"], m["kv_rank"]
            if layer["type"] == "latent_attention_2":
                t[p + "mix.dq"] = rnd(m["q_rank"], H, std=lin)
                t[p + "mix.dq.norm"] = rnd(m["q_rank"], std=0.2, mean=1.0)
                t[p + "mix.uq"] = rnd(A * (d + r), m["q_rank"], std=1.2 / m["q_rank"] ** 0.5)
                t[p + "mix.g"] = rnd(A, H, std=1.5 * lin)
            else:
                t[p + "mix.q"] = rnd(A * (d + r), H, std=1.2 * lin)
                t[p + "mix.g"] = rnd(A * dv, H, std=1.5 * lin)
            t[p + "mix.dkv"] = rnd(R + r, H, std=1.2 * lin)
            t[p + "mix.dkv.norm"] = rnd(R, std=0.2, mean=1.0)
            t[p + "mix.uk"] = rnd(A * d, R, std=1.2 / R ** 0.5)
            t[p + "mix.uv"] = rnd(A * dv, R, std=1.0 / R ** 0.5)
        t[p + "mix.o"] = rnd(H, A * dv, std=1.0 / (A * dv) ** 0.5)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            t[p + "norm2"] = rnd(H, std=0.2, mean=0.7)
            t[p + "mlp.up"] = rnd(ff, H, std=lin)
            t[p + "mlp.down"] = rnd(H, ff, std=1.0 / ff ** 0.5)
    return t


_FOLDERS = {}


def write_folder(cfg, rows, seed, dtype, prefix="zazerax_"):
    from safetensors.torch import save_file
    d = tempfile.mkdtemp(prefix=prefix)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in make_tensors(cfg, rows, seed, dtype).items()},
              os.path.join(d, "model.safetensors"))
    return d


def folder_for(name, dtype=torch.float32, seed=0):
    """A temporary model folder of configuration ``name`` (made once per run)."""
    key = (name, dtype, seed)
    if key not in _FOLDERS:
        _FOLDERS[key] = write_folder(CONFIGS[name], BIAS_ROWS[name], seed, dtype,
                                     prefix=f"zazerax_{name}_")
    return _FOLDERS[key]


def _cleanup():
    for d in _FOLDERS.values():
        shutil.rmtree(d, ignore_errors=True)


atexit.register(_cleanup)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(folder, toks, streams=None):
    from plain import zazerax_plain as P
    return P.forward(P.read_config(folder), P.read_weights(folder), toks, streams)
