"""Small Ramilorn configurations and a writer of model folders for the tests.

The writer makes every tensor under its checkpoint name from the configuration
dictionary alone (it does not ask the library which names it expects), with scales
chosen so that faults show: queries and keys large enough for scores of order one,
sinks of order one, router logits spread wide enough that choices are not close calls.
"""
import json
import os
import shutil
import tempfile

import torch


def mixer(heads, kv_heads, dim, vdim, scale, coef, every, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads,
         "q_temp": {"coef": coef, "every": every}, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, count, keep):
    return {"expert": {"ff": ff}, "kind": "moe",
            "router": {"experts": experts, "groups": {"count": count, "keep": keep}, "top": top}}


def config(width, vocab, layers, eps=1e-5, mult=0.5, cap=30.0):
    return {"architecture": "Ramilorn",
            "layers": [{"mixer": m, "mlp": f, "type": "attention"} for m, f in layers],
            "logit_softcap": cap, "norm": {"eps": eps}, "residual_mult": mult,
            "vocab": vocab, "width": width}


# R1: small odd sizes (every kernel's general form): grouped kv heads, a layer without a
# feed-forward, two layers that attend to an earlier layer's keys and values.
_m1 = dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, coef=0.4, every=8)
R1 = config(72, 200, [
    (mixer(**_m1), moe(8, 3, 40, 4, 2)),
    (mixer(**_m1), moe(8, 3, 40, 4, 2)),
    (mixer(**_m1, kv_from=1), moe(8, 3, 40, 4, 2)),
    (mixer(**_m1), None),
    (mixer(**_m1, kv_from=3), moe(8, 3, 40, 4, 2)),
], eps=1e-5, mult=0.7, cap=20.0)

# R2: value heads wider than the keys', as many kv heads as query heads, one expert per
# token, no groups to speak of, a short temperature period.
_m2 = dict(heads=6, kv_heads=6, dim=32, vdim=48, scale=0.2, coef=0.25, every=5)
R2 = config(96, 150, [
    (mixer(**_m2), moe(6, 1, 56, 1, 1)),
    (mixer(**_m2), moe(6, 1, 56, 1, 1)),
    (mixer(**_m2, kv_from=0), moe(6, 1, 56, 1, 1)),
], eps=3e-6, mult=1.0, cap=12.0)

# R3: head size 64 and four query heads per kv head: the sizes that take the tensor-core
# attention kernels and the decode kernel that forms q, k and v itself; groups of one
# expert each.
_m3 = dict(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.11, coef=0.3, every=16)
R3 = config(128, 320, [
    (mixer(**_m3), moe(4, 2, 64, 4, 3)),
    (mixer(**_m3, kv_from=0), moe(4, 2, 64, 4, 3)),
    (mixer(**_m3), moe(4, 2, 64, 4, 3)),
    (mixer(**_m3, kv_from=2), moe(4, 2, 64, 4, 3)),
], eps=1e-5, mult=0.4, cap=25.0)

# R4: narrower values than keys, head size 128 keys, layers differing in every size.
R4 = config(160, 260, [
    (mixer(2, 1, 128, 128, 0.08, 0.5, 32), moe(10, 4, 48, 5, 3)),
    (mixer(4, 2, 48, 24, 0.15, 0.2, 7), moe(4, 2, 96, 2, 2)),
    (mixer(4, 2, 48, 24, 0.15, 0.2, 7, kv_from=1), None),
], eps=1e-4, mult=0.9, cap=40.0)

CONFIGS = {"R1": R1, "R2": R2, "R3": R3, "R4": R4}


def make_tensors(cfg, seed, dtype):
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    H, V = cfg["width"], cfg["vocab"]
    t = {"embed": rnd(V, H, std=0.5), "final.norm": rnd(H, std=0.2, mean=1.0),
         "final.norm.b": rnd(H, std=0.2)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] is not None else [])
        for n in names:
            t[p + n] = rnd(H, std=0.2, mean=1.0)
            t[p + n + ".b"] = rnd(H, std=0.2)
        A, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        qk = (1.5 / (m["scale"] * d ** 0.5)) ** 0.5 / H ** 0.5      # scores of order 1.5
        t[p + "mix.q"] = rnd(A * d, H, std=qk)
        if m.get("kv_from") is None:
            t[p + "mix.k"] = rnd(G * d, H, std=qk)
            t[p + "mix.v"] = rnd(G * dv, H, std=1.0 / H ** 0.5)
        t[p + "mix.o"] = rnd(H, A * dv, std=1.0 / (A * dv) ** 0.5)
        t[p + "mix.sink"] = rnd(A, std=1.0, mean=0.5)
        f = layer["mlp"]
        if f is not None:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            t[p + "mlp.router"] = rnd(E, H, std=2.0 / H ** 0.5)
            t[p + "mlp.correction"] = rnd(E, std=0.3)
            for e in range(E):
                t[f"{p}mlp.e{e}.gate"] = rnd(ff, H, std=1.0 / H ** 0.5)
                t[f"{p}mlp.e{e}.up"] = rnd(ff, H, std=1.0 / H ** 0.5)
                t[f"{p}mlp.e{e}.down"] = rnd(H, ff, std=1.0 / ff ** 0.5)
    return t


_FOLDERS = {}


def folder_for(name, dtype=torch.float32, seed=0):
    """A temporary model folder of configuration ``name`` (made once per run)."""
    key = (name, dtype, seed)
    if key not in _FOLDERS:
        from safetensors.torch import save_file
        d = tempfile.mkdtemp(prefix=f"ramilorn_{name}_")
        cfg = CONFIGS[name]
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in make_tensors(cfg, seed, dtype).items()},
                  os.path.join(d, "model.safetensors"))
        _FOLDERS[key] = d
    return _FOLDERS[key]


def _cleanup():
    for d in _FOLDERS.values():
        shutil.rmtree(d, ignore_errors=True)


import atexit
atexit.register(_cleanup)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(folder, toks, streams=None, experts=None):
    from plain import ramilorn_plain as P
    return P.forward(P.read_config(folder), P.read_weights(folder), toks, streams, experts)
