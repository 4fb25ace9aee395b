"""Zazerax without a GPU: the configuration reader and its errors, the lowering to part
specs and a run order, tensor names and the loader, and the plain implementation's
mechanisms on cases worked out by hand."""
import copy
import json
import math
import os

import pytest
import torch

from agave_b200.config import ConfigError, load_config, resolve_architecture
from agave_b200.config.base import (AttentionSpec, DenseFeedForwardSpec, LatentAttentionSpec,
                                    LayerNormSpec)
from agave_b200.config.zazerax import ZazeraxConfig
from agave_b200.models.decoder import decoder_param_specs
from agave_b200.parts.attention import AttentionMixer
from agave_b200.parts.rope import RotaryEmbedding
from agave_b200.weights import WeightsError, load_weights
from plain import zazerax_plain as P
from zazerax_util import BIAS_ROWS, CONFIGS, folder_for, make_tensors


def with_rows(name):
    """The configuration with the distance tables' row counts written into it (what a
    folder's tensor shapes give otherwise)."""
    raw = copy.deepcopy(CONFIGS[name])
    for i, layer in enumerate(raw["layers"]):
        if layer["type"] == "attention":
            src = layer.get("weights_of", i)
            layer["mixer"]["bias_rows"] = BIAS_ROWS[name][src]
    return raw


# ------------------------------------------------------------------- reading
def test_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Zazerax"}).name == "Zazerax"
    assert resolve_architecture({"model_type": "zazerax"}).name == "Zazerax"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_reading_and_writing_round_trip(name):
    cfg = ZazeraxConfig.from_dict(with_rows(name))
    again = ZazeraxConfig.from_dict(cfg.to_dict())
    assert again == cfg
    assert len(cfg.layers) == len(CONFIGS[name]["layers"])


def test_rows_of_the_distance_table_come_from_the_folder():
    folder = folder_for("Z1")
    entry, cfg = load_config(folder)
    assert entry.name == "Zazerax"
    assert cfg.bias_rows == (0, 6, 0, 6, 0)
    with pytest.raises(ConfigError, match="rows are unknown"):
        ZazeraxConfig.from_dict(CONFIGS["Z1"])


@pytest.mark.parametrize("path, value, match", [
    (("vocab",), None, "vocab"),
    (("embedding",), None, "embedding"),
    (("norm", "eps"), None, "norm.eps"),
    (("layers", 0, "type"), "conv", "not a mixer"),
    (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mixer", "rot", "dims"), 4, "rot.dims"),
    (("layers", 0, "mixer", "rot_dim"), 5, "even"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), None, "factor"),
    (("layers", 1, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 1, "mixer", "bias_max"), 2, "bias_max"),
    (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 2, "mixer", "q_rank"), None, "q_rank"),
    (("layers", 0, "mlp", "kind"), "moe", "not a feed-forward"),
    (("layers", 3, "weights_of"), 3, "another layer"),
    (("layers", 3, "weights_of"), 4, "without tensors"),
    (("layers", 3, "weights_of"), 0, "must equal"),
])
def test_errors_name_the_key(path, value, match):
    raw = with_rows("Z1")
    d = raw
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        ZazeraxConfig.from_dict(raw)


# ------------------------------------------------------------------ lowering
def test_lowering_to_parts_and_run_order():
    cfg = ZazeraxConfig.from_dict(with_rows("Z1"))
    spec = cfg.to_model_spec()
    assert cfg.owners() == (0, 1, 2)
    assert len(spec.blocks) == 3 and not spec.tie_embeddings
    assert [(c.block, c.cache, c.writes_cache) for c in spec.schedule] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (1, 3, True), (0, 4, True)]
    assert spec.embed_scale == 2.5
    b0, b1, b2 = spec.blocks
    assert all(b.arrangement == "post" and b.norm == LayerNormSpec(eps=1e-5, bias=False)
               for b in spec.blocks)
    assert isinstance(b0.mixer, LatentAttentionSpec) and b0.mixer.gate == "element"
    assert b0.mixer.q_rank == 0 and not b0.mixer.position.interleaved
    assert b0.mixer.position.scaling.factor == 4.0 and b0.mixer.position.theta == 1000.0
    assert b0.feed_forward == DenseFeedForwardSpec(intermediate_size=40, activation="relu2")
    assert isinstance(b1.mixer, AttentionSpec) and b1.feed_forward is None
    m = b1.mixer
    assert (m.window, m.qk_norm_whole, m.fixed_sink, m.position) == (7, True, 0.0, None)
    assert (m.distance_bias.rows, m.distance_bias.far, m.value_dim) == (6, 30.0, 14)
    assert b2.mixer.gate == "head" and b2.mixer.q_rank == 24 and b2.mixer.position.interleaved
    assert b2.mixer.position.scaling is None


def test_tensor_names_and_loader():
    folder = folder_for("Z1")
    entry, cfg = load_config(folder)
    specs = decoder_param_specs(cfg.to_model_spec())
    names = entry.weight_names(cfg)
    want = {names.checkpoint_name(n, "") for n in specs}
    made = set(make_tensors(CONFIGS["Z1"], BIAS_ROWS["Z1"], 0, torch.float32))
    assert want == made
    assert names.checkpoint_name("blocks.2.mixer.q_down_norm.weight", "") == "l2.mix.dq.norm"
    assert names.checkpoint_name("blocks.1.mixer.distance_bias", "") == "l1.mix.rel"
    assert names.checkpoint_name("lm_head.weight", "") == "head"
    tensors = load_weights(folder, specs, names.checkpoint_name, names.prefixes)
    assert tensors["blocks.1.mixer.distance_bias"].shape == (6, 4)
    assert tensors["blocks.0.mixer.kv_down.weight"].shape == (26, 72)


def test_loader_reports_what_is_wrong(tmp_path):
    from safetensors.torch import save_file
    t = make_tensors(CONFIGS["Z1"], BIAS_ROWS["Z1"], 0, torch.float32)
    del t["l2.mix.uq"]
    t["l0.mix.uk"] = t["l0.mix.uk"][:, :5].contiguous()
    t["l4.norm1"] = torch.ones(72)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(CONFIGS["Z1"], f)
    save_file(t, str(tmp_path / "model.safetensors"))
    entry, cfg = load_config(str(tmp_path))
    names = entry.weight_names(cfg)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path), decoder_param_specs(cfg.to_model_spec()),
                     names.checkpoint_name, names.prefixes)
    assert e.value.missing == ["l2.mix.uq"]
    assert e.value.unexpected == ["l4.norm1"]
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.uk"]


# -------------------------------------------------- mechanisms, by hand and crosswise
def test_distance_rows_by_hand():
    # 8 rows, far 64: distances 0..3 have rows of their own; from 4 on
    # row = 4 + floor(log(n / 4) / log(16) * 4), capped at 7
    want = {0: 0, 3: 3, 4: 4, 7: 4, 8: 5, 15: 5, 16: 6, 31: 6, 32: 7, 64: 7, 1000: 7}
    for n, r in want.items():
        assert P.distance_bucket(n, 8, 64.0) == r, n
    lib = AttentionMixer.distance_rows(8, 64.0, 1001)
    assert [lib[n] for n in want] == list(want.values())
    for rows, far in ((6, 30.0), (12, 500.0), (4, 40.0), (20, 333.0)):
        assert AttentionMixer.distance_rows(rows, far, 700) == \
            [P.distance_bucket(n, rows, far) for n in range(700)]


def test_scaled_frequencies_by_hand_and_against_the_library():
    # dims 8, base 16, original 16: wavelengths 2 pi 16^(i/4); pair(t) = 8 ln(16 / (2 pi t)) / (2 ln 16)
    rot = {"base": 16.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 2.0,
                                                "slow": 0.25}}
    f, mult = P.rotary_frequencies(rot)
    lo = max(math.floor(8 * math.log(16 / (4 * math.pi)) / (2 * math.log(16))), 0)
    hi = min(math.ceil(8 * math.log(16 / (0.5 * math.pi)) / (2 * math.log(16))), 7)
    assert (lo, hi) == (0, 4)
    base_f = [16.0 ** (-2 * i / 8) for i in range(4)]
    want = [base_f[i] / 4 * (i / 4) + base_f[i] * (1 - i / 4) for i in range(4)]
    assert torch.allclose(f, torch.tensor(want, dtype=torch.float64), rtol=1e-14)
    assert mult == pytest.approx(0.1 * math.log(4.0) + 1.0)
    from agave_b200.config.base import RotarySpec, WavelengthScalingSpec
    for name in sorted(CONFIGS):
        for layer in CONFIGS[name]["layers"]:
            r = layer["mixer"].get("rot")
            if r is None:
                continue
            sc = r.get("scaling")
            part = RotaryEmbedding(RotarySpec(
                theta=r["base"], rotary_dim=r["dims"],
                scaling=None if sc is None else WavelengthScalingSpec(
                    sc["factor"], sc["original"], sc["fast"], sc["slow"])), r["dims"])
            lf, lm = part.frequencies()
            pf, pm = P.rotary_frequencies(r)
            assert torch.allclose(torch.tensor(lf, dtype=torch.float64), pf, rtol=1e-13)
            assert lm == pytest.approx(pm)


def test_rotation_layouts_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=torch.float64)
    rot = {"base": 100.0, "dims": 4}
    pos = torch.tensor([3])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    halves = P.rotate(x, pos, rot, interleaved=False)[0]
    assert halves[0].item() == pytest.approx(1 * math.cos(a0) - 3 * math.sin(a0))
    assert halves[2].item() == pytest.approx(3 * math.cos(a0) + 1 * math.sin(a0))
    assert halves[1].item() == pytest.approx(2 * math.cos(a1) - 4 * math.sin(a1))
    pairs = P.rotate(x, pos, rot, interleaved=True)[0]
    assert pairs[0].item() == pytest.approx(1 * math.cos(a0) - 2 * math.sin(a0))
    assert pairs[1].item() == pytest.approx(2 * math.cos(a0) + 1 * math.sin(a0))
    assert pairs[3].item() == pytest.approx(4 * math.cos(a1) + 3 * math.sin(a1))


def test_window_and_the_one_in_the_denominator_by_hand():
    # one head, keys equal to e_1 * c_j, values the position: scores are known
    q = torch.zeros(4, 1, 2, dtype=torch.float64); q[:, 0, 0] = 1.0
    k = torch.zeros(4, 1, 2, dtype=torch.float64); k[:, 0, 0] = torch.tensor([0.0, 1.0, 2.0, 3.0])
    v = torch.arange(4, dtype=torch.float64).view(4, 1, 1)
    o = P.softmax_attention(q, k, v, 1.0, window=2, one_in_denominator=True)
    e = [math.exp(x) for x in (0, 1, 2, 3)]
    assert o[0, 0, 0].item() == pytest.approx(0.0)
    assert o[1, 0, 0].item() == pytest.approx(e[1] / (1 + e[0] + e[1]))
    assert o[3, 0, 0].item() == pytest.approx((2 * e[2] + 3 * e[3]) / (1 + e[2] + e[3]))
    bias = torch.tensor([[0.5], [-1.0]], dtype=torch.float64)       # 2 rows: distance 0, >= 1
    o = P.softmax_attention(q, k, v, 1.0, window=3, bias=bias, far=8.0)
    w = [math.exp(1 - 1.0), math.exp(2 - 1.0), math.exp(3 + 0.5)]
    assert o[3, 0, 0].item() == pytest.approx((w[0] + 2 * w[1] + 3 * w[2]) / sum(w))


def test_norms_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    ln = P.layer_norm(x, w, 0.5)
    assert torch.allclose(ln, (x - 3.0) / math.sqrt(3.5 + 0.5) * w)
    rn = P.rms_norm(x, w, 0.5)
    assert torch.allclose(rn, x / math.sqrt(12.5 + 0.5) * w)
