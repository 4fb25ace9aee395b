"""Ramilorn on the CPU: the configuration reader and its errors, the lowering to part
specs and the run order, tensor names and the loader, and the plain implementation's own
mechanisms on cases worked out by hand."""
import copy
import json
import math
import os

import pytest
import torch

from agave_b200.config import ConfigError, RamilornConfig, load_config, resolve_architecture
from agave_b200.models.decoder import decoder_param_specs
from agave_b200.weights import WeightsError, load_weights
from plain import ramilorn_plain as P
from ramilorn_util import CONFIGS, folder_for, make_tensors


def test_registry_finds_the_architecture_by_its_singular_key():
    entry = resolve_architecture(CONFIGS["R1"])
    assert entry.name == "Ramilorn" and entry.config_class is RamilornConfig


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_lowering(name):
    raw = CONFIGS[name]
    cfg = RamilornConfig.from_dict(raw)
    assert cfg.to_dict() == raw
    spec = cfg.to_model_spec()
    assert spec.hidden_size == raw["width"] and spec.vocab_size == raw["vocab"]
    assert spec.logit_softcap == raw["logit_softcap"] and spec.tie_embeddings
    assert spec.embed_scale == 1.0
    for i, (layer, block, call) in enumerate(zip(raw["layers"], spec.blocks, spec.schedule)):
        m = layer["mixer"]
        a = block.mixer
        assert (a.n_heads, a.n_kv_heads, a.head_dim, a.v_dim) == (m["heads"], m["kv_heads"],
                                                                  m["dim"], m["vdim"])
        assert a.scale == m["scale"] and a.sink and a.position is None and a.qk_norm is None
        assert (a.q_temp.coef, a.q_temp.every) == (m["q_temp"]["coef"], m["q_temp"]["every"])
        assert block.residual_mult == raw["residual_mult"] and block.norm.eps == raw["norm"]["eps"]
        src = m.get("kv_from")
        assert a.own_kv == (src is None)
        assert call == type(call)(block=i, cache=i if src is None else src,
                                  writes_cache=src is None)
        if layer["mlp"] is None:
            assert block.feed_forward is None
        else:
            r = layer["mlp"]["router"]
            f = block.feed_forward
            assert (f.n_experts, f.top, f.n_groups, f.keep_groups, f.intermediate_size) == (
                r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"],
                layer["mlp"]["expert"]["ff"])
            assert f.activation == "silu"


def _broken(path, value, drop=False):
    raw = copy.deepcopy(CONFIGS["R1"])
    d = raw
    for k in path[:-1]:
        d = d[k]
    if drop:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    return raw


@pytest.mark.parametrize("path, value, drop, word", [
    (("width",), None, True, "width"),
    (("norm", "eps"), None, True, "norm.eps"),
    (("residual_mult",), "x", False, "residual_mult"),
    (("logit_softcap",), 0.0, False, "logit_softcap"),
    (("layers", 0, "type"), "recurrent", False, "type"),
    (("layers", 0, "mixer", "heads"), 3, False, "multiple"),
    (("layers", 0, "mixer", "q_temp"), None, True, "q_temp"),
    (("layers", 0, "mixer", "q_temp", "every"), 0, False, "every"),
    (("layers", 2, "mixer", "kv_from"), 2, False, "earlier"),
    (("layers", 4, "mixer", "kv_from"), 2, False, "without keys"),
    (("layers", 0, "mlp", "kind"), "dense", False, "kind"),
    (("layers", 0, "mlp", "router", "groups", "count"), 3, False, "equal groups"),
    (("layers", 0, "mlp", "router", "top"), 5, False, "top"),
    (("layers", 0, "mlp"), None, True, "mlp"),
])
def test_configuration_errors_name_the_key(path, value, drop, word):
    with pytest.raises(ConfigError) as e:
        RamilornConfig.from_dict(_broken(path, value, drop))
    assert word in str(e.value)


def test_tensor_names_and_loader():
    folder = folder_for("R1")
    entry, cfg = load_config(folder)
    specs = decoder_param_specs(cfg.to_model_spec())
    names = entry.weight_names(cfg)
    expected = set(make_tensors(CONFIGS["R1"], 0, torch.float32))
    assert {names.checkpoint_name(n, "") for n in specs} == expected
    # layers without keys and values of their own, and the one without a feed-forward,
    # ask for nothing they do not have
    assert "blocks.2.mixer.k_proj.weight" not in specs and "blocks.3.ffn.router.weight" not in specs
    assert "blocks.3.pre_ffn_norm.weight" not in specs
    t = load_weights(folder, specs, names.checkpoint_name, names.prefixes)
    assert t["blocks.0.mixer.sink"].shape == (4,) and t["final_norm.bias"].shape == (72,)


def test_loader_reports_a_missing_and_a_stray_tensor(tmp_path):
    from safetensors.torch import save_file
    t = make_tensors(CONFIGS["R2"], 1, torch.float32)
    del t["l1.mix.sink"]
    t["l2.mix.k"] = torch.zeros(6 * 32, 96)        # layer 2 attends to layer 0's keys
    with open(tmp_path / "config.json", "w") as f:
        json.dump(CONFIGS["R2"], f)
    save_file(t, str(tmp_path / "model.safetensors"))
    entry, cfg = load_config(str(tmp_path))
    names = entry.weight_names(cfg)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path), decoder_param_specs(cfg.to_model_spec()),
                     names.checkpoint_name, names.prefixes)
    assert e.value.missing == ["l1.mix.sink"] and e.value.unexpected == ["l2.mix.k"]


# ------------------------------------------------ the plain implementation by hand
def test_plain_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    b = torch.tensor([0.0, 1.0, -1.0, 0.0], dtype=torch.float64)
    var = ((1 - 3) ** 2 + (2 - 3) ** 2 + 0 + (6 - 3) ** 2) / 4
    r = 1 / math.sqrt(var + 0.5)
    want = torch.tensor([[-2 * r, -1 * r * 2 + 1, -1.0, 3 * r * 0.5]], dtype=torch.float64)
    assert torch.allclose(P.layer_norm(x, w, b, 0.5), want)


def test_plain_query_temperature_steps():
    tau = P.query_temperature(10, 0.5, 4, torch.float64)
    # positions 0..2 -> 1; 3..6 -> 1 + 0.5 ln 2; 7..9 -> 1 + 0.5 ln 3
    want = [1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 3
    assert torch.allclose(tau, torch.tensor(want, dtype=torch.float64))


def test_plain_sink_takes_its_share_of_the_weight():
    # one head, keys all zero: every score is 0, the sink is ln 3, so after t + 1 keys the
    # values' weights sum to (t + 1) / (t + 4)
    T = 5
    q = torch.ones(T, 1, 2, dtype=torch.float64)
    k = torch.zeros(T, 1, 2, dtype=torch.float64)
    v = torch.ones(T, 1, 3, dtype=torch.float64)
    out = P.sink_attention(q, k, v, torch.tensor([math.log(3.0)], dtype=torch.float64), 0.7)
    for t in range(T):
        assert torch.allclose(out[t, 0], torch.full((3,), (t + 1) / (t + 4), dtype=torch.float64))


def test_plain_router_groups_and_negative_scores():
    # six experts in three groups; logits 0 everywhere, so s = 0.5 and the correction
    # decides.  Group sums of choice scores: (-0.5 + -0.6), (-0.1 + -3), (-0.7 + -0.8):
    # groups 0 and 2 stay although group 1 holds the single best expert.  Every choice
    # score is negative, so an expert masked to 0 instead of being excluded would win.
    corr = torch.tensor([-1.0, -1.1, -0.6, -3.5, -1.2, -1.3], dtype=torch.float64)
    x = torch.zeros(1, 4, dtype=torch.float64)
    wr = torch.zeros(6, 4, dtype=torch.float64)
    r = {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}}
    ids, wt = P.route(x, wr, corr, r)
    assert ids.tolist() == [[0, 1, 4]]
    assert torch.allclose(wt, torch.full((1, 3), 0.5, dtype=torch.float64))


def test_plain_model_runs_every_configuration():
    for name in CONFIGS:
        folder = folder_for(name)
        streams = []
        z = P.forward(P.read_config(folder), P.read_weights(folder), [1, 2, 3, 4, 5, 6], streams)
        assert z.shape == (6, CONFIGS[name]["vocab"]) and torch.isfinite(z).all()
        assert len(streams) == len(CONFIGS[name]["layers"])
        assert z.abs().max() < CONFIGS[name]["logit_softcap"]
