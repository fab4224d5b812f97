"""Kopadra's configuration and plan: what config.json says is what the parts are built with."""

import copy
import math

import pytest
import torch

import kopadra_configs as KC
import plain_kopadra as PK
from ninfer_amd_mi50_b200.config.model_config import ConfigError
from ninfer_amd_mi50_b200.engine.loading import build_model
from ninfer_amd_mi50_b200.registry import architecture_names


def test_the_design_is_registered():
    assert "Kopadra" in architecture_names()


@pytest.mark.parametrize("name", sorted(KC.CONFIGS))
def test_what_each_layer_keeps_and_which_tensors_it_names(name):
    cfg, _ = KC.CONFIGS[name]
    typed, model = build_model(cfg)
    names = {s.name: s.shape for s in model.tensor_specs()}
    caches, states = model.cache_specs(), model.state_specs()
    W = cfg["width"]
    for i, L in enumerate(cfg["layers"]):
        m, call = L["mixer"], model.order[i]
        if L["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            assert caches[i] is None and states[i].shape == (H * V * D + H * D + H,)
            assert names[f"l{i}.mix.i"] == (H, W) and names[f"l{i}.mix.f.b"] == (H,) and names[f"l{i}.mix.norm"] == (H * V,)
            assert names[f"l{i}.mix.q"] == (H * D, W) and names[f"l{i}.mix.v"] == (H * V, W) and f"l{i}.mix.q.b" not in names
        else:
            src = m.get("kv_from")
            assert states[i] is None
            assert names[f"l{i}.mix.q.norm"] == (m["heads"] * m["dim"],) and names[f"l{i}.mix.g"] == (m["heads"] * m["vdim"], W)
            if src is None:
                assert call.cache == i and call.append
                if m["dim"] == m["vdim"] and m["dim"] % 16 == 0:
                    assert (caches[i].num_kv_heads, caches[i].head_dim, caches[i].row_width) == (m["kv_heads"], m["dim"], 0)
                else:
                    assert caches[i].row_width == m["kv_heads"] * (m["dim"] + m["vdim"])
                assert names[f"l{i}.mix.k.norm"] == (m["kv_heads"] * m["dim"],) and f"l{i}.mix.v.b" in names
            else:
                assert caches[i] is None and call.cache == src and not call.append
                assert not any(n.startswith(f"l{i}.mix.k") or n.startswith(f"l{i}.mix.v") for n in names)
        f = L["mlp"]
        assert (f"l{i}.norm2" in names) == (f is not None)
        if f and f["kind"] == "moe":
            r = f["router"]
            total = r["experts"] + r.get("identity", 0)
            assert names[f"l{i}.mlp.router"] == (total, W) and names[f"l{i}.mlp.correction"] == (total,)
            assert f"l{i}.mlp.e{r['experts'] - 1}.down" in names and f"l{i}.mlp.e{r['experts']}.down" not in names
            assert (f"l{i}.mlp.shared.up" in names) == ("shared" in f)
    assert "head" not in names and "final.norm" in names and "embed" in names


def test_sizes_and_constants_come_from_the_configuration():
    cfg = copy.deepcopy(KC.SHARING)
    typed, model = build_model(cfg)
    assert model.plan.logit_softcap == 9.0 and model.plan.tie_word_embeddings
    b0, b1, b2 = model.blocks[0], model.blocks[1], model.blocks[2]
    assert (b0.mixer.scale, b1.mixer.scale) == (0.3, 0.25) and b0.mixer.own_kv and not b1.mixer.own_kv
    p = b0.mixer.position
    assert (p.rotary_dim, p.theta, p.factor, p.original, p.fast, p.slow) == (8, 500.0, 4.0, 64.0, 8.0, 1.0)
    assert abs(p.magnitude - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert model.blocks[3].mixer.position.magnitude == 1.0
    assert b0.norm1.eps == 1e-5 and type(b0.norm1).__name__ == "LayerNorm"
    f = b1.feed_forward
    assert (f.num_experts, f.identity_experts, f.top_k, f.groups, f.route_scale) == (6, 2, 3, (4, 2), 2.5)
    assert f.shared_intermediate_size == 56 and not f.shared_gate and f.has_correction
    assert (b2.mixer.gate_cap, b2.mixer.heads, b2.mixer.dim, b2.mixer.value_dim) == (6.0, 3, 16, 24)
    assert abs(b2.mixer.query_scale - 0.25) < 1e-12
    assert b0.feed_forward.activation == (4, 0.0, 0.0)
    cfg["layers"][2]["mixer"].pop("gate_cap")
    cfg["layers"][1]["mlp"]["router"] = {"experts": 6, "top": 2}
    cfg["layers"][0]["mixer"]["rot"].pop("scaling")
    cfg["layers"][1]["mixer"]["rot"].pop("scaling")
    del cfg["logit_softcap"]
    typed, model = build_model(cfg)
    f = model.blocks[1].feed_forward
    assert model.blocks[2].mixer.gate_cap == 0.0 and (f.identity_experts, f.groups, f.route_scale) == (0, None, 1.0)
    assert type(model.blocks[0].mixer.position).__name__ == "RotaryHalfSplit" and model.plan.logit_softcap == 0.0


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "names no other layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "no keys of its own"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "no keys of its own"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "differ"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(base=499.0), "differ"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "even and at most"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.5), "factor"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "cannot give"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "cannot give"),
    (lambda c: c["layers"][3]["mlp"]["router"].update(top=4), "exceeds"),
    (lambda c: c["layers"][0].update(type="recurrent"), "known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "known"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_configuration_that_cannot_run_is_refused(change, message):
    cfg = copy.deepcopy(KC.SHARING)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg)


@pytest.mark.parametrize("rot", [
    {"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}},
    {"base": 1e6, "dims": 64, "scaling": {"factor": 32.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"base": 10000.0, "dims": 6, "scaling": {"factor": 2.0, "original": 5, "fast": 4.0, "slow": 3.9}},     # the ramp is one step
    {"base": 50.0, "dims": 10, "scaling": {"factor": 16.0, "original": 100000, "fast": 2.0, "slow": 0.25}},  # everything above the ramp
    {"base": 300.0, "dims": 12, "scaling": {"factor": 1.0, "original": 32, "fast": 4.0, "slow": 0.5}},
])
def test_stretched_frequencies_are_the_plain_rules(rot):
    from ninfer_amd_mi50_b200.parts.position import RotaryHalfSplitBlended
    sc = rot["scaling"]
    part = RotaryHalfSplitBlended(head_dim=rot["dims"] + 4, theta=rot["base"], rotary_dim=rot["dims"], factor=sc["factor"],
                                  original=sc["original"], fast=sc["fast"], slow=sc["slow"])
    table, dims = part.rotary_table(torch.device("cpu"))
    want, magnitude = PK.rotary_frequencies(rot)
    assert dims == rot["dims"] and table.dtype == torch.float32
    assert torch.allclose(table.double(), want, rtol=1e-7, atol=0.0)
    assert abs(part.magnitude - magnitude) < 1e-12
