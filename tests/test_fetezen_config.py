"""Fetezen's configuration and plan: what config.json says is what the parts are built with."""

import copy

import pytest

import fetezen_configs as FC
from ninfer_amd_mi50_b200.config.model_config import ConfigError
from ninfer_amd_mi50_b200.engine.loading import build_model
from ninfer_amd_mi50_b200.registry import architecture_names


def test_the_design_is_registered():
    assert "Fetezen" in architecture_names()


@pytest.mark.parametrize("name", sorted(FC.CONFIGS))
def test_readers_of_another_layers_keys_hold_no_pages_and_no_key_tensors(name):
    cfg, _ = FC.CONFIGS[name]
    typed, model = build_model(cfg)
    names = {s.name for s in model.tensor_specs()}
    specs = model.cache_specs()
    for i, L in enumerate(cfg["layers"]):
        src = L["mixer"].get("kv_from")
        call = model.order[i]
        if src is None:
            assert specs[i] is not None and call.cache == i and call.append
            assert specs[i].row_width == L["mixer"]["kv_heads"] * (L["mixer"]["dim"] + L["mixer"]["vdim"])
            assert f"l{i}.mix.k" in names and f"l{i}.mix.v.b" in names and f"l{i}.mix.k.norm" in names
        else:
            assert specs[i] is None and call.cache == src and not call.append
            assert not any(n.startswith(f"l{i}.mix.k") or n.startswith(f"l{i}.mix.v") for n in names)
        assert f"l{i}.mix.q.norm" in names and f"l{i}.mix.talk" in names and f"l{i}.mix.sink" in names
        assert (f"l{i}.hc1.mix" in names) == ("streams" in cfg)
        assert (f"l{i}.hc2.mix" in names) == ("streams" in cfg and L["mlp"] is not None)
        assert (f"l{i}.norm2" in names) == (L["mlp"] is not None)
    assert "head" in names and "final.norm" in names and "embed" in names


def test_sizes_and_constants_come_from_the_configuration():
    cfg = copy.deepcopy(FC.SHARING)
    typed, model = build_model(cfg)
    assert model.streams == 2 and model.plan.logit_softcap == 9.0
    b0, b1 = model.blocks[0], model.blocks[1]
    assert (b0.mixer.chunk, b1.mixer.chunk, model.blocks[2].mixer.chunk) == (21, 50, 0)
    assert (b0.mixer.scale, b1.mixer.scale) == (0.3, 0.25)
    assert b0.mixer.position.rotary_dim == 8 and b0.mixer.position.theta == 500.0
    assert b0.norm1.groups == 3 and model.final_norm.groups == 3 and b0.norm1.eps == 1e-5
    assert b0.streams == 2 and b0.learned
    assert b1.feed_forward.top_k == 2 and b1.feed_forward.num_experts == 5 and b1.feed_forward.shared_intermediate_size == 56
    assert model.blocks[2].feed_forward.shared_intermediate_size == 0
    shapes = {s.name: s.shape for s in model.tensor_specs()}
    assert shapes["l0.mix.v"] == (2 * 24, 96) and shapes["l0.mix.o"] == (96, 6 * 24) and shapes["l0.mix.q.norm"] == (16,)
    assert shapes["l1.mlp.table"] == (211, 2) and shapes["l0.mlp.act"] == (4,) and shapes["l1.mlp.shared.sg"] == (1, 96)
    cfg["streams"] = 4
    cfg["norm"]["groups"] = 1
    cfg["layers"][0]["mixer"]["mask"]["size"] = 64
    del cfg["logit_softcap"]
    typed, model = build_model(cfg)
    assert model.streams == 4 and model.blocks[0].norm1.groups == 1 and model.blocks[0].mixer.chunk == 64
    assert model.plan.logit_softcap == 0.0
    typed, plain = build_model(FC.PLAIN)
    assert typed.streams is None and plain.streams == 1 and not plain.blocks[0].learned


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "names no other layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "no keys of its own"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "sizes differ"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "even and at most"),
    (lambda c: c["norm"].update(groups=7), "does not divide"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0].update(type="recurrent"), "known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "known"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_configuration_that_cannot_run_is_refused(change, message):
    cfg = copy.deepcopy(FC.SHARING)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg)
