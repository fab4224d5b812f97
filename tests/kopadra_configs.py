"""Small Kopadra configurations for the tests.  The sizes are awkward on purpose: widths that are no
power of two, key and value sizes that are equal (the head-major pages) and that differ (one row a
token), sizes that are no multiple of 8, one key head and as many as query heads, rotated dimensions
fewer than the head, all of it and none, plain and stretched frequencies, readers of another layer's
keys, recurrent layers first, in the middle and twice in a row, capped and uncapped gates, layers
without a feed-forward, experts with and without groups, identity experts, a shared expert, every
expert chosen and one of many, with and without the cap on the logits."""

import torch

import vekasun_configs as VC

read_folder = VC.read_folder


def attention(heads, kv_heads, dim, vdim, scale, rot=None, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def mlstm(heads, dim, vdim, cap=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap is not None:
        m["gate_cap"] = cap
    return {"type": "mlstm", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity=None, groups=None, scale=None, shared=None):
    r = {"experts": experts, "top": top}
    if identity is not None:
        r["identity"] = identity
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# head-major pages (16 = 16) read by a second layer; a recurrent layer in the middle; a row-layout attention
# (8 against 24) read by a layer without a feed-forward; groups of which half are kept, two identity experts
SHARING = {
    "architecture": "Kopadra", "vocab": 211, "width": 96, "logit_softcap": 9.0, "norm": {"eps": 1e-5},
    "layers": [
        layer(attention(6, 2, 16, 16, 0.3, rot=(500.0, 8), scaling=(4.0, 64, 8.0, 1.0)), dense(72)),
        layer(attention(6, 2, 16, 16, 0.25, rot=(500.0, 8), scaling=(4.0, 64, 8.0, 1.0), kv_from=0),
              moe(40, 6, 3, identity=2, groups=(4, 2), scale=2.5, shared=56)),
        layer(mlstm(3, 16, 24, cap=6.0), dense(48)),
        layer(attention(4, 4, 8, 24, 0.35, rot=(10000.0, 8)), moe(24, 3, 2)),
        layer(attention(8, 4, 8, 24, 0.5, rot=(10000.0, 8), kv_from=3), None),
    ],
}

# nothing a multiple of 8 where it can be helped; the recurrent layer first and uncapped; no cap on the logits;
# every expert chosen (identity included); no rotation in one layer
AWKWARD = {
    "architecture": "Kopadra", "vocab": 97, "width": 100, "norm": {"eps": 2e-5},
    "layers": [
        layer(mlstm(5, 10, 7), moe(20, 4, 5, identity=1, scale=0.7)),
        layer(attention(3, 3, 12, 20, 0.4, rot=(300.0, 6), scaling=(2.0, 32, 4.0, 0.5)), moe(20, 5, 2, identity=1, groups=(3, 3), shared=36)),
        layer(attention(6, 3, 12, 20, 0.3, rot=(300.0, 6), scaling=(2.0, 32, 4.0, 0.5), kv_from=1), dense(52)),
        layer(attention(2, 1, 20, 20, 0.22), dense(36)),
    ],
}

# heads of 64 and 128 (the split-key decode kernel and the flash kernels), one key head for eight query heads, two
# recurrent layers in a row (one without a feed-forward), a group of which one is kept, the whole head turned
WIDE = {
    "architecture": "Kopadra", "vocab": 131, "width": 128, "logit_softcap": 20.0, "norm": {"eps": 1e-5},
    "layers": [
        layer(attention(8, 2, 64, 64, 0.06, rot=(1000.0, 32), scaling=(8.0, 128, 16.0, 2.0)), dense(64)),
        layer(mlstm(2, 64, 40, cap=4.0), None),
        layer(mlstm(4, 32, 32, cap=12.0), dense(40)),
        layer(attention(8, 1, 128, 128, 0.04, rot=(250.0, 128)), moe(32, 7, 2, identity=1, groups=(2, 1), scale=1.25, shared=24)),
        layer(attention(8, 1, 128, 128, 0.03, rot=(250.0, 128), kv_from=3), moe(16, 4, 1, groups=(4, 2))),
    ],
}

CONFIGS = {"sharing": (SHARING, 61), "awkward": (AWKWARD, 62), "wide": (WIDE, 63)}

# factors that take the random weights (standard deviation 0.02) out of their nearly linear range
LIVELY = {".mix.q": 6.0, ".mix.k": 6.0, ".mix.v": 5.0, ".mix.g": 8.0, ".q.b": 20.0, ".k.b": 20.0, ".v.b": 10.0,
          ".mix.i": 8.0, ".mix.f": 8.0, ".i.b": 20.0, ".gate": 6.0, ".up": 6.0, ".router": 25.0}
# ... less so for the configuration with the large heads, whose five layers otherwise magnify a rounding of the
# projections tenfold on most rows
MILD = {".mix.q": 2.0, ".mix.k": 2.0, ".mix.v": 2.0, ".mix.g": 3.0, ".q.b": 6.0, ".k.b": 6.0, ".v.b": 4.0,
        ".mix.i": 4.0, ".mix.f": 4.0, ".i.b": 8.0, ".gate": 2.0, ".up": 2.0, ".router": 25.0}
SCALES = {"wide": MILD}
# the recurrence alone is tried with gates that swing further (their projections reach three times the smaller caps)
SWINGING = dict(LIVELY, **{".mix.i": 20.0, ".mix.f": 20.0, ".i.b": 30.0})


def lively_tensors(cfg, seed):
    """Replacements for the tensors whose random draw would hide their mechanism: corrections large
    enough to change who is chosen, norms on q and k that vary over the projection, forget biases of both
    signs."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for i, L in enumerate(cfg["layers"]):
        m, f = L["mixer"], L["mlp"]
        if L["type"] == "attention":
            out[f"l{i}.mix.q.norm"] = torch.rand(m["heads"] * m["dim"], generator=g) * 1.4 + 0.3
            if m.get("kv_from") is None:
                out[f"l{i}.mix.k.norm"] = torch.rand(m["kv_heads"] * m["dim"], generator=g) * 1.4 + 0.3
        else:
            out[f"l{i}.mix.f.b"] = torch.linspace(-1.0, 4.0, m["heads"])
        if f and f["kind"] == "moe":
            E = f["router"]["experts"] + f["router"].get("identity", 0)
            out[f"l{i}.mlp.correction"] = (torch.rand(E, generator=g) - 0.5) * 0.6
    return out


def write_folder(config, seed, out_dir, replace=None, scale=None):
    """A model folder with the engine's seeded random tensors, the lively replacements above and
    whatever `replace` names on top."""
    import os
    from safetensors import safe_open
    from safetensors.torch import save_file
    from ninfer_amd_mi50_b200.weights import write_random_model
    write_random_model(config, seed, out_dir)
    path = os.path.join(out_dir, "model.safetensors")
    tensors = {}
    with safe_open(path, framework="pt") as f:
        for n in f.keys():
            tensors[n] = f.get_tensor(n)
    for n in list(tensors):
        for suffix, factor in (LIVELY if scale is None else scale).items():
            if n.endswith(suffix):
                tensors[n] = (tensors[n].float() * factor).to(torch.bfloat16)
    new = lively_tensors(config, seed)
    new.update(replace or {})
    for n, t in new.items():
        assert n in tensors and tuple(tensors[n].shape) == tuple(t.shape), n
        tensors[n] = t.to(torch.bfloat16).contiguous()
    save_file(tensors, path)
    return out_dir
