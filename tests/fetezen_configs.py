"""Small Fetezen configurations for the tests.  The sizes are awkward on purpose: widths that are no
power of two, key and value sizes that differ and are no multiple of 8, chunks shorter and longer
than a page and no multiple of one, a layer that sees every earlier position, one key head and as
many as query heads, rotated dimensions fewer than the head and none at all, one residual stream,
several, and none declared, one norm group and several, every expert chosen and one of many, with
and without a shared expert, layers that read another layer's keys and values (with a chunk of
their own), a layer without a feed-forward, with and without the cap on the logits; and one with
heads of 128 and with 16 heads, which the tensor-core attention kernel serves with clusters."""

import torch

import vekasun_configs as VC

read_folder = VC.read_folder


def attention(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# two streams, three norm groups; a chunk of 21 over pages of 16; a reader of layer 0 with a longer chunk;
# a layer that sees everything; value size larger than key size; half of the head turned
SHARING = {
    "architecture": "Fetezen", "vocab": 211, "width": 96, "streams": 2, "logit_softcap": 9.0,
    "norm": {"eps": 1e-5, "groups": 3},
    "layers": [
        layer(attention(6, 2, 16, 24, 0.3, chunk=21, rot=(500.0, 8)), dense(72)),
        layer(attention(6, 2, 16, 24, 0.25, chunk=50, rot=(500.0, 8), kv_from=0), moe(40, 5, 2, shared=56)),
        layer(attention(4, 4, 8, 8, 0.35, rot=(10000.0, 8)), moe(24, 3, 3)),
        layer(attention(4, 4, 8, 8, 0.5, chunk=64, rot=(10000.0, 8), kv_from=2), None),
    ],
}

# no streams declared (the plain residual sum), one group, no cap, no rotation in one layer, one key head,
# a chunk of one position, top 1
PLAIN = {
    "architecture": "Fetezen", "vocab": 157, "width": 80, "norm": {"eps": 3e-6},
    "layers": [
        layer(attention(4, 1, 32, 16, 0.18, chunk=100), moe(24, 7, 1)),
        layer(attention(5, 5, 8, 16, 0.4, chunk=1, rot=(77.0, 4)), dense(56)),
        layer(attention(2, 2, 16, 16, 0.25, chunk=5, rot=(100.0, 16)), moe(16, 2, 1, shared=8)),
    ],
}

# nothing a multiple of 8 where it can be helped; one declared stream (its constants are learned);
# four streams would be the other end and stand in the mechanism tests
AWKWARD = {
    "architecture": "Fetezen", "vocab": 97, "width": 100, "streams": 1, "logit_softcap": 30.0,
    "norm": {"eps": 2e-5, "groups": 5},
    "layers": [
        layer(attention(3, 3, 12, 20, 0.4, chunk=33, rot=(300.0, 6)), moe(20, 7, 2, shared=36)),
        layer(attention(6, 3, 12, 20, 0.3, chunk=7, rot=(300.0, 6), kv_from=0), dense(52)),
    ],
}

# heads of 128 and many heads: the tensor-core attention kernel deals them out over clusters of two CTAs; a reader
# of layer 0 with a longer chunk; key heads shared by two and by eight query heads; a layer that sees everything
WIDE = {
    "architecture": "Fetezen", "vocab": 131, "width": 128, "streams": 2, "logit_softcap": 20.0,
    "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        layer(attention(8, 4, 128, 64, 0.09, chunk=48, rot=(1000.0, 64)), moe(32, 6, 2, shared=24)),
        layer(attention(8, 4, 128, 64, 0.08, chunk=100, rot=(1000.0, 64), kv_from=0), dense(64)),
        layer(attention(16, 2, 32, 32, 0.2, rot=(300.0, 16)), None),
    ],
}

CONFIGS = {"sharing": (SHARING, 51), "plain": (PLAIN, 52), "awkward": (AWKWARD, 53), "wide": (WIDE, 54)}

# factors that take the random weights (standard deviation 0.02) out of their nearly linear range
LIVELY = {".mix.q": 6.0, ".mix.k": 6.0, ".mix.v": 4.0, ".q.b": 20.0, ".k.b": 20.0, ".v.b": 10.0, ".o.b": 10.0,
          ".up": 6.0, ".shared.sg": 30.0}


def lively_tensors(cfg, seed):
    """Replacements for the tensors whose random draw would hide their mechanism: the streams'
    constants (a mix far from the identity, reads and writes of both signs), the heads' mixing
    matrix, sinks from strong to absent, the activation's four numbers, and expert tables whose
    rows differ."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    S = cfg.get("streams")
    for i, L in enumerate(cfg["layers"]):
        H = L["mixer"]["heads"]
        out[f"l{i}.mix.talk"] = torch.eye(H) * 0.8 + torch.randn((H, H), generator=g) * 0.4
        out[f"l{i}.mix.sink"] = torch.linspace(3.0, -4.0, H)
        f = L["mlp"]
        if S:
            for q in (1, 2) if f else (1,):
                out[f"l{i}.hc{q}.in"] = torch.randn(S, generator=g) * 0.7 + 0.6
                out[f"l{i}.hc{q}.out"] = torch.randn(S, generator=g) * 0.7 + 0.8
                out[f"l{i}.hc{q}.mix"] = torch.eye(S) * 0.7 + torch.randn((S, S), generator=g) * 0.35
        if f and f["kind"] == "dense":
            out[f"l{i}.mlp.act"] = torch.tensor([0.9, -0.6, 0.4, 0.25])
    return out


def tables(cfg, seed):
    """Expert tables with rows of different experts, drawn per token id."""
    g = torch.Generator().manual_seed(seed + 1)
    out = {}
    for i, L in enumerate(cfg["layers"]):
        f = L["mlp"]
        if f and f["kind"] == "moe":
            E, k = f["router"]["experts"], f["router"]["top"]
            out[f"l{i}.mlp.table"] = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(cfg["vocab"])]).to(torch.int32)
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
    new.update(tables(config, seed))
    new.update(replace or {})
    for n, t in new.items():
        assert n in tensors and tuple(tensors[n].shape) == tuple(t.shape), n
        tensors[n] = t.contiguous() if t.dtype == torch.int32 else t.to(torch.bfloat16).contiguous()
    save_file(tensors, path)
    return out_dir
