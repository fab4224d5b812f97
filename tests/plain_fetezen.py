"""A plain, slow statement of the Fetezen design: whole sequences on the CPU, one function per
mechanism, written from the design's equations and sharing no code with the engine.

`forward(config, tensors, tokens)` takes config.json's dictionary, the checkpoint's tensors by name
(any float dtype; integer tables as they are) and one request's token ids, and returns float64
logits ``[tokens, vocab]`` and the summed residual streams after every layer.  Everything runs in
float64 unless `dtype` says otherwise, so that it can stand as the exact answer.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def group_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis is cut into `groups` equal consecutive parts; each part is divided by its own
    sqrt(mean(part^2) + eps); the whole is multiplied by w."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half_split(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, D]: dimension i < dims/2 is paired with i + dims/2 and the pair is turned by
    positions * base^(-2i/dims); dimensions from `dims` on pass unchanged."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                     # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, chunk: Optional[int]) -> torch.Tensor:
    """[T, T] bool: key j is seen from position i iff j <= i and, with chunks, both lie in the same
    chunk counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor, seen: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T]; the denominator also holds exp(sink_h), which has no key and no value."""
    s = scores.masked_fill(~seen[None], -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def keys_and_values(m: Dict, t: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor,
                    eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """What a layer with projections of its own puts into its cache: keys after norm and rotation
    [T, G, D], values [T, G, Dv]."""
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, D)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(T, G, Dv)
    k = unit_rms(k, eps) * t[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        k = rotate_half_split(k, positions, float(rot["base"]), int(rot["dims"]))
    return k, v


def attention(m: Dict, t: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor, eps: float,
              kv: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, D)
    q = unit_rms(q, eps) * t[p + "q.norm"]
    rot = m.get("rot")
    if rot:
        q = rotate_half_split(q, positions, float(rot["base"]), int(rot["dims"]))
    k, v = kv
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)                                 # query head h reads key head h // rep
    vh = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kh) * float(m["scale"])
    scores = torch.einsum("hg,gij->hij", t[p + "talk"], scores)          # heads' scores mixed before the mask
    mask = m.get("mask")
    w = sink_softmax(scores, t[p + "sink"], visible(T, int(mask["size"]) if mask else None))
    o = torch.einsum("hij,jhd->ihd", w, vh).reshape(T, H * Dv)
    return o @ t[p + "o"].T + t[p + "o.b"]


def poly_norm(z: torch.Tensor, act: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = [act[i] for i in range(4)]
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(t: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    return poly_norm(h @ t[p + "up"].T, t[p + "act"], eps) @ t[p + "down"].T


def expert(t: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return gelu_erf(h @ t[p + "up"].T) @ t[p + "down"].T


def table_moe(f: Dict, t: Dict[str, torch.Tensor], p: str, h: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Each token id's experts stand in a table; every chosen expert weighs 1/top."""
    top = int(f["router"]["top"])
    chosen = t[p + "table"][tokens.long()].long()                        # [T, top]
    out = torch.zeros_like(h)
    for r in range(h.shape[0]):
        for e in chosen[r].tolist():
            out[r] += expert(t, f"{p}e{e}.", h[r:r + 1])[0] / top
    if f.get("shared"):
        gate = torch.sigmoid(h @ t[p + "shared.sg"].T)                   # [T, 1]
        out = out + gate * expert(t, p + "shared.", h)
    return out


def feed_forward(f: Dict, t: Dict[str, torch.Tensor], p: str, h: torch.Tensor, tokens: torch.Tensor, eps: float):
    if f["kind"] == "dense":
        return dense_ff(t, p, h, eps)
    return table_moe(f, t, p, h, tokens)


def forward(config: Dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            positions: Optional[torch.Tensor] = None):
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    tok = torch.tensor(tokens, dtype=torch.long)
    T = tok.numel()
    pos = torch.arange(T) if positions is None else positions
    eps = float(config["norm"]["eps"])
    groups = int(config["norm"].get("groups") or 1)
    s = config.get("streams")
    x = t["embed"][tok]
    streams = [x.clone() for _ in range(int(s))] if s else None
    caches: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    after = []

    def sublayer(q: int, i: int, fn):
        nonlocal x, streams
        p = f"l{i}."
        w = t[f"{p}norm{q}"]
        if streams is None:
            x = x + fn(group_rms_norm(x, w, groups, eps))
            return
        hc = f"{p}hc{q}."
        u = sum(t[hc + "in"][a] * streams[a] for a in range(len(streams)))
        y = fn(group_rms_norm(u, w, groups, eps))
        mix, out = t[hc + "mix"], t[hc + "out"]                           # mix is indexed [from, to]
        streams = [sum(mix[a, b] * streams[a] for a in range(len(streams))) + out[b] * y
                   for b in range(len(streams))]

    for i, L in enumerate(config["layers"]):
        m, p = L["mixer"], f"l{i}.mix."

        def mixer(h, i=i, m=m, p=p):
            src = m.get("kv_from")
            if src is None:
                caches[i] = keys_and_values(m, t, p, h, pos, eps)
                src = i
            return attention(m, t, p, h, pos, eps, caches[src])

        sublayer(1, i, mixer)
        f = L.get("mlp")
        if f:
            sublayer(2, i, lambda h, f=f, i=i: feed_forward(f, t, f"l{i}.mlp.", h, tok, eps))
        after.append(x.clone() if streams is None else sum(streams))
    x = after[-1]
    logits = group_rms_norm(x, t["final.norm"], groups, eps) @ t["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits, after
