"""A plain, slow, whole-sequence implementation of the Kopadra design, one function per mechanism.

Written from the design's equations in double precision on the CPU with torch's elementary
operations only; it shares no code with the engine.  `forward(cfg, w, tokens)` runs one request's
tokens at once and returns the logits of every position (and the stream after every layer).

The design: pre-norm layers (layer norm with a weight, no bias) around a mixer and a feed-forward.
Mixers: grouped-query softmax attention (biases, one RMS norm over the whole q and the whole k
projection, a rotation of the first dimensions of each head with frequencies blended between the
plain and the stretched ones, an elementwise sigmoid output gate; a layer may read another layer's
keys and values), or a matrix-memory recurrence (mLSTM) with capped exponential gates and a running
maximum.  Feed-forwards: dense gated with the tanh GELU, or routed SiLU-gated experts chosen among
groups with a correction added to the choice scores only, identity experts, and a shared expert.
The logits come from the embedding table and are capped by a tanh.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64

# (generator, size) or None: every projection's output is disturbed by that fraction of itself, which shows the
# rows whose logits hang on a near-cancellation (they are as touchy to a rounding of the projections)
NOISE = None


def proj(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    y = h @ w.T
    if NOISE is not None:
        y = y * (1.0 + NOISE[1] * torch.randn(y.shape, generator=NOISE[0], dtype=F64))
    return y


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotary_frequencies(rot: Dict) -> Tuple[torch.Tensor, float]:
    """(frequency of pair i for i < dims / 2, factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Dict]) -> torch.Tensor:
    """x [T, heads, dim]: the first rot.dims of each head turned, pair (i, i + dims / 2)."""
    if not rot or not int(rot["dims"]):
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    a = positions.to(F64)[:, None] * f[None, :]                      # [T, dims / 2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float,
                          positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """What a layer with keys of its own keeps per token: keys after norm and rotation, values."""
    G, D, Dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = proj(h, w[p + "k"]) + w[p + "k.b"]
    v = proj(h, w[p + "v"]) + w[p + "v.b"]
    k = rms(k, eps) * w[p + "k.norm"]
    k = rotate(k.view(-1, G, D), positions, m.get("rot"))
    return k, v.view(-1, G, Dv)


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float,
                    positions: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """h [T, width]; k [T, G, D], v [T, G, Dv] are the keys and values it reads (its own or another layer's)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = proj(h, w[p + "q"]) + w[p + "q.b"]
    q = rms(q, eps) * w[p + "q.norm"]
    q = rotate(q.view(T, H, D), positions, m.get("rot"))
    out = torch.zeros((T, H, Dv), dtype=F64)
    causal = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~causal, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(proj(h, w[p + "g"]))
    return proj(out.reshape(T, H * Dv) * gate, w[p + "o"])


def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (proj(h, w[p + "q"])).view(T, H, D) * D ** -0.5
    k = (proj(h, w[p + "k"])).view(T, H, D)
    v = (proj(h, w[p + "v"])).view(T, H, Dv)
    cap = m.get("gate_cap")
    capped = (lambda z: float(cap) * torch.tanh(z / float(cap))) if cap else (lambda z: z)       # no cap given: as they are
    ig = capped(h @ w[p + "i"].T + w[p + "i.b"])                                        # [T, H] log input gate
    fg = torch.nn.functional.logsigmoid(capped(h @ w[p + "f"].T + w[p + "f.b"]))
    out = torch.zeros((T, H, Dv), dtype=F64)
    for hd in range(H):
        S = torch.zeros((D, Dv), dtype=F64)
        n = torch.zeros((D,), dtype=F64)
        mx = 0.0
        for t in range(T):
            f, i = float(fg[t, hd]), float(ig[t, hd])
            m_new = max(f + mx, i)
            a, b = math.exp(f + mx - m_new), math.exp(i - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            den = max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = rms(out, eps).reshape(T, H * Dv) * w[p + "norm"]
    return proj(o * torch.sigmoid(proj(h, w[p + "g"])), w[p + "o"])


def gated_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, act) -> torch.Tensor:
    return proj(act(proj(h, w[p + "gate"])) * proj(h, w[p + "up"]), w[p + "down"])


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, r: Dict, chosen=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top]); experts >= r.experts are identity experts.
    `chosen`: the experts are given (someone else's choice), only the weights are worked out."""
    E = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)                                    # [T, E]
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = E // count
        best = choice.view(-1, count, per).max(dim=-1).values                            # [T, count]
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    idx = torch.topk(choice, top, dim=-1).indices if chosen is None else chosen
    wt = torch.gather(s, 1, idx)
    wt = wt / (wt.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return idx, wt


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: Dict, chosen=None) -> torch.Tensor:
    r = f["router"]
    real = int(r["experts"])
    idx, wt = route(h, w, p, r, chosen)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y = h[t] if e >= real else gated_mlp(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
            out[t] += wt[t, j] * y
    if f.get("shared"):
        out = out + gated_mlp(h, w, p + "shared.", silu)
    return out


def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], chosen=None):
    """-> (logits [T, vocab], streams [layers, T, width]) in double precision.  `chosen`: for every routed
    layer in order, the experts [T, top] to use instead of the model's own choice."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    kept: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    streams = []
    routed = 0
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, w, p + "mix.", m, eps, positions)
                src = i
            x = x + attention_mixer(h, w, p + "mix.", m, eps, positions, *kept[src])
        elif L["type"] == "mlstm":
            x = x + mlstm_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f:
            h = layer_norm(x, w[p + "norm2"], eps)
            if f["kind"] == "dense":
                x = x + gated_mlp(h, w, p + "mlp.", gelu_tanh)
            else:
                x = x + moe(h, w, p + "mlp.", f, None if chosen is None else chosen[routed])
                routed += 1
        streams.append(x.clone())
    h = layer_norm(x, w["final.norm"], eps)
    logits = h @ w["embed"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams)
