"""Kopadra: its config.json keys, and configuration -> plan of parts.

A decoder-only model whose layers are listed one by one in config.json.  Every layer is pre-norm
(layer norm with a weight, no bias): ``x += mixer(norm1(x))``, then ``x += ff(norm2(x))``.  Two mixers:

* ``attention``: grouped-query softmax attention with biases on q, k and v, one RMS norm over the whole
  q and the whole k projection, a rotation of the first dimensions of every head whose frequencies may be
  stretched for long contexts (``rot.scaling``), a score scale from the configuration, key and value
  sizes of their own, and an output gate ``sigmoid(W_g h)`` element by element before the out-projection.
  A layer may read another layer's keys and values instead of projecting its own (``kv_from``).
* ``mlstm``: a matrix-memory recurrence with exponential gates capped by a tanh and stabilised by a
  running maximum; each head's output over its root mean square, a weight, a sigmoid gate.

The feed-forward is dense and gated with the tanh GELU, or a mixture of SiLU-gated experts: softmax
scores over all experts, a correction added for the choice only, experts chosen among the best groups,
identity experts (their output is their input), weights divided by their sum and scaled, and a shared
expert that is added for every token.  The head is the embedding table; the logits are capped by a tanh.

config.json (every size and constant comes from here or from a tensor's shape)::

    architecture   "Kopadra"
    vocab, width, logit_softcap?
    norm           {eps}
    layers[i]      {type: "attention" | "mlstm", mixer, mlp}
      attention mixer  {heads, kv_heads, dim, vdim, scale, kv_from?: j,
                        rot?: {base, dims, scaling?: {factor, original, fast, slow}}}
      mlstm mixer      {heads, dim, vdim, gate_cap?}
      mlp    null, {kind: "dense", ff}, or
             {kind: "moe", expert: {ff}, shared?: {ff},
              router: {experts, top, identity?, scale?, groups?: {count, keep}}}

Tensors: ``embed``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*`` (experts ``e<n>.{gate,up,down}``, ``router``, ``correction``, ``shared.{gate,up,down}``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec, opt_float, req_int)
from ..registry import register_architecture

LAYER_TYPES = ("attention", "mlstm")
_NAMES = (("norm1", "norm1"), ("mixer", "mix"), ("norm2", "norm2"), ("feed_forward", "mlp"))


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _float(d: Dict[str, Any], key: str, where: str) -> float:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {where}{key!r} is missing")
    try:
        return opt_float(d, key, 0.0)
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}")) from None


def _int(d: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    try:
        v = req_int(d, key)
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}")) from None
    if v < least:
        raise ConfigError(f"config.json: {where}{key!r} must be at least {least}, got {v}")
    return v


@dataclass(frozen=True)
class RotationSizes:
    base: float
    dims: int
    # (factor, original, fast, slow) of the stretched frequencies, or None for the plain ones
    scaling: Optional[Tuple[float, float, float, float]]


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationSizes]
    kv_from: Optional[int]


@dataclass(frozen=True)
class MlstmSizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float             # 0: the gates' projections enter uncapped


@dataclass(frozen=True)
class MlpSizes:
    kind: str                   # "dense" | "moe"
    ff: int
    experts: int = 0            # experts with matrices
    identity: int = 0           # further experts whose output is their input
    top: int = 0
    scale: float = 1.0
    groups: Optional[Tuple[int, int]] = None    # (count, keep)
    shared_ff: int = 0


@dataclass(frozen=True)
class KopadraLayer:
    type: str
    mixer: Any                  # AttentionSizes | MlstmSizes
    mlp: Optional[MlpSizes]


def _rotation(m: Dict[str, Any], where: str, dim: int) -> Optional[RotationSizes]:
    if m.get("rot") is None:
        return None
    rot = _obj(m, "rot", where)
    where += "rot."
    dims, base = _int(rot, "dims", where, least=0), _float(rot, "base", where)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}dims={dims} must be even and at most dim={dim}")
    if base <= 1:
        raise ConfigError(f"config.json: {where}base must be above 1")
    if dims == 0:
        return None
    scaling = None
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", where)
        scaling = tuple(_float(sc, k, where + "scaling.") for k in ("factor", "original", "fast", "slow"))
        if scaling[0] < 1 or min(scaling[1:]) <= 0:
            raise ConfigError(f"config.json: {where}scaling needs factor >= 1 and positive original, fast, slow")
    return RotationSizes(base, dims, scaling)


def _attention(m: Dict[str, Any], where: str, n_layers: int, i: int) -> AttentionSizes:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads={heads} is not a multiple of kv_heads={kv}")
    dim = _int(m, "dim", where)
    src = m.get("kv_from")
    if src is not None:
        src = _int(m, "kv_from", where, least=0)
        if src >= n_layers or src == i:
            raise ConfigError(f"config.json: {where}kv_from={src} names no other layer")
    return AttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=_int(m, "vdim", where), scale=_float(m, "scale", where),
                          rot=_rotation(m, where, dim), kv_from=src)


def _mlstm(m: Dict[str, Any], where: str) -> MlstmSizes:
    cap = _float(m, "gate_cap", where) if m.get("gate_cap") is not None else 0.0
    if cap < 0:
        raise ConfigError(f"config.json: {where}gate_cap must be positive")
    return MlstmSizes(heads=_int(m, "heads", where), dim=_int(m, "dim", where), vdim=_int(m, "vdim", where), gate_cap=cap)


def _mlp(f: Optional[Dict[str, Any]], where: str) -> Optional[MlpSizes]:
    if f is None:
        return None
    if not isinstance(f, dict):
        raise ConfigError(f"config.json: {where[:-1]} must be an object or null")
    kind = f.get("kind")
    if kind == "dense":
        return MlpSizes("dense", ff=_int(f, "ff", where))
    if kind == "moe":
        ex, ro = _obj(f, "expert", where), _obj(f, "router", where)
        w = where + "router."
        experts, top = _int(ro, "experts", w), _int(ro, "top", w)
        identity = _int(ro, "identity", w, least=0) if ro.get("identity") is not None else 0
        scale = _float(ro, "scale", w) if ro.get("scale") is not None else 1.0
        groups = None
        if ro.get("groups") is not None:
            g = _obj(ro, "groups", w)
            groups = (_int(g, "count", w + "groups."), _int(g, "keep", w + "groups."))
            total = experts + identity
            if total % groups[0] or groups[1] > groups[0] or (total // groups[0]) * groups[1] < top:
                raise ConfigError(f"config.json: {w}groups: {total} experts in {groups[0]} groups of which {groups[1]} "
                                  f"are kept cannot give top={top} choices")
        if top > experts + identity:
            raise ConfigError(f"config.json: {w}top={top} exceeds the {experts + identity} experts")
        return MlpSizes("moe", ff=_int(ex, "ff", where + "expert."), experts=experts, identity=identity, top=top,
                        scale=scale, groups=groups,
                        shared_ff=_int(_obj(f, "shared", where), "ff", where + "shared.") if f.get("shared") is not None else 0)
    raise ConfigError(f"config.json: {where}kind = {kind!r}; known: ['dense', 'moe']")


@dataclass(frozen=True)
class KopadraConfig:
    vocab: int
    width: int
    eps: float
    logit_softcap: float            # 0: none
    layers: Tuple[KopadraLayer, ...]

    ARCHITECTURE = "Kopadra"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KopadraConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[KopadraLayer] = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type = {kind!r}; known: {list(LAYER_TYPES)}")
            m = _obj(L, "mixer", where)
            mixer = _attention(m, where + "mixer.", len(raw), i) if kind == "attention" else _mlstm(m, where + "mixer.")
            layers.append(KopadraLayer(kind, mixer, _mlp(L.get("mlp"), where + "mlp.")))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from if L.type == "attention" else None
            if j is None:
                continue
            if layers[j].type != "attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j}: that layer has no keys of its own")
            o = layers[j].mixer
            if (o.kv_heads, o.dim, o.vdim, o.rot) != (L.mixer.kv_heads, L.mixer.dim, L.mixer.vdim, L.mixer.rot):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layer {j} but its "
                                  "key heads, sizes or rotation differ")
            if j > i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} names a later layer")
        norm = _obj(d, "norm", "")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        cap = _float(d, "logit_softcap", "") if d.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps, logit_softcap=cap, layers=tuple(layers))


def _position_spec(m: AttentionSizes) -> Optional[PartSpec]:
    if m.rot is None:
        return None
    if m.rot.scaling is None:
        return PartSpec.make("rotary_half_split", head_dim=m.dim, theta=m.rot.base, rotary_dim=m.rot.dims)
    factor, original, fast, slow = m.rot.scaling
    return PartSpec.make("rotary_half_split_blended", head_dim=m.dim, theta=m.rot.base, rotary_dim=m.rot.dims,
                         factor=factor, original=original, fast=fast, slow=slow)


def _mixer_spec(cfg: KopadraConfig, L: KopadraLayer) -> PartSpec:
    m = L.mixer
    if L.type == "mlstm":
        return PartSpec.make("mlstm", hidden_size=cfg.width, heads=m.heads, dim=m.dim, value_dim=m.vdim, eps=cfg.eps,
                             gate_cap=m.gate_cap or None)
    return PartSpec.make("whole_norm_gated_attention", hidden_size=cfg.width, heads=m.heads, kv_heads=m.kv_heads,
                         head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=cfg.eps, position=_position_spec(m),
                         own_kv=m.kv_from is None, bias=True, gate=True)


_DENSE_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))
_MOE_NAMES = (("router", "router"), ("correction", "correction"), ("gate", "e{e}.gate"), ("up", "e{e}.up"),
              ("down", "e{e}.down"), ("shared_gate", "shared.gate"), ("shared_up", "shared.up"),
              ("shared_down", "shared.down"))


def _ff_spec(cfg: KopadraConfig, f: Optional[MlpSizes]) -> PartSpec:
    if f is None:
        return PartSpec.make("none")
    if f.kind == "dense":
        return PartSpec.make("dense_swiglu", hidden_size=cfg.width, intermediate_size=f.ff, activation=("gelu_tanh",),
                             tensor_names=_DENSE_NAMES)
    return PartSpec.make("sparse_moe_swiglu", hidden_size=cfg.width, num_experts=f.experts, top_k=f.top,
                         norm_topk_prob=True, moe_intermediate_size=f.ff, shared_intermediate_size=f.shared_ff,
                         tensor_names=_MOE_NAMES, correction=True, groups=f.groups, identity_experts=f.identity,
                         route_scale=f.scale, shared_gate=False)


def build_plan(cfg: KopadraConfig) -> ModelPlan:
    norm = PartSpec.make("layer_norm", size=cfg.width, eps=cfg.eps, weight_name="")
    layers = tuple(LayerSpec("pre_norm", norm, _mixer_spec(cfg, L), _ff_spec(cfg, L.mlp), prefix=f"l{i}.", names=_NAMES)
                   for i, L in enumerate(cfg.layers))
    # a layer with keys of its own appends to its own slot; one without reads its source's
    order = []
    for i, L in enumerate(cfg.layers):
        src = L.mixer.kv_from if L.type == "attention" else None
        order.append(LayerCall(i, i if src is None else src, src is None))
    return ModelPlan(vocab_size=cfg.vocab, hidden_size=cfg.width, layers=layers, order=tuple(order), final_norm=norm,
                     tie_word_embeddings=True, embedding_name="embed", final_norm_name="final.norm.",
                     logit_softcap=cfg.logit_softcap)


register_architecture(KopadraConfig.ARCHITECTURE, KopadraConfig.from_dict, build_plan)
