"""Fetezen: its config.json keys, and configuration -> plan of parts.

A decoder-only model whose layers are listed one by one in config.json.  A token carries several
residual streams (hyper-connections): each sublayer reads a learned combination of them, normed by
an RMS norm taken in groups, and its output changes all streams through a learned mix.  Every layer
has an ``attention`` mixer: grouped-query softmax attention with biases, a per-head RMS norm on
queries and keys, a rotation over the first dimensions of each head, the heads' scores mixed by a
learned matrix before the softmax, a mask of chunks counted from position 0, a learned sink in the
softmax's denominator, and key and value sizes of their own; a layer may read another layer's keys
and values instead of projecting its own (``kv_from``).  The feed-forward is dense with the
polynomial-of-norms activation, or a mixture of ungated GELU experts chosen by a table over token
ids, with a gated shared expert.  The logits are capped by a tanh.

config.json (every size and constant comes from here or from a tensor's shape)::

    architecture   "Fetezen"
    vocab, width, streams?, logit_softcap?
    norm           {eps, groups?}
    layers[i]      {type: "attention", mixer, mlp}
      mixer  {heads, kv_heads, dim, vdim, scale, rot?: {base, dims}, mask?: {size}, kv_from?: j}
      mlp    null, {kind: "dense", ff}, or
             {kind: "moe", expert: {ff}, router: {experts, top}, shared?: {ff}}

Tensors: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.hc1.{in,out,mix}``, ``l<i>.hc2.{in,out,mix}``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec, opt_float, req_int)
from ..registry import register_architecture

LAYER_TYPES = ("attention",)
_NAMES = (("norm1", "norm1"), ("mixer", "mix"), ("norm2", "norm2"), ("feed_forward", "mlp"),
          ("connect1", "hc1"), ("connect2", "hc2"))


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
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int               # 0: nothing is turned
    chunk: int                  # 0: every earlier position is seen
    kv_from: Optional[int]


@dataclass(frozen=True)
class MlpSizes:
    kind: str                   # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0


@dataclass(frozen=True)
class FetezenLayer:
    type: str
    mixer: AttentionSizes
    mlp: Optional[MlpSizes]


def _attention(m: Dict[str, Any], where: str, n_layers: int, i: int) -> AttentionSizes:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads={heads} is not a multiple of kv_heads={kv}")
    dim = _int(m, "dim", where)
    base, dims = 10000.0, 0
    if m.get("rot") is not None:
        rot = _obj(m, "rot", where)
        dims, base = _int(rot, "dims", where + "rot.", least=0), _float(rot, "base", where + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most dim={dim}")
        if base <= 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
    chunk = 0
    if m.get("mask") is not None:
        chunk = _int(_obj(m, "mask", where), "size", where + "mask.")
    src = m.get("kv_from")
    if src is not None:
        src = _int(m, "kv_from", where, least=0)
        if src >= n_layers or src == i:
            raise ConfigError(f"config.json: {where}kv_from={src} names no other layer")
    return AttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=_int(m, "vdim", where),
                          scale=_float(m, "scale", where), rot_base=base, rot_dims=dims, chunk=chunk, kv_from=src)


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
        out = MlpSizes("moe", ff=_int(ex, "ff", where + "expert."), experts=_int(ro, "experts", where + "router."),
                       top=_int(ro, "top", where + "router."),
                       shared_ff=_int(_obj(f, "shared", where), "ff", where + "shared.") if f.get("shared") is not None else 0)
        if out.top > out.experts:
            raise ConfigError(f"config.json: {where}router.top={out.top} exceeds experts={out.experts}")
        return out
    raise ConfigError(f"config.json: {where}kind = {kind!r}; known: ['dense', 'moe']")


@dataclass(frozen=True)
class FetezenConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    streams: Optional[int]          # None: one stream and the plain residual sum
    logit_softcap: float            # 0: none
    layers: Tuple[FetezenLayer, ...]

    ARCHITECTURE = "Fetezen"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FetezenConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[FetezenLayer] = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type = {kind!r}; known: {list(LAYER_TYPES)}")
            layers.append(FetezenLayer(kind, _attention(_obj(L, "mixer", where), where + "mixer.", len(raw), i),
                                       _mlp(L.get("mlp"), where + "mlp.")))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from
            if j is None:
                continue
            o = layers[j].mixer
            if o.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j}: that layer has no keys of its own")
            if (o.kv_heads, o.dim, o.vdim) != (L.mixer.kv_heads, L.mixer.dim, L.mixer.vdim):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layer {j} but its "
                                  "key heads or sizes differ")
            if j > i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} names a later layer")
        norm = _obj(d, "norm", "")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        groups = _int(norm, "groups", "norm.") if norm.get("groups") is not None else 1
        width = _int(d, "width", "")
        if width % groups:
            raise ConfigError(f"config.json: norm.groups={groups} does not divide width={width}")
        streams = _int(d, "streams", "") if d.get("streams") is not None else None
        cap = _float(d, "logit_softcap", "") if d.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return cls(vocab=_int(d, "vocab", ""), width=width, eps=eps, groups=groups, streams=streams,
                   logit_softcap=cap, layers=tuple(layers))


def _mixer_spec(cfg: FetezenConfig, m: AttentionSizes) -> PartSpec:
    position = None
    if m.rot_dims:
        position = PartSpec.make("rotary_half_split", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims)
    return PartSpec.make("talking_heads_attention", hidden_size=cfg.width, heads=m.heads, kv_heads=m.kv_heads,
                         head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=cfg.eps, chunk=m.chunk or None,
                         position=position, own_kv=m.kv_from is None, bias=True, qk_norm=True, talk=True, sink=True)


def _ff_spec(cfg: FetezenConfig, f: Optional[MlpSizes]) -> PartSpec:
    if f is None:
        return PartSpec.make("none")
    if f.kind == "dense":
        return PartSpec.make("dense_poly_norm", hidden_size=cfg.width, intermediate_size=f.ff, eps=cfg.eps)
    return PartSpec.make("table_routed_gelu", hidden_size=cfg.width, num_experts=f.experts, top_k=f.top,
                         vocab_size=cfg.vocab, moe_intermediate_size=f.ff, shared_intermediate_size=f.shared_ff)


def build_plan(cfg: FetezenConfig) -> ModelPlan:
    norm = PartSpec.make("group_rms_norm", size=cfg.width, eps=cfg.eps, groups=cfg.groups, weight_name="")
    arrangement = (("streams", cfg.streams or 1), ("learned", cfg.streams is not None))
    layers = tuple(LayerSpec("hyper_connections", norm, _mixer_spec(cfg, L.mixer), _ff_spec(cfg, L.mlp),
                             prefix=f"l{i}.", names=_NAMES, arrangement_params=arrangement)
                   for i, L in enumerate(cfg.layers))
    # a layer with keys of its own appends to its own slot; one without reads its source's
    order = tuple(LayerCall(i, i if L.mixer.kv_from is None else L.mixer.kv_from, L.mixer.kv_from is None)
                  for i, L in enumerate(cfg.layers))
    return ModelPlan(vocab_size=cfg.vocab, hidden_size=cfg.width, layers=layers, order=order, final_norm=norm,
                     tie_word_embeddings=False, embedding_name="embed", final_norm_name="final.norm.",
                     head_name="head", streams=cfg.streams or 1, logit_softcap=cfg.logit_softcap)


register_architecture(FetezenConfig.ARCHITECTURE, FetezenConfig.from_dict, build_plan)
