"""Grouped-query softmax attention whose heads talk before the softmax, over chunks, with a sink.

With H query heads, G key/value heads (query head h reads head ``h // (H / G)``), key size D, value
size Dv and the layer's input x:

    q = W_q x + b_q,  k = W_k x + b_k,  v = W_v x + b_v
    q, k: RMS norm per head over D with one weight vector for all heads, then the first `rot`
          dimensions turned by the position (pairs (i, i + rot/2))
    s_g(i, j)  = (q_g(i) . k(j)) * scale
    s'_h(i, j) = sum_g talk[h, g] s_g(i, j)                 the heads' scores are mixed
    j is seen from i  iff  j <= i and (no chunk or i // chunk == j // chunk)
    p_h(i, .)  = softmax over the seen j, with exp(sink_h) added to the denominator
    out = W_o concat_h(sum_j p_h(i, j) v(j)) + b_o

Chunks are counted from a request's position 0, not from where a prompt was cut.  The cache keeps
one row a token, ``[k after norm and rotation | v]``, so key and value sizes may differ.  A layer
with `own_kv` false has no key and value tensors: it is run against another layer's cache slot
(`LayerCall(cache=that layer, append=False)`) with queries, mask, talk and sink of its own.
The mixing, the sink, the chunks, the norms, the rotation and the biases can each be left out.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StepContext, TensorSpec


@register_part("mixer", "talking_heads_attention")
class TalkingHeadsAttention(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("out", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
                     ("v_bias", "v.b"), ("out_bias", "o.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                     ("talk", "talk"), ("sink", "sink"))

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 eps: float, prefix: str, chunk: Optional[int] = None, position: Optional[PartSpec] = None,
                 own_kv: bool = True, bias: bool = True, qk_norm: bool = True, talk: bool = True, sink: bool = True,
                 tensor_names=None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.chunk = int(chunk) if chunk else 0
        self.position = build_part("position", position) if position is not None else None
        self.own_kv, self.has_bias, self.qk_norm = bool(own_kv), bool(bias), bool(qk_norm)
        self.has_talk, self.has_sink = bool(talk), bool(sink)
        self.q_width = self.heads * self.head_dim
        self.k_width, self.v_width = self.kv_heads * self.head_dim, self.kv_heads * self.value_dim
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.b_in = self.w_o = self.b_o = self.q_norm = self.k_norm = self.talk = self.sink = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    # ---- weights ----------------------------------------------------------------------
    def _projections(self):
        return ("q", "k", "v") if self.own_kv else ("q",)

    def tensor_specs(self) -> List[TensorSpec]:
        W, H = self.hidden_size, self.heads
        width = {"q": self.q_width, "k": self.k_width, "v": self.v_width}
        specs = [TensorSpec(self._n(n), (width[n], W)) for n in self._projections()]
        specs.append(TensorSpec(self._n("out"), (W, H * self.value_dim)))
        if self.has_bias:
            specs += [TensorSpec(self._n(n + "_bias"), (width[n],), role="vector") for n in self._projections()]
            specs.append(TensorSpec(self._n("out_bias"), (W,), role="vector"))
        if self.qk_norm:
            specs.append(TensorSpec(self._n("q_norm"), (self.head_dim,), role="vector", init="norm"))
            if self.own_kv:
                specs.append(TensorSpec(self._n("k_norm"), (self.head_dim,), role="vector", init="norm"))
        if self.has_talk:
            specs.append(TensorSpec(self._n("talk"), (H, H), role="vector"))
        if self.has_sink:
            specs.append(TensorSpec(self._n("sink"), (H,), role="vector"))
        return specs

    def load(self, fetch: Fetch) -> None:
        self.w_in = torch.cat([fetch(self._n(n)) for n in self._projections()], dim=0).contiguous()
        self.w_o = fetch(self._n("out"))
        if self.has_bias:
            self.b_in = torch.cat([fetch(self._n(n + "_bias")) for n in self._projections()]).contiguous()
            self.b_o = fetch(self._n("out_bias"))
        if self.qk_norm:
            self.q_norm = fetch(self._n("q_norm"))
            self.k_norm = fetch(self._n("k_norm")) if self.own_kv else None
        self.talk = fetch(self._n("talk")).contiguous() if self.has_talk else None
        self.sink = fetch(self._n("sink")) if self.has_sink else None

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    # ---- cache ------------------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        # every key stays: a layer that reads this slot may look further back than this one
        return CacheSpec("full", row_width=self.k_width + self.v_width)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert cache is not None, "attention needs a cache slot"
        if cache.append != self.own_kv:
            raise RuntimeError("a layer with keys of its own appends them; one without reads another layer's slot")
        H, G, D, Dv = self.heads, self.kv_heads, self.head_dim, self.value_dim
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)        # float32 sums [T, q | k | v]
        inv_freq, rot = (None, 0)
        if self.position is not None:
            inv_freq, rot = self.position.rotary_table(x.device)
        q = kernels.head_norm_rope_append(proj, self.b_in, self.q_norm, self.k_norm, self.eps, inv_freq, rot, ctx,
                                          H, G if self.own_kv else 0, D, Dv, cache.pages, cache.block_table,
                                          cache.page_size, x.dtype)
        o = kernels.talking_attention(q, H, G, D, Dv, cache.pages, cache.block_table, cache.page_size, ctx,
                                      self.chunk, self.scale, self.talk, self.sink)
        y = kernels.linear(o, self.w_o, out_dtype=torch.float32 if self.b_o is not None else None)
        if self.b_o is not None:
            y = kernels.add_bias_rows(y, self.b_o, x.dtype)
        return y
