"""Grouped-query softmax attention with one norm over the whole query and key projections, a
rotation, values of their own and an elementwise output gate.

With H query heads, G key/value heads (query head h reads head ``h // (H / G)``), key size D, value
size Dv and the layer's input x:

    q = W_q x + b_q,  k = W_k x + b_k,  v = W_v x + b_v
    q' = q / rms(q) * w_qn,  k' = k / rms(k) * w_kn        one norm over the WHOLE projection, all heads
                                                           at once, weights of the projection's width
    then the first `rot` dimensions of every q' and k' head turned by the position
    s(i, j) = (q'_h(i) . k'(j)) * scale,  j seen from i iff j <= i,  p = softmax over the seen j
    out = W_o (concat_h(sum_j p_h(i, j) v(j)) * sigmoid(W_g x))     the gate element by element

The cache keeps k' (after norm and rotation) and v.  With Dv == D (a multiple of 16) they lie in the
usual head-major pages, which the flash, split-key and tcgen05 attention kernels read; otherwise one
row a token ``[k' | v]``, which the kernels for unequal key and value sizes read.  A layer with
`own_kv` false has no key and value tensors: it is run against another layer's cache slot
(`LayerCall(cache=that layer, append=False)`) with queries, gate and output projection of its own.
Biases, the norms, the rotation and the gate can each be left out.  The projections that read x
(q, k, v and the gate) are one matrix, fused at load; its product is taken as float32 sums so that
biases and norms see unrounded values.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StepContext, TensorSpec


@register_part("mixer", "whole_norm_gated_attention")
class WholeNormGatedAttention(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("out", "o"), ("q_bias", "q.b"),
                     ("k_bias", "k.b"), ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 eps: float, prefix: str, position: Optional[PartSpec] = None, own_kv: bool = True, bias: bool = True,
                 gate: bool = True, tensor_names=None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.position = build_part("position", position) if position is not None else None
        self.own_kv, self.has_bias, self.has_gate = bool(own_kv), bool(bias), bool(gate)
        self.q_width = self.heads * self.head_dim
        self.k_width, self.v_width = self.kv_heads * self.head_dim, self.kv_heads * self.value_dim
        self.o_width = self.heads * self.value_dim
        # the usual pages (and their kernels) when keys and values are of one size those kernels take
        self.head_major = self.head_dim == self.value_dim and self.head_dim in kernels.SUPPORTED_HEAD_DIMS
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_o = self.b_q = self.b_k = self.b_v = self.q_norm = self.k_norm = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    # ---- weights ----------------------------------------------------------------------
    def _projections(self):
        return (("q", self.q_width),) + ((("k", self.k_width), ("v", self.v_width)) if self.own_kv else ()) + \
            ((("gate", self.o_width),) if self.has_gate else ())

    def tensor_specs(self) -> List[TensorSpec]:
        W = self.hidden_size
        specs = [TensorSpec(self._n(n), (width, W)) for n, width in self._projections()]
        specs.append(TensorSpec(self._n("out"), (W, self.o_width)))
        kv = ("q", "k", "v") if self.own_kv else ("q",)
        width = {"q": self.q_width, "k": self.k_width, "v": self.v_width}
        if self.has_bias:
            specs += [TensorSpec(self._n(n + "_bias"), (width[n],), role="vector") for n in kv]
        specs += [TensorSpec(self._n(n + "_norm"), (width[n],), role="vector", init="norm") for n in kv if n != "v"]
        return specs

    def load(self, fetch: Fetch) -> None:
        self.w_in = torch.cat([fetch(self._n(n)) for n, _ in self._projections()], dim=0).contiguous()
        self.w_o = fetch(self._n("out"))
        if self.has_bias:
            self.b_q = fetch(self._n("q_bias"))
            if self.own_kv:
                self.b_k, self.b_v = fetch(self._n("k_bias")), fetch(self._n("v_bias"))
        self.q_norm = fetch(self._n("q_norm"))
        self.k_norm = fetch(self._n("k_norm")) if self.own_kv else None

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    # ---- cache ------------------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        if self.head_major:
            return CacheSpec("full", self.kv_heads, self.head_dim)
        return CacheSpec("full", row_width=self.k_width + self.v_width)

    def check_limits(self, dtype: torch.dtype, max_context: int, page_size: int) -> None:
        if self.head_major:
            kernels.check_attention_limits(dtype, self.head_dim, max_context, page_size)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert cache is not None, "attention needs a cache slot"
        if cache.append != self.own_kv:
            raise RuntimeError("a layer with keys of its own appends them; one without reads another layer's slot")
        H, G, D, Dv = self.heads, self.kv_heads, self.head_dim, self.value_dim
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)        # float32 sums [T, q | k | v | gate]
        inv_freq, rot, magnitude = None, 0, 1.0
        if self.position is not None:
            inv_freq, rot = self.position.rotary_table(x.device)
            magnitude = float(self.position.magnitude)
        k0 = self.q_width
        v0 = k0 + self.k_width
        g0 = v0 + self.v_width if self.own_kv else k0
        q = kernels.whole_norm_rope_append(proj, 0, k0, v0, self.b_q, self.b_k, self.b_v, self.q_norm, self.k_norm,
                                           self.eps, inv_freq, rot, magnitude, H, G if self.own_kv else 0, D, Dv, ctx,
                                           cache.pages, cache.block_table, cache.page_size, x.dtype)
        if self.head_major:
            o = kernels.paged_attention(q, H, G, D, cache.pages, cache.block_table, cache.page_size, ctx, 0, self.scale)
        else:
            o = kernels.talking_attention(q, H, G, D, Dv, cache.pages, cache.block_table, cache.page_size, ctx, 0,
                                          self.scale, None, None)
        if self.has_gate:
            o = kernels.sigmoid_gate_rows(o, proj, g0)
        return kernels.linear(o, self.w_o)
