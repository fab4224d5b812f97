"""Matrix-memory recurrence with exponential gates (mLSTM), its state in the request's slot.

Per head, with q_t, k_t of size D, v_t of size V and the layer's input x_t:

    q = W_q x * D^-1/2,  k = W_k x,  v = W_v x
    i_t = cap tanh((w_i . x + b_i) / cap)                    log input gate, one number a head
    f_t = logsigmoid(cap tanh((w_f . x + b_f) / cap))        log forget gate
    m_t = max(f_t + m_{t-1}, i_t)                            running maximum, m_0 = 0
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T       (S, n start at zero)
    n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's o over its own root mean square; the heads side by side times a weight, times
``sigmoid(W_g x)``; out-projection.  What a request keeps between steps is (S, n, m) of every head,
float32, of fixed size (`state_spec`), so prompts cut into portions, decoded tokens and mixed batches
all run the same two kernels: one walks a request's rows for the gates' numbers and the normaliser
(``mlstm_gates``), the other is the linear-attention recurrence with a decay, an input factor and an
output factor a row (``decay_linear_attention`` with `gates`); both continue from the slot and leave it
updated.  Gates, maximum, decays, state and sums are 32-bit in both modes; everything that reads x is
one matrix, fused at load, whose product is taken as float32 sums, so q, k, v and the gates' projections
enter the recurrence unrounded.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import CacheView, Fetch, Mixer, StateSpec, StepContext, TensorSpec


@register_part("mixer", "mlstm")
class MatrixMemoryLstm(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("out", "o"), ("norm", "norm"),
                     ("input", "i"), ("forget", "f"), ("input_bias", "i.b"), ("forget_bias", "f.b"))

    def __init__(self, hidden_size: int, heads: int, dim: int, value_dim: int, eps: float, prefix: str,
                 gate_cap: Optional[float] = None, query_scale: Optional[float] = None, tensor_names=None):
        self.hidden_size, self.heads, self.dim, self.value_dim = int(hidden_size), int(heads), int(dim), int(value_dim)
        if not 1 <= self.dim <= kernels.LINEAR_ATTENTION_MAX_DIM:
            raise ValueError(f"dim {self.dim} outside 1..{kernels.LINEAR_ATTENTION_MAX_DIM}")
        self.eps, self.prefix = float(eps), prefix
        self.gate_cap = 0.0 if not gate_cap else float(gate_cap)           # 0: the gates' projections enter uncapped
        self.query_scale = self.dim ** -0.5 if query_scale is None else float(query_scale)
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.value_dim
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_o = self.norm_w = self.b_i = self.b_f = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    def tensor_specs(self) -> List[TensorSpec]:
        W, H = self.hidden_size, self.heads
        return [TensorSpec(self._n("q"), (self.qk_width, W)), TensorSpec(self._n("k"), (self.qk_width, W)),
                TensorSpec(self._n("v"), (self.v_width, W)), TensorSpec(self._n("gate"), (self.v_width, W)),
                TensorSpec(self._n("out"), (W, self.v_width)),
                TensorSpec(self._n("norm"), (self.v_width,), role="vector", init="norm"),
                TensorSpec(self._n("input"), (H, W)), TensorSpec(self._n("forget"), (H, W)),
                TensorSpec(self._n("input_bias"), (H,), role="vector"),
                TensorSpec(self._n("forget_bias"), (H,), role="vector", init="norm")]

    def load(self, fetch: Fetch) -> None:
        # one matrix for everything that reads x: q, k, v, the output gate and the two gates' projections
        self.w_in = torch.cat([fetch(self._n(n)) for n in ("q", "k", "v", "gate", "input", "forget")], dim=0).contiguous()
        self.w_o = fetch(self._n("out"))
        self.norm_w = fetch(self._n("norm"))
        self.b_i, self.b_f = fetch(self._n("input_bias")), fetch(self._n("forget_bias"))

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + 4 * self.v_width

    # ---- state ------------------------------------------------------------------------
    @property
    def _n_off(self) -> int:
        return self.heads * self.value_dim * self.dim

    @property
    def _m_off(self) -> int:
        return self._n_off + self.heads * self.dim

    def state_spec(self) -> StateSpec:
        """S of every head [heads][value column][dim], then n [heads][dim], then m [heads]; float32."""
        return StateSpec((self._m_off + self.heads,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert state is not None, "the recurrence needs a state slot"
        H, D, V = self.heads, self.dim, self.value_dim
        # float32 sums [T, q | k | v | gate | input | forget]: the recurrence takes them unrounded
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        i0 = 2 * self.qk_width + 2 * self.v_width
        gates = kernels.mlstm_gates(proj, 0, self.qk_width, self.query_scale, proj, i0, i0 + H, self.b_i, self.b_f,
                                    self.gate_cap, state, self._n_off, self._m_off, ctx, H, D)
        o = kernels.decay_linear_attention(proj, 0, self.qk_width, 2 * self.qk_width, None, None, 0, 1.0, False, state,
                                           ctx, H, D, V, q_scale=self.query_scale, gates=gates)
        g = kernels.group_rmsnorm_gate(o, proj, 2 * self.qk_width + self.v_width, self.norm_w, self.eps, H,
                                       kernels.GATE_SIGMOID, x.dtype)
        return kernels.linear(g, self.w_o)
