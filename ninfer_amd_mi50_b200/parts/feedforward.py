"""Feed-forward parts: a dense SwiGLU MLP, and routed SwiGLU experts with a gated
shared expert.

Dense (src/models/model.hip:334-336, gate and up fused to ``[2I, H]`` at load,
model.hip:586-605): ``ffn = Wdown (silu(Wgate x) * Wup x)``, ``silu(g) = g / (1 + exp(-g))``
(src/ops/kernels.hip:131-140).

Sparse (model.hip:338-433; routing in ``moe_route_cpu``, src/ops/moe.hip:49-106):
router logits in float32, softmax over all experts, the k largest probabilities
(ties to the lower index), weights ``p_e`` or, with ``norm_topk_prob``, ``p_e / sum(selected)``
(the reference always renormalises, moe.hip:77-82); every selected expert is a SwiGLU
MLP; ``moe = sum_i w_i y_i`` in selection order.  The shared expert and its sigmoid gate
(``ffn = moe + sigmoid(w_sg x) * shared(x)``) are Qwen2-MoE's and absent from the
reference.  Unlike the reference, routing never leaves the device.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import BiasedOutput, FeedForward, Fetch, RoutedSum, StepContext, TensorSpec


def gated_activation(spec):
    """A feed-forward's gated activation from its description: None or ("silu",) is silu(gate) * up;
    ("capped", limit, alpha) is g' * sigmoid(alpha g') * (u' + 1) with g' = min(gate, limit) and
    u' = clamp(up, -limit, limit); ("gelu_tanh",) is gelu_tanh(gate) * up with the tanh form of the GELU."""
    if spec is None or tuple(spec) == ("silu",):
        return None
    spec = tuple(spec)
    if spec == ("gelu_tanh",):
        return kernels.ACT_GELU_TANH
    if len(spec) == 3 and spec[0] == "capped":
        return kernels.capped_activation(float(spec[1]), float(spec[2]))
    raise ValueError(f"unknown gated activation {spec!r}")


_SIDE_STREAMS = {}


def _side_stream(device: torch.device, urgent: bool = False) -> "torch.cuda.Stream":
    """The second stream of a device; `urgent`: the one whose CTAs are placed before others'."""
    key = (str(device), urgent)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device, priority=-1 if urgent else 0)
    return _SIDE_STREAMS[key]


@register_part("feed_forward", "none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: the block then ends with its mixer (and has no second norm)."""
    graph_safe = True
    absent = True

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def forward(self, x: torch.Tensor, ctx: StepContext):
        raise RuntimeError("a layer without a feed-forward has nothing to run")


@register_part("feed_forward", "dense_swiglu")
class DenseSwiglu(FeedForward):
    graph_safe = True

    DEFAULT_NAMES = (("gate", "gate_proj.weight"), ("up", "up_proj.weight"), ("down", "down_proj.weight"),
                     ("gate_bias", "gate_proj.bias"), ("up_bias", "up_proj.bias"), ("down_bias", "down_proj.bias"))

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str, activation=None, bias: bool = False,
                 tensor_names=None):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.prefix = prefix
        self.activation, self.has_bias = gated_activation(activation), bool(bias)
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    def tensor_specs(self) -> List[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        specs = [TensorSpec(self._n("gate"), (I, H)), TensorSpec(self._n("up"), (I, H)),
                 TensorSpec(self._n("down"), (H, I))]
        if self.has_bias:
            specs += [TensorSpec(self._n("gate_bias"), (I,), role="vector"),
                      TensorSpec(self._n("up_bias"), (I,), role="vector"),
                      TensorSpec(self._n("down_bias"), (H,), role="vector")]
        return specs

    def load(self, fetch: Fetch) -> None:
        self.w_gate_up = torch.cat([fetch(self._n("gate")), fetch(self._n("up"))], dim=0).contiguous()
        self.w_down = fetch(self._n("down"))
        if self.has_bias:
            self.b_gate_up = torch.cat([fetch(self._n("gate_bias")), fetch(self._n("up_bias"))]).contiguous()
            self.b_down = fetch(self._n("down_bias"))

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x: torch.Tensor, ctx: StepContext):
        if not self.has_bias and (self.activation is None or self.activation == kernels.ACT_GELU_TANH):
            # an activation without constants of its own sits where silu does: in the first product's epilogue
            act = {} if self.activation is None else {"act": self.activation}
            return kernels.linear(kernels.linear_swiglu(x, self.w_gate_up, **act), self.w_down)
        # biases (or another activation): both products hand on their float32 sums, so that a bias
        # meets an unrounded value; the second bias is left to whoever reads the output next
        gu = kernels.linear(x, self.w_gate_up, out_dtype=torch.float32)
        act = kernels.gated_bias_act(gu, self.b_gate_up, self.activation, x.dtype)
        y = kernels.linear(act, self.w_down, out_dtype=torch.float32)
        return BiasedOutput(y, self.b_down) if self.has_bias else y


@register_part("feed_forward", "sparse_moe_swiglu")
class SparseMoeSwiglu(FeedForward):
    graph_safe = True

    # set to a list to collect each call's selected experts (measurement only)
    record_routing = None

    # tensor names below the prefix; `{e}` is the expert's number
    DEFAULT_NAMES = (("router", "gate.weight"), ("gate", "experts.{e}.gate_proj.weight"),
                     ("up", "experts.{e}.up_proj.weight"), ("down", "experts.{e}.down_proj.weight"),
                     ("shared_gate", "shared_expert.gate_proj.weight"), ("shared_up", "shared_expert.up_proj.weight"),
                     ("shared_down", "shared_expert.down_proj.weight"), ("shared_router", "shared_expert_gate.weight"),
                     ("correction", "correction"))

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, norm_topk_prob: bool,
                 moe_intermediate_size: int, shared_intermediate_size: int, prefix: str,
                 scoring: str = "softmax", weight_on: str = "output", tensor_names=None, activation=None,
                 correction: bool = False, groups=None, identity_experts: int = 0, route_scale: float = 1.0,
                 shared_gate: bool = True):
        """Further rules of choice (any of them makes the routing `ruled`; softmax scores, weights on the
        outputs and divided by their sum):
        `correction`: a float32 vector added to the scores for the choice only, not for the weights;
        `groups` (count, keep): the experts form `count` equal groups of neighbours, a group scores as its
        best choice score, and only experts of the `keep` best groups can be chosen;
        `identity_experts`: that many further experts after the `num_experts` with matrices, whose output is
        their input (the router has rows for them, and they count in the groups);
        `route_scale`: a factor on the weights;
        `shared_gate` false: the shared expert is added as it is, without a sigmoid gate of its own."""
        self.activation = gated_activation(activation)
        self.has_correction, self.identity_experts = bool(correction), int(identity_experts)
        self.groups = (int(groups[0]), int(groups[1])) if groups else None
        self.route_scale, self.shared_gate = float(route_scale), bool(shared_gate)
        self.ruled = (self.has_correction or self.groups is not None or self.identity_experts > 0
                      or self.route_scale != 1.0 or not self.shared_gate)
        if self.ruled and (scoring != "softmax" or weight_on != "output" or not norm_topk_prob):
            raise ValueError("routing with further rules of choice: softmax scores, weights on the outputs, divided by their sum")
        if self.ruled and self.shared_gate and shared_intermediate_size > 0:
            raise ValueError("routing with further rules of choice serves a shared expert without a gate only")
        total = int(num_experts) + self.identity_experts
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or total % count or not 1 <= keep <= count or (total // count) * keep < top_k:
                raise ValueError(f"{total} experts in {count} groups of which {keep} are kept cannot give {top_k} choices")
        self.correction = None
        if self.activation is not None and shared_intermediate_size > 0:
            raise ValueError("a shared expert is served with the silu-gated activation only")
        if not 1 <= top_k <= total:
            raise ValueError(f"top_k={top_k} must lie in [1, experts={total}]")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"scoring {scoring!r}: 'softmax' or 'sigmoid'")
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on {weight_on!r}: 'output' or 'input'")
        self.scoring, self.weight_on = scoring, weight_on
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        kernels.check_router_sizes(total, top_k)
        self.hidden_size, self.num_experts, self.top_k = int(hidden_size), int(num_experts), int(top_k)
        self.norm_topk_prob = bool(norm_topk_prob)
        self.moe_intermediate_size = int(moe_intermediate_size)
        self.shared_intermediate_size = int(shared_intermediate_size)
        self.prefix = prefix
        self.w_router = self.w13 = self.w2 = self.ws13 = self.ws2 = self.ws_packed = None
        self.w_router_split = None

    @property
    def has_shared(self) -> bool:
        return self.shared_intermediate_size > 0

    def _n(self, what: str, e: int = 0) -> str:
        return self.prefix + self.names[what].format(e=e)

    @property
    def plain_routed(self) -> bool:
        """The usual routed sum: softmax scores, weights on the experts' outputs, no further rules."""
        return self.scoring == "softmax" and self.weight_on == "output" and not self.ruled

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I, Is = self.prefix, self.hidden_size, self.moe_intermediate_size, self.shared_intermediate_size
        specs = [TensorSpec(self._n("router"), (self.num_experts + self.identity_experts, H), role="router")]
        if self.has_correction:
            specs.append(TensorSpec(self._n("correction"), (self.num_experts + self.identity_experts,), role="vector"))
        for e in range(self.num_experts):
            specs += [TensorSpec(self._n("gate", e), (I, H)),
                      TensorSpec(self._n("up", e), (I, H)),
                      TensorSpec(self._n("down", e), (H, I))]
        if self.has_shared:
            specs += [TensorSpec(self._n("shared_gate"), (Is, H)),
                      TensorSpec(self._n("shared_up"), (Is, H)),
                      TensorSpec(self._n("shared_down"), (H, Is))]
            if self.shared_gate:
                specs.append(TensorSpec(self._n("shared_router"), (1, H), role="router"))
        return specs

    def load(self, fetch: Fetch) -> None:
        p, H, I, E = self.prefix, self.hidden_size, self.moe_intermediate_size, self.num_experts
        router = fetch(self._n("router"))
        if self.has_correction:
            self.correction = fetch(self._n("correction")).contiguous()
        if self.has_shared and self.shared_gate:
            # one matrix yields the router logits and the shared expert's gate logit
            router = torch.cat([router, fetch(self._n("shared_router"))], dim=0)
        self.w_router = router.contiguous()
        self.w_router_split = kernels.split_router(self.w_router) if self.w_router.is_cuda else None
        first = fetch(self._n("gate", 0))
        self.w13 = torch.empty((E, 2 * I, H), dtype=first.dtype, device=first.device)
        self.w2 = torch.empty((E, H, I), dtype=first.dtype, device=first.device)
        for e in range(E):
            self.w13[e, :I].copy_(first if e == 0 else fetch(self._n("gate", e)))
            self.w13[e, I:].copy_(fetch(self._n("up", e)))
            self.w2[e].copy_(fetch(self._n("down", e)))
        del first
        if (self.w13.is_cuda and self.w13.dtype == torch.bfloat16 and kernels.can_pack(I, H)
                and kernels.can_pack(H, I)):
            # the bfloat16 kernels stream the experts from a tile layout; the row-major form goes
            self.w13 = kernels.pack_weights(self.w13, swiglu=True)
            self.w2 = kernels.pack_weights(self.w2, swiglu=False)
        if self.has_shared:
            self.ws13 = torch.cat([fetch(self._n("shared_gate")), fetch(self._n("shared_up"))],
                                  dim=0).contiguous()
            self.ws2 = fetch(self._n("shared_down"))
            # a second copy in the experts' tile layout, cut into chunks of the experts' width: decode
            # steps then serve the shared expert inside the experts' persistent launch (prompt steps
            # keep the row-major form for the library's products)
            self.ws_packed = None
            if (isinstance(self.w13, kernels.PackedWeights) and kernels.TUNING["moe_stream_shared"]
                    and self.ws13.dtype == torch.bfloat16 and self.plain_routed):
                self.ws_packed = kernels.pack_shared_expert(self.ws13, self.ws2.contiguous(), I)

    def weight_bytes(self) -> int:
        n = self.w_router.numel() * 4 + self._expert_total_bytes()
        if self.has_shared:
            n += (self.ws13.numel() + self.ws2.numel()) * self.ws2.element_size()
        return n

    def _expert_total_bytes(self) -> int:
        if isinstance(self.w13, kernels.PackedWeights):
            return self.w13.nbytes() + self.w2.nbytes()
        return (self.w13.numel() + self.w2.numel()) * self.w2.element_size()

    def expert_bytes(self) -> int:
        """Bytes of one routed expert's matrices."""
        return self._expert_total_bytes() // self.num_experts

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The same arithmetic in four arrangements, chosen by the number of rows (thresholds in
        `kernels.TUNING`, each with the measurement behind it):
        6 to 16 rows - routing, experts and shared expert in one persistent launch;
        up to 64 rows - the shared expert on a second stream beside the router and the experts
        (which are one persistent launch from 6 rows on);
        more rows - the routing on a second stream beside the shared expert's products.
        (Without a shared expert, or with the thresholds moved: one kernel after the other.)"""
        E, k = self.num_experts, self.top_k
        if self.ruled:
            return self._forward_ruled(x)
        if not self.plain_routed:
            return self._forward_scored(x)
        if (self.ws_packed is not None and x.is_cuda
                and kernels.can_route_and_run_experts(x, self.w_router, self.w13, self.w2, E, k, shared=self.ws_packed)):
            # a decode step: routing, the experts' products and the shared expert's are one persistent launch
            idx, wts, gate, plan, y, sum_wts, sum_plan = kernels.route_and_run_experts(
                x, self.w_router, E, k, self.norm_topk_prob, self.w13, self.w2, shared=self.ws_packed, act=self.activation)
            if SparseMoeSwiglu.record_routing is not None:
                SparseMoeSwiglu.record_routing.append(idx.clone())
            return RoutedSum(y, sum_plan, sum_wts, None, None, x.dtype)
        # The shared expert needs nothing from the router, so on small steps (where kernels are
        # too short to fill the device) it runs beside the routed path on a second stream;
        # inside a captured graph that becomes a parallel branch.
        fork = self.has_shared and x.is_cuda and x.shape[0] <= kernels.TUNING["shared_fork_max_rows"]
        shared = None

        def start_shared():
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                kernels.chain_break()       # its input comes from the other stream
                return main, side, kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)

        # The shared expert starts beside the router (whose kernels leave the memory idle) up to
        # `shared_fork_late_rows` rows, beyond that after it, beside the experts' products.
        late = x.shape[0] > kernels.TUNING["shared_fork_late_rows"]
        # In large steps it is the other way round: the shared expert's products fill the device,
        # and the routing - a chain of short kernels of a few CTAs - runs beside them.
        beside = kernels.TUNING["route_beside_shared_min_rows"]
        beside = self.has_shared and x.is_cuda and not fork and 0 < beside <= x.shape[0]
        # A decode step without a shared expert beside it: routing and both products of the experts
        # are one persistent launch.  (With a shared expert on the second stream the router's own
        # kernels are the better choice: they leave the memory idle, and the shared expert's first
        # product fills exactly that gap.  Measured at 8 tokens and A2.7B sizes: 3.45 ms a step with
        # the router's kernels, 3.61 ms with the routing inside the launch; without the second
        # stream 3.74 against 3.61.)
        fused = (x.is_cuda and not beside and not fork
                 and kernels.can_route_and_run_experts(x, self.w_router, self.w13, self.w2, E, k))
        if fork and not late:
            main, side, shared = start_shared()
        gathered = None
        y = None
        if beside:
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device, urgent=True)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                kernels.chain_break()
                idx, wts, gate, plan = kernels.route(x, self.w_router, E, k, self.norm_topk_prob,
                                                     split=self.w_router_split)
                if kernels.moe_uses_gathered_rows(x, self.w13):
                    gathered = kernels.moe_gather(x, plan, k)
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
            main.wait_stream(side)
            kernels.chain_break()
        elif fused:
            idx, wts, gate, plan, y = kernels.route_and_run_experts(x, self.w_router, E, k, self.norm_topk_prob,
                                                                    self.w13, self.w2, act=self.activation)
        else:
            idx, wts, gate, plan = kernels.route(x, self.w_router, E, k, self.norm_topk_prob,
                                                 split=self.w_router_split)
            if fork and late:
                main, side, shared = start_shared()
        if SparseMoeSwiglu.record_routing is not None:
            SparseMoeSwiglu.record_routing.append(idx.clone())
        if y is None:
            y = kernels.moe_experts(x, self.w13, self.w2, plan, k, gathered=gathered, act=self.activation)
        if fork:
            main.wait_stream(side)
            kernels.chain_break()           # the kernel that adds up also reads what the other stream produced
        elif self.has_shared and not beside:
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
        # not added up here: the next norm does it inside its own kernel (`RoutedSum`); whoever
        # cannot calls `materialize()`, which is `kernels.moe_combine`
        return RoutedSum(y, plan, wts, shared, gate, x.dtype)

    def _forward_ruled(self, x: torch.Tensor):
        """The routed sum under further rules of choice (`kernels.route_ruled`).  Identity experts are groups
        of the plan like the others, after the experts with matrices: both products run over the latter's
        rows, and the identity experts' rows of the result are filled with copies of their tokens' input, so
        the sum that is left pending needs to know nothing of them."""
        E, k = self.num_experts, self.top_k
        groups, keep = self.groups if self.groups is not None else (0, 0)
        idx, wts, plan, real_plan = kernels.route_ruled(x, self.w_router, E + self.identity_experts, k, self.correction,
                                                        groups, keep, self.route_scale, real_experts=E,
                                                        split=self.w_router_split)
        if SparseMoeSwiglu.record_routing is not None:
            SparseMoeSwiglu.record_routing.append(idx.clone())
        if self.identity_experts:
            y = kernels.moe_gemm2(kernels.moe_gemm1(x, self.w13, real_plan, k, act=self.activation), self.w2, real_plan,
                                  plan_is_older=True)
            kernels.identity_expert_rows(x, plan, k, E, y)
        else:
            y = kernels.moe_experts(x, self.w13, self.w2, plan, k, act=self.activation)
        shared = None
        if self.has_shared:
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
        return RoutedSum(y, plan, wts, shared, None, x.dtype)

    def _forward_scored(self, x: torch.Tensor):
        """The routed sum with sigmoid scores and/or the weight on the expert's input: routing
        (one launch on small steps), then the tokens are gathered into the experts' order - and,
        with the weight on the input, multiplied by their pair's weight in the same pass - and
        both products run over the sorted rows.  The sum that is left pending then carries unit
        weights."""
        E, k = self.num_experts, self.top_k
        idx, wts, gate, plan = kernels.route(x, self.w_router, E, k, self.norm_topk_prob,
                                             split=self.w_router_split, scoring=self.scoring)
        if SparseMoeSwiglu.record_routing is not None:
            SparseMoeSwiglu.record_routing.append(idx.clone())
        if self.weight_on == "input":
            y = kernels.moe_experts_sorted(kernels.scale_gather_rows(x, plan, k, wts), self.w13, self.w2, plan,
                                           act=self.activation)
            wts = None                          # the weights are spent: the sum adds the outputs as they are
        else:
            y = kernels.moe_experts(x, self.w13, self.w2, plan, k, act=self.activation)
        shared = None
        if self.has_shared:
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
        return RoutedSum(y, plan, wts, shared, gate, x.dtype)


@register_part("feed_forward", "dense_poly_norm")
class DensePolyNorm(FeedForward):
    """An ungated dense feed-forward ``W_down act(W_up x)`` whose activation is a polynomial of normed
    powers: ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with the powers taken element by element,
    ``N(v) = v / sqrt(mean(v^2) + eps)`` over a token's whole vector, and (a, b, c, e) one learned
    tensor of four numbers.  The first product hands on its float32 sums; the means and the
    polynomial are 32-bit in both modes."""

    graph_safe = True
    DEFAULT_NAMES = (("up", "up"), ("down", "down"), ("act", "act"))

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, prefix: str, tensor_names=None):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.eps, self.prefix = float(eps), prefix
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_up = self.w_down = self.coef = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    def tensor_specs(self) -> List[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec(self._n("up"), (I, H)), TensorSpec(self._n("down"), (H, I)),
                TensorSpec(self._n("act"), (4,), role="vector", init="norm")]

    def load(self, fetch: Fetch) -> None:
        self.w_up, self.w_down, self.coef = fetch(self._n("up")), fetch(self._n("down")), fetch(self._n("act"))

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x: torch.Tensor, ctx: StepContext):
        z = kernels.linear(x, self.w_up, out_dtype=torch.float32)
        return kernels.linear(kernels.poly_norm_act(z, self.coef, self.eps, x.dtype), self.w_down)


@register_part("feed_forward", "table_routed_gelu")
class TableRoutedGelu(FeedForward):
    """A mixture of ungated experts ``W_down gelu(W_up x)`` (the exact, erf GELU; no biases) without a
    router: a table ``[vocab, top]`` names each token id's experts, each weighing ``1 / top``.  An
    optional shared expert of the same form runs for every token and is added, multiplied by
    ``sigmoid(w_sg . x)``, one number a token.  The experts' rows are sorted by expert on the device
    (the plan the routed experts of the other designs use), both products run over the sorted rows,
    and the sum is left pending as a `RoutedSum`."""

    graph_safe = True
    DEFAULT_NAMES = (("table", "table"), ("up", "e{e}.up"), ("down", "e{e}.down"), ("shared_up", "shared.up"),
                     ("shared_down", "shared.down"), ("shared_gate", "shared.sg"))

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, vocab_size: int, moe_intermediate_size: int,
                 shared_intermediate_size: int, prefix: str, tensor_names=None):
        if not 1 <= top_k <= num_experts:
            raise ValueError(f"top_k={top_k} must lie in [1, num_experts={num_experts}]")
        kernels.check_router_sizes(num_experts, top_k)
        self.hidden_size, self.num_experts, self.top_k = int(hidden_size), int(num_experts), int(top_k)
        self.vocab_size = int(vocab_size)
        self.moe_intermediate_size, self.shared_intermediate_size = int(moe_intermediate_size), int(shared_intermediate_size)
        self.prefix = prefix
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.table = self.w_up = self.w_down = self.ws_up = self.ws_down = self.w_sg = None
        self._wts = {}

    @property
    def has_shared(self) -> bool:
        return self.shared_intermediate_size > 0

    def _n(self, what: str, e: int = 0) -> str:
        return self.prefix + self.names[what].format(e=e)

    def tensor_specs(self) -> List[TensorSpec]:
        H, I, Is = self.hidden_size, self.moe_intermediate_size, self.shared_intermediate_size
        specs = [TensorSpec(self._n("table"), (self.vocab_size, self.top_k), role="table",
                            init=f"distinct:{self.num_experts}")]
        for e in range(self.num_experts):
            specs += [TensorSpec(self._n("up", e), (I, H)), TensorSpec(self._n("down", e), (H, I))]
        if self.has_shared:
            specs += [TensorSpec(self._n("shared_up"), (Is, H)), TensorSpec(self._n("shared_down"), (H, Is)),
                      TensorSpec(self._n("shared_gate"), (1, H))]
        return specs

    def load(self, fetch: Fetch) -> None:
        H, I, E = self.hidden_size, self.moe_intermediate_size, self.num_experts
        self.table = fetch(self._n("table")).contiguous()
        lo, hi = int(self.table.min()), int(self.table.max())
        if lo < 0 or hi >= E:
            raise ValueError(f"{self._n('table')}: entries {lo}..{hi} name experts outside 0..{E - 1}")
        first = fetch(self._n("up", 0))
        self.w_up = torch.empty((E, I, H), dtype=first.dtype, device=first.device)
        self.w_down = torch.empty((E, H, I), dtype=first.dtype, device=first.device)
        for e in range(E):
            self.w_up[e].copy_(first if e == 0 else fetch(self._n("up", e)))
            self.w_down[e].copy_(fetch(self._n("down", e)))
        del first
        if (self.w_up.is_cuda and self.w_up.dtype == torch.bfloat16 and kernels.can_pack(I, H)
                and kernels.can_pack(H, I)):
            self.w_up = kernels.pack_weights(self.w_up, swiglu=False)
            self.w_down = kernels.pack_weights(self.w_down, swiglu=False)
        if self.has_shared:
            self.ws_up, self.ws_down = fetch(self._n("shared_up")), fetch(self._n("shared_down"))
            self.w_sg = fetch(self._n("shared_gate"))

    def _expert_total_bytes(self) -> int:
        if isinstance(self.w_up, kernels.PackedWeights):
            return self.w_up.nbytes() + self.w_down.nbytes()
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def expert_bytes(self) -> int:
        return self._expert_total_bytes() // self.num_experts

    def weight_bytes(self) -> int:
        n = self._expert_total_bytes() + self.table.numel() * 4
        if self.has_shared:
            n += (self.ws_up.numel() + self.ws_down.numel() + self.w_sg.numel()) * self.ws_down.element_size()
        return n

    def _weights(self, T: int, device) -> torch.Tensor:
        """float32 [T, top] of 1 / top, kept by row count (a step's graph may name it again)."""
        key = (T, str(device))
        if key not in self._wts:
            self._wts[key] = torch.full((T, self.top_k), 1.0 / self.top_k, dtype=torch.float32, device=device)
        return self._wts[key]

    def forward(self, x: torch.Tensor, ctx: StepContext):
        E, k = self.num_experts, self.top_k
        idx = kernels.table_route(self.table, ctx.token_ids, E)
        plan = kernels.moe_plan(idx, E)
        a = kernels.moe_rows_gemm(x, self.w_up, plan, k, from_tokens=True, gelu=True)
        y = kernels.moe_rows_gemm(a, self.w_down, plan, k, from_tokens=False)
        shared = gate = None
        if self.has_shared:
            shared = kernels.linear(kernels.gelu_erf_(kernels.linear(x, self.ws_up)), self.ws_down)
            gate = kernels.linear(x, self.w_sg, out_dtype=torch.float32)          # [T, 1] logits
        return RoutedSum(y, plan, self._weights(x.shape[0], x.device), shared, gate, x.dtype)
