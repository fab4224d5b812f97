"""The generic decoder: embedding, a list of blocks run in a given order, final norm,
output head.

Reference counterpart: ``Impl::forward_batch`` (src/models/model.hip:994-1032) with
``begin_rows`` (embedding gather, 697-724), the per-layer loop (1021-1025) and
``finalize`` (727-755: final RMSNorm and LM head only on the rows whose logits are
wanted; the head is the embedding matrix when ``tie_word_embeddings``, 497-499).
Which blocks exist and in which order they run is data (`ModelPlan`), not code.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .. import kernels
from ..config.model_config import LayerCall, ModelPlan
from ..registry import build_part, part_class
from .base import CacheSpec, CacheView, Fetch, RoutedSum, StateSpec, StepContext, StreamUpdate, TensorSpec, summed


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.vocab_size, self.hidden_size = plan.vocab_size, plan.hidden_size
        self.blocks = []
        for spec in plan.layers:
            norm1 = build_part("norm", spec.norm, prefix=spec.name_of("norm1"))
            mixer = build_part("mixer", spec.mixer, prefix=spec.name_of("mixer"))
            norm2 = build_part("norm", spec.norm, prefix=spec.name_of("norm2"))
            ffn = build_part("feed_forward", spec.feed_forward, prefix=spec.name_of("feed_forward"))
            block_cls = part_class("block", spec.arrangement)
            # an arrangement with tensors of its own (a layer scale, say) is told the layer's names
            extra = {"spec": spec} if getattr(block_cls, "wants_spec", False) else {}
            extra.update(dict(spec.arrangement_params))
            self.blocks.append(block_cls(norm1, mixer, norm2, ffn, **extra))
        self.embedding_extras = [build_part("embedding", e) for e in plan.embedding_extras]
        self.final_norm = build_part("norm", plan.final_norm, prefix=plan.final_norm_name)
        self.streams = int(plan.streams)
        if not 1 <= self.streams <= kernels.MAX_STREAMS:
            raise ValueError(f"{self.streams} residual streams a token; the kernels take 1 to {kernels.MAX_STREAMS}")
        if self.streams > 1 and plan.embedding_extras:
            raise ValueError("rows added to the embedding and several residual streams do not go together")
        self.order: List[LayerCall] = list(plan.order)
        vectors = dict(plan.stream_vectors)
        for call in self.order:
            if not (0 <= call.layer < len(self.blocks) and call.cache >= 0):
                raise ValueError(f"execution order names a layer that does not exist: {call}")
            if call.add_vector is not None and not (
                    call.add_vector[0] in vectors and 0 <= call.add_vector[1] < vectors[call.add_vector[0]]):
                raise ValueError(f"execution order adds a vector the plan does not have: {call}")
        # cache and state slots: usually one per layer (slot i is layer i's); an order that gives a
        # layer a slot of its own per call names more
        self.num_cache_slots = max([len(self.blocks)] + [c.cache + 1 for c in self.order])
        self.num_state_slots = max([len(self.blocks)] + [c.state_slot() + 1 for c in self.order])
        # what the embedding's extras keep per request lives in state slots after the layers'
        self.extra_state_slot0 = self.num_state_slots
        # called with (index of the layer run, stream) after every run when set: for inspection only,
        # and only meaningful for arrangements that leave nothing pending
        self.probe: Optional[Callable[[int, torch.Tensor], None]] = None
        self.vectors: Dict[str, torch.Tensor] = {}
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ---- what the model needs ---------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        V, H = self.vocab_size, self.hidden_size
        specs = [TensorSpec(self.plan.embedding_name, (V, H))]
        for b in self.blocks:
            specs += b.tensor_specs()
        for e in self.embedding_extras:
            specs += e.tensor_specs()
        specs += self.final_norm.tensor_specs()
        for name, rows in self.plan.stream_vectors:
            specs.append(TensorSpec(name, (rows, H), role="vector"))
        if not self.plan.tie_word_embeddings:
            specs.append(TensorSpec(self.plan.head_name, (V, H)))
        return specs

    def load(self, fetch: Fetch) -> None:
        self.embedding = fetch(self.plan.embedding_name)
        for b in self.blocks:
            b.load(fetch)
        for e in self.embedding_extras:
            e.load(fetch)
        self.final_norm.load(fetch)
        self.vectors = {name: fetch(name) for name, _ in self.plan.stream_vectors}
        self.head = self.embedding if self.plan.tie_word_embeddings else fetch(self.plan.head_name)

    def _slot_specs(self, count: int, slot_of, spec_of, what: str) -> list:
        specs: list = [None] * count
        named = set()
        for call in self.order:
            slot, spec = slot_of(call), spec_of(self.blocks[call.layer])
            if slot in named and specs[slot] != spec:
                raise ValueError(f"{what} slot {slot} is shared by layers that keep different things")
            named.add(slot)
            specs[slot] = spec
        called = {call.layer for call in self.order}
        for i, b in enumerate(self.blocks):          # a layer the order never runs keeps its own slot;
            if i not in named and i not in called:   # one that only ever reads another's slot keeps none
                specs[i] = spec_of(b)
        return specs

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        """What each cache slot keeps in pages (None: nothing).  Slot i belongs to layer i unless
        the order says otherwise."""
        return self._slot_specs(self.num_cache_slots, lambda c: c.cache, lambda b: b.cache_spec(), "cache")

    def state_specs(self) -> List[Optional[StateSpec]]:
        specs = self._slot_specs(self.num_state_slots, lambda c: c.state_slot(), lambda b: b.state_spec(), "state")
        return specs + [e.state_spec() for e in self.embedding_extras]

    @property
    def graph_safe(self) -> bool:
        return (all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
                and all(e.graph_safe for e in self.embedding_extras))

    def check_limits(self, dtype: torch.dtype, max_context: int, page_size: int) -> None:
        for b in self.blocks:
            b.check_limits(dtype, max_context, page_size)
        self.final_norm.check_limits(dtype, max_context, page_size)

    def weight_bytes(self) -> int:
        n = sum(b.weight_bytes() for b in self.blocks) + self.final_norm.weight_bytes()
        n += sum(e.weight_bytes() for e in self.embedding_extras)
        n += sum(v.numel() * 4 for v in self.vectors.values())
        return n + self.head.numel() * self.head.element_size()

    # ---- one pass over the step's rows --------------------------------------------------
    def forward(self, ctx: StepContext,
                cache_view: Callable[[int, bool], Optional[CacheView]],
                state_of: Callable[[int], Optional[torch.Tensor]]) -> torch.Tensor:
        """Run every row of the step; return float32 logits [R, vocab] for ctx.logit_rows."""
        h = torch.empty((ctx.T, self.hidden_size * self.streams), dtype=torch.float32, device=ctx.device)
        if self.streams == 1:
            kernels.embed_rows(self.embedding, ctx.token_ids, h)
        else:
            kernels.embed_copies(self.embedding, ctx.token_ids, h, self.streams)
        for i, e in enumerate(self.embedding_extras):
            e.add(h, ctx, state_of(self.extra_state_slot0 + i))
        pending = None
        for run, call in enumerate(self.order):
            if call.add_vector is not None:
                # (the pending contribution has not been added yet; the sums commute)
                kernels.add_row_vector(h, self.vectors[call.add_vector[0]][call.add_vector[1]])
            pending = self.blocks[call.layer].forward(
                h, pending, ctx, cache_view(call.cache, call.append), state_of(call.state_slot()))
            if self.probe is not None:
                pending = self.blocks[call.layer].settle(h, pending)
                self.probe(run, h)
        R = ctx.logit_rows.numel()
        if R == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=ctx.device)
        if isinstance(pending, StreamUpdate) and getattr(self.final_norm, "takes_stream_update", False):
            pass                                     # the norm applies the update in its own pass over the rows
        elif not self.final_norm.takes_unsummed or not isinstance(pending, (torch.Tensor, RoutedSum, type(None))):
            pending = summed(pending)
        x = self.final_norm.add_norm_rows(h, pending, ctx.logit_rows, ctx.dtype)
        logits = kernels.linear(x, self.head, out_dtype=torch.float32)
        if self.plan.logit_scale != 1.0:
            logits.mul_(self.plan.logit_scale)
        if self.plan.logit_softcap > 0.0:
            kernels.softcap(logits, self.plan.logit_softcap)
        return logits
