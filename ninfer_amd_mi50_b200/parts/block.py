"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

Pre-norm, as the reference runs a layer (src/models/model.hip:206-444):
``x1 = norm1(h)`` -> mixer -> ``h += o`` fused with ``x2 = norm2(h)`` (model.hip:311) ->
feed-forward -> ``h += ffn``.  The last sum is left pending so that it fuses with the next
block's first norm, which is what the reference's ``fused_residual_rmsnorm`` does one
stage earlier.  A layer whose feed-forward is ``"none"`` is ``h += mixer(norm1(h))`` alone.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..registry import register_part
from .base import Block, CacheView, FeedForward, Fetch, Mixer, Norm, RoutedSum, StepContext, TensorSpec, summed


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        if getattr(self.feed_forward, "absent", False):
            return (self.norm1, self.mixer)             # no feed-forward: no second norm either
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def load(self, fetch: Fetch) -> None:
        for p in self.parts():
            p.load(fetch)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts())

    def check_limits(self, dtype, max_context, page_size) -> None:
        for p in self.parts():
            p.check_limits(dtype, max_context, page_size)

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[CacheView], state: Optional[torch.Tensor]
                ) -> Optional[torch.Tensor]:
        if not self.norm1.takes_unsummed or not isinstance(pending, (torch.Tensor, RoutedSum, type(None))):
            pending = summed(pending)
        x1 = self.norm1.add_norm(h, pending, ctx.dtype)
        a = self.mixer.forward(x1, ctx, cache, state)
        if getattr(self.feed_forward, "absent", False):
            return a                                    # the mixer's output is what is left pending
        x2 = self.norm2.add_norm(h, a, ctx.dtype)
        return self.feed_forward.forward(x2, ctx)


@register_part("block", "sublayer_norm_scaled")
class SublayerNormScaledBlock(Block):
    """The norm sits on each sublayer's output, and a learned vector scales it per channel:

        h += scale1 * norm1(mixer(h));   h += scale2 * norm2(feed_forward(h))

    The sublayers read the stream itself.  In bfloat16 mode they read its rounding, which the
    kernel that adds a sublayer's output writes beside the float32 stream (`StreamCopy`), so the
    stream is not read again for it.  Nothing is left pending: each sum happens at once, in the
    same kernel as the norm and the scale.  A layer whose feed-forward is ``"none"`` has the first
    line only.
    """

    wants_spec = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward, spec=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        names = dict(spec.names) if spec is not None else {}
        prefix = spec.prefix if spec is not None else ""
        self.width = norm1.size
        self.scale_names = (prefix + names.get("scale1", "scale1"), prefix + names.get("scale2", "scale2"))
        self.scale1 = self.scale2 = None

    @property
    def has_ff(self) -> bool:
        return not getattr(self.feed_forward, "absent", False)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward) if self.has_ff else (self.norm1, self.mixer)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for p in self.parts() for s in p.tensor_specs()]
        for name in self.scale_names[:2 if self.has_ff else 1]:
            specs.append(TensorSpec(name, (self.width,), role="vector", init="norm"))
        return specs

    def load(self, fetch: Fetch) -> None:
        for p in self.parts():
            p.load(fetch)
        self.scale1 = fetch(self.scale_names[0])
        self.scale2 = fetch(self.scale_names[1]) if self.has_ff else None

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts()) + 4 * self.width * (2 if self.has_ff else 1)

    def check_limits(self, dtype, max_context, page_size) -> None:
        for p in self.parts():
            p.check_limits(dtype, max_context, page_size)

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]):
        from .. import kernels
        from .base import BiasedOutput, StreamCopy
        copy_dtype = None if ctx.dtype == torch.float32 else ctx.dtype       # 32-bit mode reads the stream itself
        if isinstance(pending, StreamCopy):
            x = pending.x
        else:
            delta = summed(pending)                  # another arrangement ran before: add what it left
            if delta is not None:
                h.add_(delta.to(torch.float32))
            x = None
        if x is None:
            x = h if copy_dtype is None else kernels.cast_rows(h, copy_dtype)
        a = self.mixer.forward(x, ctx, cache, state)
        x = self.norm1.add_scaled_norm(h, a, self.scale1, copy_dtype)
        if self.has_ff:
            f = self.feed_forward.forward(h if copy_dtype is None else x, ctx)
            bias = None
            if isinstance(f, BiasedOutput):          # the norm's kernel adds the bias in its own pass
                f, bias = f.y, f.bias
            x = self.norm2.add_scaled_norm(h, f, self.scale2, copy_dtype, bias=bias)
        return StreamCopy(x)


@register_part("block", "hyper_connections")
class HyperConnectionBlock(Block):
    """Pre-norm sublayers over several residual streams a token.  For sublayer q (1: mixer, 2:
    feed-forward) with its constants in_q [S], out_q [S], mix_q [S, S] (indexed [from, to]):

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] * y

    all streams at once from the old ones.  The stream tensor is ``[T, S * width]``; the update of
    one sublayer, the read for the next and its norm are one kernel, so the last update of a block is
    left pending (`StreamUpdate`) for whoever reads the streams next.  With `learned` false there are
    no tensors and in = out = 1, mix = identity: for S = 1 that is the ordinary pre-norm residual
    block.  The norms are asked for their weight, groups and eps; the kernel does the arithmetic.
    """

    wants_spec = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward, spec=None,
                 streams: int = 1, learned: bool = True, tensor_names=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.streams, self.learned = int(streams), bool(learned)
        if self.streams < 1:
            raise ValueError("a token has at least one residual stream")
        if not self.learned and self.streams != 1:
            raise ValueError("several residual streams need their constants")
        for n in (norm1, norm2):
            if not all(hasattr(n, a) for a in ("weight", "eps", "size")):
                raise TypeError("the arrangement over several streams takes norms that are an RMS norm with a weight")
        names = dict(spec.names) if spec is not None else {}
        prefix = spec.prefix if spec is not None else ""
        own = dict((("in", "in"), ("out", "out"), ("mix", "mix")))
        own.update(dict(tensor_names or ()))
        self._names = [{k: prefix + names.get(f"connect{q}", f"hc{q}") + "." + v for k, v in own.items()} for q in (1, 2)]
        self.consts = [None, None]               # per sublayer: (in, out, mix) float32 on the device

    @property
    def has_ff(self) -> bool:
        return not getattr(self.feed_forward, "absent", False)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward) if self.has_ff else (self.norm1, self.mixer)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for p in self.parts() for s in p.tensor_specs()]
        if self.learned:
            S = self.streams
            for n in self._names[:2 if self.has_ff else 1]:
                specs += [TensorSpec(n["in"], (S,), role="vector", init="norm"),
                          TensorSpec(n["out"], (S,), role="vector", init="norm"),
                          TensorSpec(n["mix"], (S, S), role="vector")]
        return specs

    def load(self, fetch: Fetch) -> None:
        for p in self.parts():
            p.load(fetch)
        if self.learned:
            for q, n in enumerate(self._names[:2 if self.has_ff else 1]):
                self.consts[q] = (fetch(n["in"]).contiguous(), fetch(n["out"]).contiguous(), fetch(n["mix"]).contiguous())

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts())

    def check_limits(self, dtype, max_context, page_size) -> None:
        for p in self.parts():
            p.check_limits(dtype, max_context, page_size)

    def _const(self, q: int):
        return self.consts[q] if self.learned else (None, None, None)

    @staticmethod
    def _groups(norm) -> int:
        return int(getattr(norm, "groups", 1))

    def _pending(self, h, pending):
        """(y, mix, out) of what the block before left: its own kind, or an ordinary sum."""
        from .base import StreamUpdate
        if isinstance(pending, StreamUpdate):
            return pending.y, pending.mix, pending.out
        y = summed(pending)
        if y is not None and self.streams != 1:
            raise TypeError("an ordinary residual sum cannot be added to several streams")
        return y, None, None

    def settle(self, h: torch.Tensor, pending):
        from .. import kernels
        y, mix, out = self._pending(h, pending)
        if y is not None:
            kernels.streams_mix_norm(h, self.streams, y, mix, out, None, None, 0.0, 1, None)
        return None

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]):
        from .. import kernels
        from .base import StreamUpdate
        S = self.streams
        y, mix, out = self._pending(h, pending)
        in1, out1, mix1 = self._const(0)
        x1 = kernels.streams_mix_norm(h, S, y, mix, out, in1, self.norm1.weight, self.norm1.eps,
                                      self._groups(self.norm1), ctx.dtype)
        a = self.mixer.forward(x1, ctx, cache, state)
        if not self.has_ff:
            return StreamUpdate(a, mix1, out1)
        in2, out2, mix2 = self._const(1)
        x2 = kernels.streams_mix_norm(h, S, a, mix1, out1, in2, self.norm2.weight, self.norm2.eps,
                                      self._groups(self.norm2), ctx.dtype)
        return StreamUpdate(summed(self.feed_forward.forward(x2, ctx)), mix2, out2)
