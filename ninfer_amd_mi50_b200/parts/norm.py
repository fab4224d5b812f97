"""RMS normalisation, fused with the residual sum.

``inv = rsqrt(mean(x^2) + eps); y = x * inv * w`` with the weight multiplying directly
(src/ops/kernels.hip:17-41); the sum ``h += r`` happens in the same pass
(``fused_residual_rmsnorm_kernel``, src/ops/kernels.hip:100-129).  Here the residual
stream stays in float32 between layers, so the sum, the mean of squares and the product
are all 32-bit in both modes.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import Fetch, Norm, RoutedSum, TensorSpec, summed


@register_part("norm", "rms_norm")
class RmsNorm(Norm):
    graph_safe = True
    takes_unsummed = True

    def __init__(self, size: int, eps: float, prefix: str, weight_name: str = "weight", one_plus: bool = False):
        """`one_plus`: the stored weight lies around zero and 1 + w multiplies.  `weight_name` "":
        the checkpoint names the weight by the norm's own name, without a suffix."""
        self.size, self.eps, self.prefix = int(size), float(eps), prefix
        self.weight_name, self.one_plus = weight_name, bool(one_plus)
        self.weight: Optional[torch.Tensor] = None

    def _name(self) -> str:
        return self.prefix + self.weight_name if self.weight_name else self.prefix.rstrip(".")

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self._name(), (self.size,), role="vector", init="linear" if self.one_plus else "norm")]

    def load(self, fetch: Fetch) -> None:
        self.weight = fetch(self._name())
        if self.one_plus:
            # held as 1 + w: the float32 sum is the one a kernel would form from w anyway
            self.weight = (self.weight + 1.0).contiguous()

    def add_scaled_norm(self, h, delta, scale, out_dtype, bias=None):
        """h += scale * norm(delta + bias) (in place, 32-bit): the norm sits on a sublayer's output,
        not on its input.  Returns the updated stream in `out_dtype` (None: nothing)."""
        if isinstance(delta, RoutedSum):
            if delta.shared is None and bias is None and delta.plan.top_k <= kernels.FUSED_COMBINE_MAX_K:
                # the experts' weighted sum is added up inside the norm's kernel
                return kernels.routed_scaled_norm_add(h, delta.y, delta.plan.inv, delta.wts, delta.plan.top_k,
                                                      self.weight, scale, self.eps, out_dtype)
            delta = summed(delta)
        return kernels.scaled_norm_add(h, delta, bias, self.weight, scale, self.eps, out_dtype)

    def weight_bytes(self) -> int:
        return self.size * 4

    def _fusable(self, delta, out_dtype, rows: int) -> bool:
        return (isinstance(delta, RoutedSum) and out_dtype == torch.bfloat16 and delta.wts is not None
                and kernels.can_fuse_combine_norm(delta.y, self.size, rows, delta.wts.shape[1]))

    def add_norm(self, h, delta, out_dtype):
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
        if self._fusable(delta, out_dtype, h.shape[0]):
            # the experts' weighted sum, the residual add and the norm in one kernel
            kernels.moe_combine_add_rmsnorm(delta.y, delta.plan, delta.wts, delta.shared, delta.gate, h, None,
                                            self.weight, self.eps, out)
        else:
            kernels.add_rmsnorm(h, summed(delta), self.weight, self.eps, out)
        return out

    def add_norm_rows(self, h, delta, rows, out_dtype):
        out = torch.empty((rows.numel(), h.shape[1]), dtype=out_dtype, device=h.device)
        if self._fusable(delta, out_dtype, rows.numel()):
            kernels.moe_combine_add_rmsnorm(delta.y, delta.plan, delta.wts, delta.shared, delta.gate, h, rows,
                                            self.weight, self.eps, out)
        else:
            kernels.add_rmsnorm_rows(h, summed(delta), rows, self.weight, self.eps, out)
        return out


@register_part("norm", "layer_norm")
class LayerNorm(Norm):
    """Layer norm with a weight and no bias, fused with the residual sum:
    ``y = (x - mean(x)) / sqrt(var(x) + eps) * w`` with ``var`` the mean of the squared
    deviations from the mean.  Sum, mean, variance and product are 32-bit in both modes."""

    graph_safe = True
    takes_unsummed = True

    def __init__(self, size: int, eps: float, prefix: str, weight_name: str = "weight"):
        self.size, self.eps, self.prefix, self.weight_name = int(size), float(eps), prefix, weight_name
        self.weight: Optional[torch.Tensor] = None

    def _name(self) -> str:
        # a checkpoint may name the weight by the norm's own name ("<layer>.norm1"), without a suffix
        return self.prefix + self.weight_name if self.weight_name else self.prefix.rstrip(".")

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self._name(), (self.size,), role="vector", init="norm")]

    def load(self, fetch: Fetch) -> None:
        self.weight = fetch(self._name())

    def weight_bytes(self) -> int:
        return self.size * 4

    @staticmethod
    def _routed(delta, out_dtype):
        """The routed experts' pending sum in the form the kernel adds up itself, or None."""
        if (isinstance(delta, RoutedSum) and delta.shared is None and delta.y.dtype == out_dtype
                and delta.plan.top_k <= kernels.FUSED_COMBINE_MAX_K):
            return (delta.y, delta.plan.inv, delta.wts, delta.plan.top_k)
        return None

    def add_norm(self, h, delta, out_dtype):
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
        routed = self._routed(delta, out_dtype)
        kernels.add_layernorm(h, None if routed else summed(delta), None, self.weight, self.eps, out, routed=routed)
        return out

    def add_norm_rows(self, h, delta, rows, out_dtype):
        out = torch.empty((rows.numel(), h.shape[1]), dtype=out_dtype, device=h.device)
        routed = self._routed(delta, out_dtype)
        kernels.add_layernorm(h, None if routed else summed(delta), rows, self.weight, self.eps, out, routed=routed)
        return out


@register_part("norm", "group_rms_norm")
class GroupRmsNorm(Norm):
    """RMS norm in groups: the row is cut into `groups` equal consecutive parts, each divided by its
    own ``sqrt(mean(part^2) + eps)``, and the whole multiplied by the weight.  One group is the usual
    RMS norm.  Fused with the residual sum; the stream may hold several copies a token (`h` is then
    ``[T, streams * size]``), in which case the norm reads their plain sum and a pending
    `StreamUpdate` is applied in the same pass.  Sum, means and products are 32-bit in both modes."""

    graph_safe = True
    takes_unsummed = False
    takes_stream_update = True

    def __init__(self, size: int, eps: float, prefix: str, groups: int = 1, weight_name: str = "weight"):
        self.size, self.eps, self.prefix = int(size), float(eps), prefix
        self.groups, self.weight_name = int(groups), weight_name
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"a row of {self.size} does not split into {self.groups} equal groups")
        self.weight: Optional[torch.Tensor] = None

    def _name(self) -> str:
        return self.prefix + self.weight_name if self.weight_name else self.prefix.rstrip(".")

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self._name(), (self.size,), role="vector", init="norm")]

    def load(self, fetch: Fetch) -> None:
        self.weight = fetch(self._name())

    def weight_bytes(self) -> int:
        return self.size * 4

    def _apply(self, h, delta, rows, out_dtype):
        from .base import StreamUpdate
        S = h.shape[1] // self.size
        if isinstance(delta, StreamUpdate):
            y, mix, out = delta.y, delta.mix, delta.out
        else:
            y, mix, out = summed(delta), None, None
        return kernels.streams_mix_norm(h, S, y, mix, out, None, self.weight, self.eps, self.groups, out_dtype,
                                        rows=rows)

    def add_norm(self, h, delta, out_dtype):
        return self._apply(h, delta, None, out_dtype)

    def add_norm_rows(self, h, delta, rows, out_dtype):
        return self._apply(h, delta, rows, out_dtype)
