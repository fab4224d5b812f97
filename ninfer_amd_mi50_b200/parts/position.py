"""Rotary position embedding, half-split pairing.

For ``i < D/2``: ``angle = float(pos) * inv_freq[i]``, ``inv_freq[i] = theta^(-2i/D)``
evaluated in single precision on the host (src/models/model.hip:636-639);
``x'[i] = x[i] cos - x[i + D/2] sin``, ``x'[i + D/2] = x[i] sin + x[i + D/2] cos``
(src/ops/kernels.hip:73-94).  Applied to every query and key head, never to values.
The rotation itself runs inside the fused rotate-and-append kernel; this part owns the
table and the parameters.
"""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..registry import register_part
from .base import PositionEncoding


def rotary_inverse_frequencies(head_dim: int, theta: float, rotary_dim: Optional[int] = None
                               ) -> torch.Tensor:
    """float32 [rotary_dim / 2]: powf(theta, -2 i / D) with float operands."""
    rot = head_dim if rotary_dim is None else rotary_dim
    i = np.arange(rot // 2, dtype=np.float32)
    expo = (np.float32(-2.0) * i / np.float32(rot)).astype(np.float32)
    inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    return torch.from_numpy(inv)


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and in (0, {head_dim}]")
        self._table = {}

    def rotary_table(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int]]:
        key = str(device)
        if key not in self._table:
            self._table[key] = rotary_inverse_frequencies(
                self.head_dim, self.theta, self.rotary_dim).to(device)
        return self._table[key], self.rotary_dim


def blended_inverse_frequencies(rotary_dim: int, theta: float, factor: float, original: float, fast: float,
                                slow: float) -> torch.Tensor:
    """float32 [rotary_dim / 2]: the plain frequencies f_i = theta^(-2i / rot) blended with the stretched
    ones f_i / factor by a ramp over the pair index.  With dim(t) = rot ln(original / (2 pi t)) / (2 ln theta)
    - the index whose wave turns t times over `original` positions - lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), rot - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``.  Evaluated in double precision, rounded once."""
    import math
    rot = int(rotary_dim)
    i = np.arange(rot // 2, dtype=np.float64)
    f = np.power(float(theta), -2.0 * i / rot)

    def dim_of(turns: float) -> float:
        return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), rot - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return torch.from_numpy((f / factor * ramp + f * (1.0 - ramp)).astype(np.float32))


@register_part("position", "rotary_half_split_blended")
class RotaryHalfSplitBlended(RotaryHalfSplit):
    """The half-split rotation with frequencies stretched for contexts longer than the `original` one
    (the YaRN scheme): fast waves keep their frequency, slow ones are divided by `factor`, those between
    are blended (`blended_inverse_frequencies`), and cosine and sine are both multiplied by
    ``0.1 ln(factor) + 1`` (`magnitude`)."""

    def __init__(self, head_dim: int, theta: float, factor: float, original: float, fast: float, slow: float,
                 rotary_dim: Optional[int] = None):
        super().__init__(head_dim, theta, rotary_dim)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        if not (self.factor >= 1.0 and self.original > 0 and self.fast > 0 and self.slow > 0 and self.theta > 1.0):
            raise ValueError("stretched rotation: factor >= 1, original, fast and slow positive, base above 1")
        import math
        self.magnitude = 0.1 * math.log(self.factor) + 1.0

    def rotary_table(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int]]:
        key = str(device)
        if key not in self._table:
            self._table[key] = blended_inverse_frequencies(self.rotary_dim, self.theta, self.factor, self.original,
                                                           self.fast, self.slow).to(device)
        return self._table[key], self.rotary_dim


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position information enters queries or keys."""

    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def apply(self, q, k, positions) -> None:
        return None
