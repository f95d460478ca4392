"""Rotary position encoding, rotate-half ("neox") pairing.

Reference: models/rotary.py:36-45 (inv_freq[j] = theta^(-2j/D), angle = position * inv_freq[j])
and models/rotary.py:13-22 (y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin on the two halves).
The angle, sine and cosine are float32 on the device.  There is no table over all positions
(``max_positions`` only bounds what a request may reach): the sines and cosines of the positions
of one step are computed once per step and read by every layer.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from ..registry import register_part
from .base import PositionEncoding, Runtime


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    graph_capturable = True

    def __init__(self, name: str, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None):
        super().__init__(name)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        # the same float32 expression as the reference, evaluated once on the host
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(rt.device)

        self._table = rt.shared(f"rotary.table.{self.theta!r}.{self.rotary_dim}", rt.max_tokens, self.rotary_dim,
                                dtype=torch.float32)

    def fused_rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx) -> Optional[torch.Tensor]:
        def make():
            table = self._table[:ctx.positions.numel()]
            ops.rope_table(self.inv_freq, ctx.positions, table)
            return table
        return ctx.shared_in_step(("rotary_neox", self.theta, self.rotary_dim), make)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        ops.rope(x, self.inv_freq, self.rotary_dim, positions, out, self.rt.status)
        return out


@register_part("position", "rotary_stretched")
class RotaryStretched(PositionEncoding):
    """Rotate-half rotation whose frequencies may be stretched for contexts longer than the ``original`` one (the
    scheme of Peng et al., "YaRN: Efficient Context Window Extension of Large Language Models"): with
    f_i = base^(-2i / dims),

        pair(t) = dims * ln(original / (2 pi t)) / (2 ln base)          the pair that turns t times in `original`
        lo = max(floor(pair(fast)), 0);  hi = min(ceil(pair(slow)), dims - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        freq_i = f_i / factor * ramp_i + f_i * (1 - ramp_i)

    and sines and cosines multiplied by ``magnitude[0] * ln(factor) + magnitude[1]``.  Without ``scaling`` the plain
    frequencies and magnitude 1.  The frequencies are evaluated in float64 on the host and kept in float32; angles
    are float32(position) * freq on the device.  The kernels that take ``frequencies()`` rotate the first ``dims``
    values of a vector and let the rest pass."""

    graph_capturable = True

    def __init__(self, name: str, dims: int, base: float, scaling: Optional[dict] = None):
        super().__init__(name)
        self.dims, self.base = int(dims), float(base)
        if self.dims % 2 or self.dims < 0:
            raise ValueError(f"rotation {name}: dims {self.dims} must be even")
        half = self.dims // 2
        freq = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        self.magnitude = 1.0
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])

            def pair(turns: float) -> float:
                return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(pair(float(scaling["fast"]))), 0)
            hi = min(math.ceil(pair(float(scaling["slow"]))), self.dims - 1)
            for i in range(half):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
            m0, m1 = scaling.get("magnitude", (0.1, 1.0))
            self.magnitude = float(m0) * math.log(factor) + float(m1)
        self._freq = freq

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.freq = torch.tensor(self._freq, dtype=torch.float64).to(torch.float32).to(rt.device)

    def frequencies(self) -> Tuple[torch.Tensor, float, int]:
        """(float32 frequencies [dims / 2] on the device, magnitude, dims)."""
        return self.freq, self.magnitude, self.dims
