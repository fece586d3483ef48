"""Position encodings.

``rope_half_split`` rotates pairs ``(i, i + rotary_dim/2)`` of a head by the angle
``pos * theta^(-2i / rotary_dim)`` (kernels/cuda/dense/dense_common.cuh:166-180).
The inverse frequencies are computed once in float64 and rounded to float32; the
angle ``pos * inv_freq`` and its sine and cosine are evaluated in float32 inside
the fused norm + rotate + store kernel (the reference calls ``powf`` per element
on the device; the ladder is the same).

``rope_stretched`` is the same rotation with the ladder stretched for contexts longer than the
``original`` one: pair ``i`` of ``n = rotary_dim / 2`` keeps its frequency ``f_i`` where it
turns often, gets ``f_i / factor`` where it turns rarely, and a blend between.  With
``d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)`` - the (fractional) pair that
turns ``t`` times within ``original`` positions - ``lo = max(floor(d(fast)), 0)``,
``hi = min(ceil(d(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``,
the frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``.  Cosine and sine are both
multiplied by ``magnitude = 0.1 * ln(factor) + 1``; kernels that rotate read it from
``PositionEncoding.magnitude``.

Both take ``interleaved`` (default false): pair ``i`` is then the neighbours ``(2i, 2i + 1)``
instead of ``(i, i + rotary_dim/2)``, on the same ladder.
"""

from __future__ import annotations

import math

import torch

from ..config.errors import UnsupportedShape
from .base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope_half_split")
class RopeHalfSplit(PositionEncoding):
    def __init__(self, spec, env, head_dim: int):
        super().__init__(spec, env)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params.get("rotary_dim") or head_dim)
        self.interleaved = bool(spec.params.get("interleaved", False))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise UnsupportedShape("rotary_dim", self.rotary_dim, f"must be even and at most the head size {head_dim}")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * i / self.rotary_dim)).to(torch.float32).to(env.device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim


@POSITION_ENCODINGS.register("rope_stretched")
class RopeStretched(RopeHalfSplit):
    """``params``: ``theta``, ``rotary_dim``, ``factor``, ``original``, ``fast``, ``slow``."""

    def __init__(self, spec, env, head_dim: int):
        super().__init__(spec, env, head_dim)
        p = spec.params
        factor, original = float(p["factor"]), float(p["original"])
        fast, slow = float(p["fast"]), float(p["slow"])
        if factor < 1.0 or original <= 0 or fast <= 0 or slow <= 0 or self.theta <= 1.0:
            raise UnsupportedShape("rotation stretch", (factor, original, fast, slow), "factor >= 1, positive lengths and turns, theta > 1")

        def pair_turning(times: float) -> float:
            return self.rotary_dim * math.log(original / (2.0 * math.pi * times)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(pair_turning(fast)), 0)
        hi = min(math.ceil(pair_turning(slow)), self.rotary_dim - 1)
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        ladder = self.theta ** (-2.0 * i / self.rotary_dim)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        self.inv_freq = (ladder / factor * ramp + ladder * (1.0 - ramp)).to(torch.float32).to(env.device)
        self.magnitude = 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def __init__(self, spec, env, head_dim: int):
        super().__init__(spec, env)

    def rotary(self):
        return None, 0
