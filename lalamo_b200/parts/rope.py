"""Rotary position embedding (``lalamo/modules/rope.py:94-102``): the inverse frequencies
``theta ** (-2i / rotary_dim)`` as a 32-bit table; angles, sines and cosines are computed
in 32-bit inside the kernel that applies them.  With a :class:`~lalamo_b200.config.plan.YarnScaling` the
table holds the stretched frequencies and ``magnitude`` the factor on sines and cosines."""

from __future__ import annotations

import math
from typing import Mapping

import torch

from ..config.plan import RopeSpec, YarnScaling
from .base import PositionEncoding, Runtime, register_part

__all__ = ["Rope", "stretched_frequencies"]


def stretched_frequencies(rotary_dim: int, theta: float, scaling: YarnScaling) -> tuple[torch.Tensor, float]:
    """``(frequencies [rotary_dim / 2] in 32-bit, factor on sines and cosines)`` under ``scaling``: pairs below the one that
    turns ``fast`` times within the original context keep their frequency, pairs above the one that turns ``slow`` times
    have it divided by ``factor``, those between are blended linearly in the pair's index.  Worked out in 64-bit."""
    pairs = rotary_dim // 2
    index = torch.arange(pairs, dtype=torch.float64)
    frequency = torch.tensor(float(theta), dtype=torch.float64) ** (-2.0 * index / rotary_dim)

    def pair_turning(turns: float) -> float:
        return rotary_dim * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    low = max(math.floor(pair_turning(scaling.fast)), 0)
    high = min(math.ceil(pair_turning(scaling.slow)), rotary_dim - 1)
    ramp = ((index - low) / max(high - low, 0.001)).clamp(0.0, 1.0)
    blended = frequency / scaling.factor * ramp + frequency * (1.0 - ramp)
    return blended.to(torch.float32), 0.1 * math.log(scaling.factor) + 1.0


@register_part(RopeSpec)
class Rope(PositionEncoding):
    def __init__(self, spec: RopeSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.magnitude = 1.0
        if spec.scaling is None:
            channel = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32)
            inverse = 1.0 / (torch.tensor(spec.theta, dtype=torch.float32) ** (channel / spec.rotary_dim))
        else:
            inverse, self.magnitude = stretched_frequencies(spec.rotary_dim, spec.theta, spec.scaling)
        self.rotary_dim = spec.rotary_dim
        self.inv_freq = inverse.to(device=runtime.device, dtype=torch.float32).contiguous()
