"""Position encodings.

``rope``: non-interleaved ("rotate half") rotary positions over the whole head size. The tables
are built once in float64 and stored in float32, as the reference does
(src/llmserve/models/layers.py:47-63); they stay float32 in the bfloat16 path too, so rotation
angles are never rounded to 16 bits. Frequency scaling ``linear`` and ``llama3`` follow
src/llmserve/models/layers.py:24-58.

``none``: no position information (for mixers that carry order in their own state).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


@dataclass(frozen=True)
class RotarySpec:
    head_dim: int
    theta: float
    scaling_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_positions: int = 0
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


def rotary_inverse_frequencies(spec: RotarySpec) -> torch.Tensor:
    """float64 ``[head_dim/2]``."""
    d = spec.head_dim
    inv = 1.0 / (spec.theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    if spec.scaling_type == "linear":
        inv = inv / spec.factor
    elif spec.scaling_type == "llama3":
        old = spec.original_max_positions
        low_wavelen = old / spec.low_freq_factor
        high_wavelen = old / spec.high_freq_factor
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > low_wavelen, inv / spec.factor, inv)
        smooth = (old / wavelen - spec.low_freq_factor) / (
            spec.high_freq_factor - spec.low_freq_factor
        )
        mid = (1 - smooth) * scaled / spec.factor + smooth * scaled
        is_mid = (wavelen >= high_wavelen) & (wavelen <= low_wavelen)
        inv = torch.where(is_mid, mid, scaled)
    elif spec.scaling_type != "default":
        raise NotImplementedError(f"rope scaling {spec.scaling_type!r}")
    return inv


@POSITION_ENCODINGS.register("rope")
class RotaryPositionEncoding(PositionEncoding):
    def __init__(self, spec: RotarySpec, env) -> None:
        super().__init__(spec, env)
        if spec.head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {spec.head_dim}")
        inv = rotary_inverse_frequencies(spec)
        ang = torch.outer(torch.arange(env.max_positions, dtype=torch.float64), inv)
        self.cos = ang.cos().float().contiguous().to(env.device)
        self.sin = ang.sin().float().contiguous().to(env.device)

    def rotary_tables(self):
        return self.cos, self.sin


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    pass
