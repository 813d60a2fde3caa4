"""Position encodings applied to queries and keys inside a mixer.

A position encoding is anything that can be given as a rotation table per position:
``rotation_tables`` returns float32 cos/sin [max_positions, rotary_dim/2], and the
fused kernel rotates the pair (d, d + rotary_dim/2) of each head with them (or, with the spec's
``interleaved``, the neighbours (2 d, 2 d + 1)). Scaled or
partial rotary variants only change the table; "none" returns no table.

"rope" is the reference's rotate-half encoding over the full head:
inv_freq[i] = 1 / theta^(2i / rotary_dim), angle = pos * inv_freq[i], both in float32
(pegainfer-core/src/weight_loader.rs:730-764). The reference rounds the table to
bfloat16; here it stays float32.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from .base import PositionEncoding
from .registry import register_position_encoding
from .spec import PositionSpec

# tables are shared by all layers with the same constants on a device
_TABLES: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


@register_position_encoding("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PositionSpec) -> None:
        super().__init__(spec)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        if spec.max_positions <= 0:
            raise ValueError("max_positions must be positive")

    def rotation_tables(self, device: torch.device):
        s = self.spec
        key = (s.rotary_dim, float(s.theta), s.max_positions, s.scaling, s.precise, s.yarn, str(device))
        if key not in _TABLES:
            half = s.rotary_dim // 2
            amplitude = 1.0
            if s.yarn is not None:
                # frequencies mixed between f and f / factor by a ramp over the pair index, whose ends are the pairs that
                # make ``fast`` and ``slow`` turns within ``original`` positions; cos and sin scaled by 0.1 ln(factor) + 1
                if s.scaling is not None:
                    raise ValueError("a rotary encoding takes one way of stretching its waves, not two")
                factor, original, fast, slow = (float(v) for v in s.yarn)
                idx = torch.arange(half, dtype=torch.float64)
                f = float(s.theta) ** (-2.0 * idx / s.rotary_dim)

                def turns(t: float) -> float:
                    return s.rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(s.theta)))

                lo = max(math.floor(turns(fast)), 0)
                hi = min(math.ceil(turns(slow)), s.rotary_dim - 1)
                ramp = torch.clamp((idx - lo) / max(hi - lo, 0.001), 0.0, 1.0)
                f = f / factor * ramp + f * (1.0 - ramp)
                amplitude = 0.1 * math.log(factor) + 1.0
                ang = torch.arange(s.max_positions, dtype=torch.float64)[:, None] * f[None, :]
            elif s.scaling is None and not s.precise:
                idx = torch.arange(half, dtype=torch.float32)
                inv_freq = 1.0 / torch.pow(torch.tensor(float(s.theta), dtype=torch.float32),
                                           idx * 2.0 / s.rotary_dim)
                ang = torch.arange(s.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
            else:
                # stretched long waves: frequencies and angles are formed in float64; cos and sin are rounded once to float32
                idx = torch.arange(half, dtype=torch.float64)
                f = float(s.theta) ** (-2.0 * idx / s.rotary_dim)
                factor, low, high, original = (float(v) for v in s.scaling) if s.scaling is not None else (1.0, 1.0, 2.0, 1.0)
                wave = 2.0 * math.pi / f
                # (high == low leaves no band between the two regimes: nothing is mixed)
                t = (original / wave - low) / (high - low) if high != low else torch.zeros_like(wave)
                f = torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, (1.0 - t) * f / factor + t * f))
                ang = torch.arange(s.max_positions, dtype=torch.float64)[:, None] * f[None, :]
            _TABLES[key] = ((torch.cos(ang) * amplitude).to(torch.float32).contiguous().to(device),
                            (torch.sin(ang) * amplitude).to(torch.float32).contiguous().to(device))
        return _TABLES[key]


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    def rotation_tables(self, device: torch.device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        return None
