"""Rotary position encoding: the float32 cos/sin tables a mixer rotates with.

Angle of pair j at position p: p / theta^(j / (head_dim/2)); the tables are computed in
float64 and rounded once to float32.  Reference: src/models/jiuge/jiuge_weight.hpp:134-186
builds the same tables in float and stores them in the activation type.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import register


@register("position", "rope")
class RotaryTables:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, object]:
        return {}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec = spec
        half = spec.head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv_freq = torch.tensor(float(spec.theta), dtype=torch.float64) ** (-(j / half))
        pos = torch.arange(spec.max_positions, dtype=torch.float64)
        angle = pos[:, None] * inv_freq[None, :]
        self.cos = angle.cos().to(torch.float32).to(runtime.device).contiguous()
        self.sin = angle.sin().to(torch.float32).to(runtime.device).contiguous()
        self.interleaved = bool(spec.interleaved)
