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
        from ..kernels.host import rotary_tables
        self.spec = spec
        cos, sin = rotary_tables(float(spec.theta), spec.head_dim // 2, spec.max_positions)
        self.cos = torch.from_numpy(cos).to(runtime.device).contiguous()
        self.sin = torch.from_numpy(sin).to(runtime.device).contiguous()
        self.interleaved = bool(spec.interleaved)
        self.max_positions = spec.max_positions
