"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)).

Reference: src/models/jiuge/jiuge.cpp:247-249 — one fused gate|up product, the SwiGLU
operator over its two halves (jiuge.cpp:191-192), the down product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights import MATRIX, TensorDecl
from .base import register


@register("feed_forward", "swiglu")
class SwiGLU:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, di = spec.hidden_size, spec.intermediate_size
        return {"gate_proj.weight": TensorDecl((di, d)), "up_proj.weight": TensorDecl((di, d)),
                "down_proj.weight": TensorDecl((d, di))}

    @staticmethod
    def pack(spec, weights, prefix: str) -> Dict[str, torch.Tensor]:
        """The layer's tensors as the kernels take them: one fused matrix of the gate rows followed by the up rows
        (scripts/jiuge.py:311-323) and the down matrix.  The one place where this packing is written."""
        return {"w_gate_up": weights.get_rows([prefix + "gate_proj.weight", prefix + "up_proj.weight"], MATRIX),
                "w_down": weights.get(prefix + "down_proj.weight", MATRIX)}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        packed = self.pack(spec, weights, prefix)
        self.w_gate_up, self.w_down = packed["w_gate_up"], packed["w_down"]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        act = rt.gate_up_swiglu(h, self.w_gate_up)
        return rt.product(act, self.w_down)      # the block adds it to the residual stream
