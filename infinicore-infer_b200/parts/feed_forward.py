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

    def plan(self, program, residual_scale: float = 1.0) -> None:
        """Two records: gate | up with the activation (h -> act), down added into the stream times ``residual_scale``."""
        import ctypes
        s = self.spec
        program.emit("jk_emit_swiglu", ctypes.c_void_p(self.w_gate_up.data_ptr()), ctypes.c_void_p(self.w_down.data_ptr()),
                     ctypes.c_int(s.hidden_size), ctypes.c_int(s.intermediate_size), ctypes.c_float(residual_scale),
                     keep=(self.w_gate_up, self.w_down))

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan(program, 1.0), ctx, h, self.spec.hidden_size)
