"""RMSNorm: y = x * w / sqrt(mean(x^2) + eps), computed in float32.

Reference: ``rmsnorm`` at src/models/jiuge/jiuge.cpp:198, :246, :262 with a float32 weight
(scripts/jiuge.py:145-146).  The pending residual addition is done by the same kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..weights import VECTOR, TensorDecl
from .base import ResidualStream, register


@register("norm", "rmsnorm")
class RMSNorm:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.size,), VECTOR, init="ones")}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        self.weight = weights.get(prefix + "weight", VECTOR)

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def plan(self, program, out_scale: float = 1.0, wanted_rows: bool = False) -> None:
        """One record: add what waits for the stream, normalise every row (or the wanted rows) into the next product's
        activations."""
        import ctypes
        program.emit("jk_emit_rmsnorm", ctypes.c_void_p(self.weight.data_ptr()), ctypes.c_int(self.spec.size),
                     ctypes.c_float(self.spec.eps), ctypes.c_float(out_scale), ctypes.c_int(1 if wanted_rows else 0),
                     keep=(self.weight,))

    def forward(self, residual: ResidualStream, ctx, out_scale: float = 1.0,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalise every row, or only ``rows`` (int32 indices) of the residual stream."""
        from .. import kernels
        n = rows.numel() if rows is not None else residual.x.shape[0]
        out = self.runtime.empty(n, self.spec.size)
        delta, scale = residual.take_pending()
        kernels.add_rmsnorm(residual.x, delta, scale, self.weight, self.spec.eps, out, out_scale, rows)
        return out
