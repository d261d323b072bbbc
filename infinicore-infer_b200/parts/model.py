"""The model: embedding, the layers in their run order, final norm, output product.

Built from a ``ModelSpec`` alone.  ``forward`` runs the rows of one step and returns the
float32 logits of the wanted rows.  Reference: src/models/jiuge/jiuge.cpp:114-298
(``inferDeviceBatch``); the embedding scale, the residual scale and the logit scale are
MiniCPM's (scripts/jiuge.py:97-114) and arrive here as plain numbers of the specification.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights import MATRIX, TensorDecl
from .base import ResidualStream, Runtime, StepContext, part_class


def model_manifest(spec) -> Dict[str, TensorDecl]:
    """Every tensor the model reads, by checkpoint name.  The output matrix is optional: when
    the checkpoint has none the embedding is used (scripts/jiuge.py:182-191)."""
    out = {spec.embed_name: TensorDecl((spec.vocab_size, spec.hidden_size)),
           spec.lm_head_name: TensorDecl((spec.vocab_size, spec.hidden_size), optional=True)}
    for name, decl in part_class("norm", spec.final_norm).tensor_decls(spec.final_norm).items():
        out[spec.final_norm_prefix + name] = decl
    for i, layer in enumerate(spec.layers):
        prefix = spec.layer_prefix.format(i)
        for name, decl in part_class("block", layer).tensor_decls(layer).items():
            out[prefix + name] = decl
    return out


def cache_needs(spec) -> List[object]:
    """What each cache of the run order asks of the cache manager."""
    needs: List[object] = [None] * spec.num_caches
    for e in spec.order:
        if e.writes_cache:
            layer = spec.layers[e.layer]
            needs[e.cache] = part_class("block", layer).cache_need(layer)
    for e in spec.order:
        if not e.writes_cache:
            layer = spec.layers[e.layer]
            mine = part_class("block", layer).cache_need(layer)
            if mine != needs[e.cache]:
                raise ValueError(f"layer {e.layer} reads cache {e.cache}, which holds {needs[e.cache]}, "
                                 f"but needs {mine}")
    return needs


class Model:
    def __init__(self, spec, weights, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.embedding = weights.get(spec.embed_name, MATRIX)
        if weights.has(spec.lm_head_name):
            self.lm_head = weights.get(spec.lm_head_name, MATRIX)
        else:
            self.lm_head = self.embedding       # tied: one copy serves both ends
        self.final_norm = part_class("norm", spec.final_norm)(spec.final_norm, weights,
                                                              spec.final_norm_prefix, runtime)
        self.layers = [part_class("block", layer)(layer, weights, spec.layer_prefix.format(i), runtime)
                       for i, layer in enumerate(spec.layers)]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(layer, "graph_safe", True) for layer in self.layers)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every matrix of every run entry, the output matrix."""
        total = self.lm_head.numel() * self.lm_head.element_size()
        for e in self.spec.order:
            total += getattr(self.layers[e.layer], "weight_bytes", lambda: 0)()
        return total

    def forward(self, ctx: StepContext, views) -> torch.Tensor:
        from .. import kernels
        spec, rt = self.spec, self.runtime
        x = rt.empty(ctx.ntok, spec.hidden_size, dtype=torch.float32)
        kernels.embed(ctx.tokens, self.embedding, spec.embed_scale, x)
        residual = ResidualStream(x)
        for e in spec.order:
            self.layers[e.layer].forward(residual, ctx, views[e.cache], e.writes_cache)
        # the logit scale rides on the final norm, as in the reference (scripts/jiuge.py:198-201)
        h = self.final_norm.forward(residual, ctx, out_scale=spec.logit_scale, rows=ctx.want_rows)
        return rt.linear(h, self.lm_head, out_dtype=torch.float32)
