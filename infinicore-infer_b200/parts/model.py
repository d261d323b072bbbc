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
from .program import Program


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

    def plan(self, views, page_size: int, max_blocks: int) -> Program:
        """The whole model as a program: the embedding, the layers in their run order, the final norm over the wanted
        rows with the logit scale riding on it (as in the reference, scripts/jiuge.py:198-201), the output product."""
        import ctypes
        from .. import kernels
        spec = self.spec
        program = Program(self.runtime, spec.hidden_size, page_size, max_blocks, capacity=8 * len(spec.order) + 8)
        program.emit("jk_emit_embedding", ctypes.c_void_p(self.embedding.data_ptr()), ctypes.c_int(kernels.dtype_code(self.embedding.dtype)),
                     ctypes.c_int(spec.hidden_size), ctypes.c_float(spec.embed_scale), keep=(self.embedding,))
        hidden = spec.hidden_size
        for e in spec.order:
            layer, view = self.layers[e.layer], views[e.cache]
            if hasattr(layer, "plan"):
                layer.plan(program, view, e.writes_cache)
            else:
                program.host(_host_block(layer, view, e.writes_cache, hidden))
        if hasattr(self.final_norm, "plan"):
            self.final_norm.plan(program, out_scale=spec.logit_scale, wanted_rows=True)
        else:
            program.host(_host_final_norm(self.final_norm, spec.logit_scale, hidden))
        program.emit("jk_emit_output", ctypes.c_void_p(self.lm_head.data_ptr()), ctypes.c_int(spec.vocab_size),
                     ctypes.c_int(spec.hidden_size), keep=(self.lm_head,))
        return program


def _host_block(layer, view, writes_cache: bool, hidden: int):
    def run_block(ctx, io):
        stream = ResidualStream(io.view("x", hidden))
        layer.forward(stream, ctx, view, writes_cache)
        stream.value()
    run_block.__qualname__ = type(layer).__name__ + ".forward"
    return run_block


def _host_final_norm(norm, logit_scale: float, hidden: int):
    def run_final_norm(ctx, io):
        out = norm.forward(ResidualStream(io.view("x", hidden)), ctx, out_scale=logit_scale, rows=ctx.want_rows)
        io.view("hw", hidden, rows=out.shape[0]).copy_(out)
    run_final_norm.__qualname__ = type(norm).__name__ + ".forward"
    return run_final_norm
