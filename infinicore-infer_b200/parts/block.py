"""The pre-norm residual block: x += s * mixer(norm_a(x)); x += s * feed_forward(norm_b(x)).

Reference: one iteration of the layer loop, src/models/jiuge/jiuge.cpp:195-258; ``s`` is
MiniCPM's scale_depth / sqrt(num_layers), which the reference multiplies into the output
and down matrices on the host (scripts/jiuge.py:297, :348) and which stays a float32
constant of the block here.
"""
from __future__ import annotations

from typing import Dict

from ..weights import TensorDecl
from .base import ResidualStream, part_class, register


@register("block", "prenorm")
class PreNormBlock:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        out = {}
        for sub, prefix, family in _children(spec):
            for name, decl in part_class(family, sub).tensor_decls(sub).items():
                out[prefix + name] = decl
        return out

    @staticmethod
    def cache_need(spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec = spec
        build = lambda family, sub, p: part_class(family, sub)(sub, weights, prefix + p, runtime)
        self.mixer_norm = build("norm", spec.mixer_norm, spec.mixer_norm_prefix)
        self.mixer = build("mixer", spec.mixer, spec.mixer_prefix)
        self.ffn_norm = build("norm", spec.ffn_norm, spec.ffn_norm_prefix)
        self.feed_forward = build("feed_forward", spec.feed_forward, spec.ffn_prefix)

    @property
    def graph_safe(self) -> bool:
        """False if a part reads the step's host-side lists: its work cannot be replayed from a graph."""
        parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
        return all(getattr(p, "graph_safe", True) for p in parts)

    def weight_bytes(self) -> int:
        """Bytes of weights one pass over this block reads."""
        parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
        return sum(p.weight_bytes() for p in parts if hasattr(p, "weight_bytes"))

    def plan(self, program, view, writes_cache: bool = True) -> None:
        """The block as records, part by part.  A part that has ``plan`` emits its own; one that has not (a part of
        another kind, defined elsewhere) runs by its ``forward`` as a host step between the records."""
        s = self.spec.residual_scale
        hidden = program.hidden_size
        for norm, part, is_mixer in ((self.mixer_norm, self.mixer, True), (self.ffn_norm, self.feed_forward, False)):
            if hasattr(norm, "plan"):
                norm.plan(program)
            else:
                program.host(_host_norm(norm, hidden))
            if hasattr(part, "plan"):
                part.plan(program, view, writes_cache, s) if is_mixer else part.plan(program, s)
            else:
                program.host(_host_branch(part, view, writes_cache, s, hidden, is_mixer))

    def forward(self, residual: ResidualStream, ctx, view, writes_cache: bool = True) -> None:
        """The block by its parts' own ``forward``: what a model that arranges blocks by hand calls."""
        s = self.spec.residual_scale
        h = self.mixer_norm.forward(residual, ctx)
        residual.add(self.mixer.forward(h, ctx, view, writes_cache), s)
        h = self.ffn_norm.forward(residual, ctx)
        residual.add(self.feed_forward.forward(h, ctx), s)


def _host_norm(norm, hidden: int):
    def run_norm(ctx, io):
        out = norm.forward(ResidualStream(io.view("x", hidden)), ctx)
        io.view("h", hidden).copy_(out)
    run_norm.__qualname__ = type(norm).__name__ + ".forward"
    return run_norm


def _host_branch(part, view, writes_cache: bool, scale: float, hidden: int, is_mixer: bool):
    def run_branch(ctx, io):
        h = io.view("h", hidden)
        delta = part.forward(h, ctx, view, writes_cache) if is_mixer else part.forward(h, ctx)
        stream = ResidualStream(io.view("x", hidden))
        stream.add(delta, scale)
        stream.value()
    run_branch.__qualname__ = type(part).__name__ + ".forward"
    return run_branch


def _children(spec):
    return ((spec.mixer_norm, spec.mixer_norm_prefix, "norm"), (spec.mixer, spec.mixer_prefix, "mixer"),
            (spec.ffn_norm, spec.ffn_norm_prefix, "norm"), (spec.feed_forward, spec.ffn_prefix, "feed_forward"))
