"""Typed descriptions of a model: what each part is and which constants it has.

A specification is plain, frozen data.  It holds every size and constant that a
part needs, so that the part itself never looks at a model's configuration.  A
``ModelSpec`` is a list of layer specifications plus the order in which the
layers run; one model can therefore have different mixers and feed-forwards in
different layers, run a layer twice, or let a layer read another layer's cache.

Every specification has a ``kind``: the key under which the implementing class
is registered in ``parts``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that is incomplete or inconsistent."""


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * w / sqrt(mean(x^2) + eps)  (reference: src/models/jiuge/jiuge.cpp:198)."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding of query and key heads.

    Angle of pair ``j`` at position ``p``: ``p / theta ** (j / (head_dim / 2))``
    (reference: src/models/jiuge/jiuge_weight.hpp:134-186).  ``interleaved``
    False pairs element ``j`` with ``j + head_dim/2`` (the checkpoint's own
    layout); True pairs ``2j`` with ``2j+1`` (the layout the reference's loader
    permutes the rows to, scripts/jiuge.py:217-227).
    """
    head_dim: int
    theta: float
    max_positions: int
    interleaved: bool = False
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention over a paged key/value cache.

    ``window`` None: every earlier key is seen.  ``window`` W: a query at
    position p sees keys at positions p-W+1 .. p.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    softmax_scale: float
    position: Optional[RopeSpec] = None
    window: Optional[int] = None
    bias: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate(x)) * up(x))  (reference: src/models/jiuge/jiuge.cpp:247-249)."""
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: x += s * mixer(norm_a(x)); x += s * feed_forward(norm_b(x)).

    The four ``*_prefix`` strings are the names, below the layer's own prefix,
    under which the checkpoint stores each part's tensors.
    """
    mixer: object
    feed_forward: object
    mixer_norm: object
    ffn_norm: object
    residual_scale: float = 1.0
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    ffn_norm_prefix: str = "post_attention_layernorm."
    kind: str = "prenorm"


@dataclass(frozen=True)
class RunEntry:
    """One entry of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (whose weights run), ``cache`` names
    the cache the mixer works on.  ``writes_cache`` False means the mixer only
    reads what an earlier entry with the same ``cache`` wrote in this step.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[RunEntry, ...]
    final_norm: object
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    tie_embeddings: bool = False
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm."
    layer_prefix: str = "model.layers.{}."
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self):
        n = len(self.layers)
        writers = {}
        for pos, e in enumerate(self.order):
            if not 0 <= e.layer < n:
                raise ConfigError(f"order[{pos}] names layer {e.layer}, but there are {n} layers")
            if e.writes_cache:
                if e.cache in writers:
                    raise ConfigError(
                        f"order[{pos}] and order[{writers[e.cache]}] both write cache {e.cache}")
                writers[e.cache] = pos
            elif e.cache not in writers:
                raise ConfigError(
                    f"order[{pos}] reads cache {e.cache} before any entry has written it")

    @property
    def num_caches(self) -> int:
        return 1 + max(e.cache for e in self.order) if self.order else 0


def default_order(num_layers: int) -> Tuple[RunEntry, ...]:
    """Every layer once, in sequence, each with a cache of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(num_layers))
