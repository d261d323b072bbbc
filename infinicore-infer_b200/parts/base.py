"""What parts are made of: registries, the runtime, the step context, the residual stream.

A part is a class registered under the ``kind`` of its specification.  It is built from
(specification, weight source, name prefix, runtime) and knows nothing else: not the model
it is in, not the other layers.  Four registries hold the four families:

    norm            forward(residual, ctx, out_scale=1.0, rows=None) -> tensor [rows, size]
    position        tables for a mixer; an object the mixer knows how to use
    mixer           cache_need(spec) -> a cache need (``PagedKV``, ``StateSlot``, ...) or None   (static)
                    forward(h, ctx, view, writes_cache) -> tensor [T, hidden]
    feed_forward    forward(h, ctx) -> tensor [T, hidden]
    block           forward(residual, ctx, view, writes_cache) -> None

A part may also have ``plan(program, ...)`` (see ``parts/program.py``): it then says what it does as launch records
that the native step replays, and its ``forward`` is the same records run alone.  A part without ``plan`` runs by its
``forward`` as a host step of the program.

Every part class also has ``tensor_decls(spec) -> {local name: TensorDecl}``, a static
method that needs no GPU: the model's manifest, the loader's checks and the random-weights
mode are all derived from it.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}

_FAMILIES = {"norm": NORMS, "position": POSITIONS, "mixer": MIXERS,
             "feed_forward": FEED_FORWARDS, "block": BLOCKS}


def register(family: str, kind: str) -> Callable[[type], type]:
    """Class decorator: ``@register("mixer", "attention")``."""
    table = _FAMILIES[family]

    def deco(cls: type) -> type:
        table[kind] = cls
        return cls
    return deco


def part_class(family: str, spec) -> type:
    table = _FAMILIES[family]
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise KeyError(f"no {family} registered under kind {kind!r}; known: {sorted(table)}")
    return table[kind]


class Runtime:
    """The precision and device a model runs in, and the switches of the native step.

    ``dtype`` float32: every product runs on the CUDA cores in float32 (no tensor cores, no TF32).  ``dtype``
    bfloat16: operands are bfloat16, accumulation and (where asked) the output are float32; a product goes to this
    package's own kernels or to the library, as the reference sends its products to one
    (src/models/inference_context.cpp:59-79).  Which kernel takes which product is decided in ONE place, the native
    step (csrc/runner.cu by the rules of csrc/host_rules.h); the numbers below are what that decision reads.
    """

    def __init__(self, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        self.plain_attention = False      # True: bfloat16 attention through the row kernel too
        self.library_products_only = False   # True: every bfloat16 product goes to the library
        self.legacy_tensor_cores = False     # True: prefill attention on mma.sync even where tcgen05 is built
        # the tiled tcgen05 product takes a product from this many rows, output tiles of 128 x 128 and per cent of its
        # rows of tiles filled (jk::takes_tcgen05 of csrc/host_rules.h says where the numbers come from)
        self.tcgen05_min_rows = 129
        self.tcgen05_min_tiles = 200
        self.tcgen05_min_fill_pct = 80
        # fewest blocks for the few-rows tcgen05 kernel (None: one per SM); JK_SKINNY_MIN_BLOCKS=n sets it for a comparison
        self.skinny_min_blocks: Optional[int] = int(os.environ["JK_SKINNY_MIN_BLOCKS"]) if os.environ.get("JK_SKINNY_MIN_BLOCKS") else None
        # steps of at most 16 rows run without norm kernels (the products around a norm share its work:
        # csrc/linear_small.cu, SmallNormFuse); JK_NO_FUSED_NORM=1 keeps the norm kernels
        self.fused_norms = os.environ.get("JK_NO_FUSED_NORM") != "1"

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def routing(self):
        """(sms, tcgen05_min_rows, tcgen05_min_tiles, tcgen05_min_fill_pct, skinny_min_blocks, library_only): what
        ``jk::product_route`` reads."""
        from .. import kernels
        sms = kernels._sm_count(self.device) if self.device.type == "cuda" else 148
        return (sms, self.tcgen05_min_rows, self.tcgen05_min_tiles, self.tcgen05_min_fill_pct, self.skinny_min_blocks or 0,
                1 if self.library_products_only else 0)

    def routing_key(self):
        return self.routing() + (self.fused_norms, self.plain_attention, self.legacy_tensor_cores)

    def env(self, page_size: int, max_blocks: int):
        """The ``RunnerEnv`` of csrc/runner.h for this runtime and a cache with these pages."""
        from .. import kernels
        from .program import Routing, RunnerEnv
        return RunnerEnv(dtype=kernels.dtype_code(self.dtype), page_size=page_size, max_blocks=max_blocks,
                         fused_norms=1 if self.fused_norms else 0, plain_attention=1 if self.plain_attention else 0,
                         legacy_tensor_cores=1 if self.legacy_tensor_cores else 0, routing=Routing(*self.routing()),
                         status=kernels.gemm_status(self.device).data_ptr())


@dataclass
class StepContext:
    """One step's batch, as the parts see it.

    Rows of all requests are concatenated: request i owns rows
    ``req_start[i] .. req_start[i+1]-1`` at positions ``req_pos[i] ...``.  The ``host_*``
    lists mirror the device arrays for parts that work on the host side.
    """
    ntok: int
    nreq: int
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T]   absolute position of each row
    row_req: torch.Tensor           # int32 [T]   batch entry of each row
    req_start: torch.Tensor         # int32 [nreq + 1]
    req_pos: torch.Tensor           # int32 [nreq] position of each request's first row
    slot_ids: torch.Tensor          # int32 [nreq] state slot of each request
    block_tables: List[torch.Tensor]  # per cache group: int32 [nreq, max_blocks]
    want_rows: torch.Tensor         # int32 [n_want] rows whose logits are wanted
    n_want: int
    # the context length the step is planned for: a bucket of the live requests' lengths (0: the model's longest)
    context: int = 0
    # Work lists that the model's mixers asked for (``Mixer.step_lists``): name -> (int32 view or None, entries).
    # None with n entries stands for the rows 0..n-1.
    lists: Dict[str, tuple] = field(default_factory=dict)
    host_req_start: List[int] = field(default_factory=list)
    host_req_pos: List[int] = field(default_factory=list)
    host_slot_ids: List[int] = field(default_factory=list)
    decode_only: bool = False


class ResidualStream:
    """The float32 residual ``x`` plus at most one addition that has not been done yet: what a part that runs as a
    host step (its own ``forward``) works on.

    A mixer or feed-forward returns its output; the block calls ``add(delta, scale)``.  The sum is put off so that
    the next norm can do ``x += scale * delta`` and the normalisation in one kernel.  ``value()`` makes the stream
    whole for a part that wants plain ``x``.
    """

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.delta: Optional[torch.Tensor] = None
        self.scale: float = 1.0

    def add(self, delta: torch.Tensor, scale: float = 1.0) -> None:
        """x += scale * delta, now or at the next norm."""
        if self.delta is not None:
            self.value()
        self.delta, self.scale = delta, scale

    def take_pending(self):
        d, s = self.delta, self.scale
        self.delta, self.scale = None, 1.0
        return d, s

    def value(self) -> torch.Tensor:
        if self.delta is not None:
            from .. import kernels
            d, s = self.take_pending()
            if d.dtype not in (torch.float32, torch.bfloat16):
                d = d.float()
            kernels.residual_add(self.x, d.contiguous(), s)
        return self.x
