"""What parts are made of: registries, the runtime, the step context, the residual stream.

A part is a class registered under the ``kind`` of its specification.  It is built from
(specification, weight source, name prefix, runtime) and knows nothing else: not the model
it is in, not the other layers.  Four registries hold the four families:

    norm            forward(residual, ctx, out_scale=1.0, rows=None) -> tensor [rows, size]
    position        tables for a mixer; an object the mixer knows how to use
    mixer           cache_need(spec) -> PagedKV | StateSlot | None   (static)
                    forward(h, ctx, view, writes_cache) -> tensor [T, hidden] or PendingProduct
    feed_forward    forward(h, ctx) -> tensor [T, hidden] or PendingProduct
    block           forward(residual, ctx, view, writes_cache) -> None

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
    """The precision and device a model runs in, and the matrix product the parts use.

    ``dtype`` float32: every product runs on the CUDA cores in float32 (no tensor cores, no
    TF32).  ``dtype`` bfloat16: operands are bfloat16, accumulation and (where asked) the
    output are float32; the product goes to the library, as the reference sends its products
    to one (src/models/inference_context.cpp:59-79), or to this package's own kernels.
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
        # rows of tiles filled (takes_tcgen05 says where the numbers come from)
        self.tcgen05_min_rows = 129
        self.tcgen05_min_tiles = 200
        self.tcgen05_min_fill_pct = 80
        self.skinny_min_blocks: Optional[int] = None   # fewest blocks for the few-rows tcgen05 kernel (None: one per SM)
        # the native runner runs steps of at most 16 rows without norm kernels (the products around a norm share its
        # work: csrc/linear_small.cu, SmallNormFuse); JK_NO_FUSED_NORM=1 keeps the norm kernels
        self.fused_norms = os.environ.get("JK_NO_FUSED_NORM") != "1"

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def linear(self, h: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h [T, K] times weight [N, K] transposed -> [T, N]."""
        from .. import kernels
        if self.dtype == torch.float32:
            out = self.empty(h.shape[0], weight.shape[0], dtype=torch.float32)
            return kernels.gemm_f32(h, weight, out, bias)
        out_dtype = out_dtype or torch.bfloat16
        m, k = h.shape
        n = weight.shape[0]
        if not self.library_products_only:
            route = self.few_rows_route(m, n, k, "f32") if out_dtype == torch.float32 else "library"
            if route == "small":
                out = kernels.linear_small(h, weight, self.empty(m, n, dtype=torch.float32))
                return out if bias is None else out.add_(bias)
            if route == "skinny":
                out = kernels.gemm_skinny(h, weight, self.empty(m, n, dtype=torch.float32), kernels.TG_F32)
                return out if bias is None else out.add_(bias)
            if self.takes_tcgen05(m, n, k):
                out = kernels.gemm_tcgen05(h, weight, self.empty(m, n, dtype=out_dtype),
                                           kernels.TG_F32 if out_dtype == torch.float32 else kernels.TG_BF16)
                return out if bias is None else out.add_(bias.to(out.dtype))
        if out_dtype == torch.bfloat16:
            out = torch.mm(h, weight.t())
        else:
            out = torch.mm(h, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            out += bias.to(out.dtype)
        return out


    def gate_up_swiglu(self, h: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
        """silu(h @ Wg^T) * (h @ Wu^T) for the fused [gate | up] matrix -> [T, intermediate]."""
        from .. import kernels
        m, k = h.shape
        di = w_gate_up.shape[0] // 2
        act = self.empty(m, di)
        if self.dtype == torch.bfloat16 and not self.library_products_only:
            route = self.few_rows_route(m, di, k, "swiglu")
            if route == "small":
                return kernels.linear_small(h, w_gate_up, act, kernels.EPI_SWIGLU)
            if route == "skinny":
                return kernels.gemm_skinny(h, w_gate_up, act, kernels.TG_SWIGLU)
            if self.takes_tcgen05(m, di, k):
                return kernels.gemm_tcgen05(h, w_gate_up, act, kernels.TG_SWIGLU)
        gu = self.linear(h, w_gate_up, out_dtype=torch.float32)
        return kernels.swiglu(gu, act)

    def product(self, act: torch.Tensor, weight: torch.Tensor) -> "PendingProduct":
        """act @ weight^T that has not run yet: whoever takes it decides where the result goes (a
        tensor of its own, or straight into the residual stream)."""
        return PendingProduct(self, act, weight)

    def few_rows_route(self, m: int, n: int, k: int, kind: str) -> str:
        """Which kernel takes a bfloat16 product of at most 128 rows: ``"small"`` (the weight-streaming kernels of
        the CUDA cores, up to 16 rows), ``"skinny"`` (the tcgen05 kernel with the weights on the MMA's M side)
        or ``"library"``.  ``kind``: "f32" (plain output), "residual" (added into the stream), "swiglu" (``n`` is
        the width after the activation).  Measured on the 2B and 8B shapes: the skinny kernel reads at 5 to 6 TB/s
        once it has a block for every SM (output tiles of 128 features, 64 for SwiGLU, times the splits of K that a
        residual product allows); the small kernel loads a tile's whole slice of K before it computes, so it needs
        a second block on the SM to overlap with (a slice of 16 rows x K fits twice) or so few tiles that they
        make one wave."""
        from .. import kernels
        if self.dtype != torch.bfloat16 or self.library_products_only or m > 128:
            return "library"
        sms = kernels._sm_count(self.device)
        need = sms if self.skinny_min_blocks is None else self.skinny_min_blocks
        nk = -(-k // 64)
        if kind == "swiglu":
            blocks = -(-n // 64)
        else:
            tiles = -(-n // 128)
            splits = max(1, min(2 * sms // tiles, nk // 8)) if kind == "residual" else 1
            blocks = tiles * (-(-nk // -(-nk // splits)))
        skinny = blocks >= need and kernels.gemm_skinny_supports(m, n, k)
        if m <= 16:
            rows = 2 * n if kind == "swiglu" else n
            if kernels.linear_small_supports(m, n, k):
                if not skinny or 2 * (32 * k + 8192) <= 227 * 1024 or -(-rows // 16) <= sms:
                    return "small"
        return "skinny" if skinny else "library"

    def takes_tcgen05(self, m: int, n: int, k: int) -> bool:
        """Whether the tiled tcgen05 product takes this product (the same rule as runner_takes_tcgen05 in csrc/runner.h).
        Measured on the 1B, 2B and 8B shapes, whole steps of 160 to 2,048 rows against the library's product with
        separate elementwise kernels: a product with at least 200 output tiles of 128 x 128 whose rows fill their
        tiles of 128 to four fifths is as fast or faster here (fused epilogues, dependent launch, cuts of K for the
        products that add into the residual stream); products of fewer tiles go to the library, whose smaller tiles
        fill the SMs better.  Very wide outputs (the logits) are taken from 17 rows."""
        from .. import kernels
        if self.dtype != torch.bfloat16 or self.library_products_only or m <= 16 or not kernels.gemm_tcgen05_supports(m, n, k):
            return False
        row_tiles = -(-m // 128)
        if row_tiles * -(-n // 256) >= 3 * kernels._sm_count(self.device):
            return True
        if m < self.tcgen05_min_rows or m * 100 < self.tcgen05_min_fill_pct * row_tiles * 128:
            return False
        return row_tiles * -(-n // 128) >= self.tcgen05_min_tiles

    def fuses_residual(self, m: int, n: int, k: int) -> bool:
        return self.few_rows_route(m, n, k, "residual") == "skinny" or self.takes_tcgen05(m, n, k)


class PendingProduct:
    """A matrix product put off until its consumer is known (see ``ResidualStream.add``)."""

    def __init__(self, runtime: Runtime, act: torch.Tensor, weight: torch.Tensor):
        self.runtime, self.act, self.weight = runtime, act, weight

    def tensor(self, out_dtype: Optional[torch.dtype] = torch.float32) -> torch.Tensor:
        return self.runtime.linear(self.act, self.weight, out_dtype=out_dtype)

    def add_into(self, x: torch.Tensor, scale: float) -> bool:
        """x += scale * product in the product's own epilogue, if the runtime has such a kernel."""
        from .. import kernels
        m, k = self.act.shape
        n = self.weight.shape[0]
        if self.runtime.few_rows_route(m, n, k, "residual") == "skinny":
            kernels.gemm_skinny(self.act, self.weight, x, kernels.TG_RESIDUAL, scale)
            return True
        if not self.runtime.takes_tcgen05(m, n, k):
            return False
        kernels.gemm_tcgen05(self.act, self.weight, x, kernels.TG_RESIDUAL, scale)
        return True


SHORT_ROWS = 8      # a request with at most this many rows in a step counts as "few rows"
TILE_ROWS = 128     # rows per tile of the others; the same constant as kernels.TILE_ROWS (a test holds them equal)


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
    # Work lists for mixers that treat few-row and many-row requests differently: the rows of
    # requests that bring at most SHORT_ROWS rows, and TILE_ROWS-row tiles (batch entry, first row) of the rest.
    short_rows: Optional[torch.Tensor] = None     # int32 [n_short]; None means rows 0..n_short-1
    n_short: int = 0
    tiles: Optional[torch.Tensor] = None          # int32 [n_tiles, 2]
    n_tiles: int = 0
    host_req_start: List[int] = field(default_factory=list)
    host_req_pos: List[int] = field(default_factory=list)
    host_slot_ids: List[int] = field(default_factory=list)
    decode_only: bool = False


class ResidualStream:
    """The float32 residual ``x`` plus at most one addition that has not been done yet.

    A mixer or feed-forward returns its output; the block calls ``add(delta, scale)``.  The
    sum is put off so that the next norm can do ``x += scale * delta`` and the normalisation
    in one kernel.  ``value()`` makes the stream whole for a part that wants plain ``x``.
    """

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.delta: Optional[torch.Tensor] = None
        self.scale: float = 1.0

    def add(self, delta, scale: float = 1.0) -> None:
        """x += scale * delta, now or at the next norm.  ``delta`` is a tensor or a ``PendingProduct``;
        a pending product is added by its own epilogue where the runtime can do that."""
        if self.delta is not None:
            self.value()
        if isinstance(delta, PendingProduct):
            if delta.add_into(self.x, scale):
                return
            delta = delta.tensor(torch.float32)
        self.delta, self.scale = delta, scale

    def take_pending(self):
        d, s = self.delta, self.scale
        self.delta, self.scale = None, 1.0
        return d, s

    def value(self) -> torch.Tensor:
        if self.delta is not None:
            from .. import kernels
            d, s = self.take_pending()
            kernels.residual_add(self.x, d, s)
        return self.x
