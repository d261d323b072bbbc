"""Bindings of the host-side rules (``csrc/host_rules.h`` through ``csrc/host.cpp``): the page pool, the layout and
packing of a step's metadata, the attention mixer's work lists, the cuts of the decode attention, the product routes,
the rotary tables and the uniform numbers.  Each rule is written once, in C++, and used from there by the native step,
the C interface and (through this file) the Python engine.  The module has no device code and loads without CUDA.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from . import build as _build

_c_int, _c_p = ctypes.c_int, ctypes.c_void_p
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        h = _build.load("host")
        h.jk_pool_create.restype = _c_p
        h.jk_pool_create.argtypes = [_c_int, _c_int]
        for name in ("jk_pool_destroy", "jk_pool_available", "jk_pool_high_water"):
            getattr(h, name).argtypes = [_c_p]
        h.jk_pool_destroy.restype = None
        h.jk_pool_alloc.argtypes = [_c_p, _c_int, _c_p]
        h.jk_pool_free.argtypes = [_c_p, _c_p, _c_int]
        h.jk_pool_is_held.argtypes = [_c_p, _c_int]
        h.jk_decode_scratch_floats.restype = ctypes.c_longlong
        h.jk_uniform_for.restype = ctypes.c_float
        h.jk_uniform_for.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong]
        h.jk_rotary_tables.argtypes = [ctypes.c_double, _c_int, _c_int, ctypes.c_double, _c_p, _c_p]
        h.jk_rotary_tables.restype = None
        h.jk_step_layout.argtypes = [_c_int] * 5 + [_c_p]
        h.jk_pack_step.argtypes = [_c_p] + [_c_int] * 4 + [_c_p] * 5 + [_c_int] * 3 + [_c_p]
        h.jk_attention_work_lists.argtypes = [_c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p]
        h.jk_attention_work_lists.restype = None
        _lib = h
    return _lib


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


def _i32(values) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(values, dtype=np.int32))


# ---- constants -------------------------------------------------------------------------------------------------
def max_cache_groups() -> int:
    return lib().jk_max_cache_groups()


def max_step_lists() -> int:
    return lib().jk_max_step_lists()


def attention_short_rows() -> int:
    """A request with at most this many rows in a step goes to the decode attention row by row."""
    return lib().jk_attention_short_rows()


def attention_tile_rows() -> int:
    """Query rows per tile of the prefill attention kernels."""
    return lib().jk_attention_tile_rows()


# ---- the layout of a step's metadata -------------------------------------------------------------------------------
class StepLayout:
    """Offsets (in int32 elements) of a step's arrays inside the metadata buffer (``jk::StepLayout``)."""

    def __init__(self, T: int, B: int, n_groups: int, max_blocks: int, extra_words: int):
        g = max_cache_groups()
        if n_groups > g:
            raise ValueError(f"{n_groups} cache groups; a step's metadata holds {g} block tables")
        off = (ctypes.c_int * (8 + g))()
        self.total = lib().jk_step_layout(T, B, n_groups, max_blocks, extra_words, off)
        (self.tokens, self.positions, self.row_req, self.want_rows, self.req_start, self.req_pos, self.slot_ids) = off[:7]
        self.tables = list(off[7:7 + n_groups])
        self.extra = off[7 + g]
        self.T, self.B, self.n_groups, self.max_blocks, self.extra_words = T, B, n_groups, max_blocks, extra_words


def pack_step(host: np.ndarray, lay: StepLayout, B: int, tokens, lens, starts, slots, want,
              tables: Sequence[Optional[np.ndarray]]) -> int:
    """Zero ``host[:lay.total]`` and pack a batch of ``B`` requests into it, padded to ``lay.B`` requests (see
    ``jk::pack_step``).  ``tables[g]``: int32 ``[B, max_blocks]`` or None.  Returns the number of rows."""
    tokens, lens, starts, slots, want = _i32(tokens), _i32(lens), _i32(starts), _i32(slots), _i32(want)
    keep = [None if t is None else np.ascontiguousarray(t, dtype=np.int32) for t in tables]
    ptrs = (ctypes.c_void_p * max(1, len(keep)))(*[_ptr(t) for t in keep])
    return lib().jk_pack_step(host.ctypes.data, lay.T, B, lay.B, lay.extra_words, _ptr(tokens), _ptr(lens), _ptr(starts), _ptr(slots),
                              _ptr(want), int(want.size), lay.n_groups, lay.max_blocks, ctypes.cast(ptrs, ctypes.c_void_p))


def attention_list_capacity(T: int, B: int) -> (int, int):
    """Words that the attention's two work lists need for a step of T rows and B requests: (short rows, tiles)."""
    h = lib()
    return h.jk_attention_short_rows_capacity(T), h.jk_attention_tiles_capacity(T, B)


def attention_work_lists(B: int, pad_B: int, lens, starts, short_rows: np.ndarray, tiles: np.ndarray) -> (int, int):
    """Fill the attention's work lists for a batch (``jk::attention_work_lists``); returns (short rows, tiles)."""
    lens, starts = _i32(lens), _i32(starts)
    counts = (ctypes.c_int * 2)()
    lib().jk_attention_work_lists(B, pad_B, _ptr(lens), _ptr(starts), short_rows.ctypes.data, tiles.ctypes.data, counts)
    return counts[0], counts[1]


# ---- attention cuts, product routes ----------------------------------------------------------------------------------
def decode_splits(nrows: int, nkvh: int, group: int, context: int, window: int, sms: int, dh: int) -> int:
    """How many ways the decode attention cuts each row's keys in a step planned for ``context`` positions."""
    h = lib()
    return h.jk_decode_splits(nrows, nkvh, group, h.jk_decode_keys_hint(context, window or 0), sms, dh)


def decode_scratch_floats(nrows: int, nh: int, dh: int, splits: int) -> int:
    return lib().jk_decode_scratch_floats(nrows, nh, dh, splits)


def context_bucket(longest: int, max_positions: int) -> int:
    return lib().jk_context_bucket(longest, max_positions)


def attention_tcgen05_takes(dh: int, page_size: int) -> bool:
    return bool(lib().jk_attention_tcgen05_takes(dh, page_size))


ROUTE_LIBRARY, ROUTE_SMALL, ROUTE_SKINNY, ROUTE_TCGEN05 = 0, 1, 2, 3
PRODUCT_F32, PRODUCT_RESIDUAL, PRODUCT_SWIGLU = 0, 1, 2


def product_route(routing: Sequence[int], rows: int, n: int, k: int, kind: int, small_ok: bool = True, tcgen05_ok: bool = True) -> int:
    """``routing``: (sms, tcgen05_min_rows, tcgen05_min_tiles, tcgen05_min_fill_pct, skinny_min_blocks, library_only)."""
    arr = (ctypes.c_int * 6)(*[int(v) for v in routing])
    return lib().jk_product_route(arr, rows, n, k, kind, int(small_ok), int(tcgen05_ok))


# ---- tables and uniforms -----------------------------------------------------------------------------------------------
def rotary_tables(theta: float, half: int, positions: int, angle_scale: float = 1.0):
    """(cos, sin) float32 ``[positions, half]``: angle of pair j at position p = angle_scale * p / theta^(j / half),
    computed in float64 and rounded once."""
    cos = np.empty((positions, half), dtype=np.float32)
    sin = np.empty((positions, half), dtype=np.float32)
    lib().jk_rotary_tables(float(theta), half, positions, float(angle_scale), cos.ctypes.data, sin.ctypes.data)
    return cos, sin


def uniform_for(seed: int, index: int) -> float:
    """A float in [0, 1) from (seed, index): the splitmix64 finaliser, top 24 bits."""
    return float(lib().jk_uniform_for(int(seed) & ((1 << 64) - 1), int(index) & ((1 << 64) - 1)))


# ---- the page pool -----------------------------------------------------------------------------------------------------
class NativePagePool:
    """Handle on a ``jk::PagePool``."""

    def __init__(self, num_pages: int, reserved: int):
        self._h = lib().jk_pool_create(num_pages, reserved)
        if not self._h:
            raise ValueError(f"a pool of {num_pages} pages with {reserved} reserved holds nothing")

    def __del__(self):
        try:
            if self._h:
                lib().jk_pool_destroy(self._h)
                self._h = None
        except Exception:       # noqa: BLE001 - interpreter shutdown
            pass

    def available(self) -> int:
        return lib().jk_pool_available(self._h)

    def high_water(self) -> int:
        return lib().jk_pool_high_water(self._h)

    def alloc(self, n: int) -> Optional[List[int]]:
        out = (ctypes.c_int * max(1, n))()
        if lib().jk_pool_alloc(self._h, n, out):
            return None
        return list(out[:n])

    def free(self, pages: Sequence[int]) -> int:
        arr = (ctypes.c_int * max(1, len(pages)))(*pages)
        return lib().jk_pool_free(self._h, arr, len(pages))

    def is_held(self, page: int) -> bool:
        return bool(lib().jk_pool_is_held(self._h, page))
