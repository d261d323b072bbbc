"""Python bindings of the CUDA kernels in ``csrc``: one thin function per exported symbol.

Arguments are CUDA tensors; each binding checks types, shapes and contiguity, passes raw
device pointers and the current stream to the C function, and raises ``KernelError`` with
the library's message if it returns non-zero.  There is no fallback path: without the
compiled module a call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build
from . import host as _host

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


launch_count = 0      # kernels of this package launched through these bindings (captured ones count once)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # the raw handle of the current stream of the current device (a Stream object costs microseconds
    # to build, and every launch asks)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _check(module: str, rc: int):
    global launch_count
    launch_count += 1
    if rc:
        lib = _build.load(module)
        fn = getattr(lib, f"jk_{module}_last_error")
        fn.restype = ctypes.c_char_p
        raise KernelError(fn().decode(errors="replace") or f"kernel module {module} returned {rc}")


_c_int, _c_float, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
    """out[i, :] = scale * table[tokens[i], :], float32."""
    _need(tokens, "tokens", torch.int32); _need(table, "table"); _need(out, "out", torch.float32)
    n, d = tokens.numel(), table.shape[1]
    if out.shape[-1] != d or out.numel() < n * d:
        raise KernelError(f"embed: out {tuple(out.shape)} does not hold {n} rows of {d}")
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_embed(_ptr(tokens), _c_int(n), _ptr(table), _c_int(dtype_code(table.dtype)),
                                       _c_int(d), _c_float(scale), _ptr(out), _stream()))
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], delta_scale: float, weight: torch.Tensor,
                eps: float, out: torch.Tensor, out_scale: float = 1.0,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += delta_scale * delta (when rows is None); out = out_scale * rmsnorm(x[rows]) * weight."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    d = x.shape[-1]
    if weight.numel() != d or out.shape[-1] != d:
        raise KernelError(f"add_rmsnorm: width {d}, weight {weight.numel()}, out {out.shape[-1]}")
    if delta is not None:
        _need(delta, "delta")
        if delta.shape != x.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        nout = rows.numel()
    else:
        nout = x.numel() // d
    if out.numel() < nout * d:
        raise KernelError("add_rmsnorm: out is too small")
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_add_rmsnorm(
        _ptr(x), _ptr(delta), _c_int(dtype_code(delta.dtype) if delta is not None else F32),
        _c_float(delta_scale), _ptr(weight), _c_float(eps), _c_float(out_scale), _ptr(out),
        _c_int(dtype_code(out.dtype)), _ptr(rows), _c_int(nout), _c_int(d), _stream()))
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor, delta_scale: float) -> torch.Tensor:
    _need(x, "x", torch.float32); _need(delta, "delta")
    if delta.numel() != x.numel():
        raise KernelError("residual_add: sizes differ")
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_residual_add(_ptr(x), _ptr(delta), _c_int(dtype_code(delta.dtype)),
                                              _c_float(delta_scale), _c_ll(x.numel()), _stream()))
    return x


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, di + c]."""
    _need(gate_up, "gate_up"); _need(out, "out")
    ntok, di = out.shape
    if gate_up.shape != (ntok, 2 * di):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_swiglu(_ptr(gate_up), _c_int(dtype_code(gate_up.dtype)), _ptr(out),
                                        _c_int(dtype_code(out.dtype)), _c_int(ntok), _c_int(di), _stream()))
    return out


def rope_kv(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor, row_req: torch.Tensor,
            block_table: Optional[torch.Tensor], page_size: int, cos: Optional[torch.Tensor],
            sin: Optional[torch.Tensor], interleaved: bool, q_out: torch.Tensor,
            k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], ntok: int, nh: int, nkvh: int,
            dh: int, write_cache: bool = True) -> None:
    """Rotate query and key heads of ``qkv`` rows; write keys and values into their pages."""
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32); _need(row_req, "row_req", torch.int32)
    _need(q_out, "q_out")
    width = (nh + 2 * nkvh) * dh
    if qkv.shape[-1] != width or qkv.shape[0] < ntok:
        raise KernelError(f"rope_kv: qkv {tuple(qkv.shape)} does not hold {ntok} rows of {width}")
    if q_out.numel() < ntok * nh * dh:
        raise KernelError("rope_kv: q_out is too small")
    max_blocks = 0
    if write_cache:
        _need(block_table, "block_table", torch.int32); _need(k_pages, "k_pages"); _need(v_pages, "v_pages")
        if k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype:
            raise KernelError("rope_kv: pages and q_out must have one type")
        if tuple(k_pages.shape[1:]) != (nkvh, page_size, dh) or k_pages.shape != v_pages.shape:
            raise KernelError(f"rope_kv: pages {tuple(k_pages.shape)} are not [*, {nkvh}, {page_size}, {dh}]")
        max_blocks = block_table.shape[1]
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32)
        if cos.shape[1] != dh // 2 or sin.shape != cos.shape:
            raise KernelError("rope_kv: cos/sin tables must be [positions, head_dim/2]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_rope_kv(
        _ptr(qkv), _c_int(dtype_code(qkv.dtype)), _c_int(width), _ptr(bias), _ptr(positions), _ptr(row_req),
        _ptr(block_table), _c_int(max_blocks), _c_int(page_size), _ptr(cos), _ptr(sin),
        _c_int(1 if interleaved else 0), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
        _c_int(dtype_code(q_out.dtype)), _c_int(ntok), _c_int(nh), _c_int(nkvh), _c_int(dh),
        _c_int(1 if write_cache else 0), _stream()))


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) in float32 on the CUDA cores (no TF32)."""
    _need(a, "a", torch.float32); _need(w, "w", torch.float32); _need(out, "out", torch.float32)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise KernelError(f"gemm_f32: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    lib = _build.load("elementwise")
    _check("elementwise", lib.jk_gemm_f32(_ptr(a), _c_int(k), _ptr(w), _c_int(k), _ptr(bias), _ptr(out),
                                          _c_int(n), _c_int(m), _c_int(n), _c_int(k), _stream()))
    return out


EPI_F32, EPI_SWIGLU, EPI_RESIDUAL = 0, 1, 3


def linear_small_supports(m: int, n: int, k: int) -> bool:
    """Whether the weight-streaming kernel for steps of few rows takes this product."""
    return bool(_build.load("linear_small").jk_linear_small_supports(_c_int(m), _c_int(n), _c_int(k)))


def linear_small(act: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_F32) -> torch.Tensor:
    """out = act @ w^T for at most 16 rows of bfloat16 activations.  EPI_F32: float32 out [M, N].
    EPI_SWIGLU: w is [2N, K] (gate rows, then up rows) and out is bfloat16 [M, N] = silu(gate) * up."""
    _need(act, "act", torch.bfloat16); _need(w, "w", torch.bfloat16)
    _need(out, "out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
    m, k = act.shape
    n = w.shape[0] // (2 if epilogue == EPI_SWIGLU else 1)
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise KernelError(f"linear_small: act {tuple(act.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lib = _build.load("linear_small")
    _check("linear_small", lib.jk_linear_small(_ptr(act), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k),
                                               _c_int(out.stride(0)), _c_int(epilogue), _c_int(_sm_count(act.device)),
                                               _stream()))
    return out


def linear_small_qkv_supports(m: int, k: int, dh: int) -> bool:
    """Whether the small-row product can take the fused [q | k | v] projection with rotation and cache
    write in its epilogue."""
    return bool(_build.load("linear_small").jk_linear_small_qkv_supports(_c_int(m), _c_int(k), _c_int(dh)))


def linear_small_qkv(act: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor,
                     v_pages: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor, nh: int) -> torch.Tensor:
    """The fused [q | k | v] projection of at most 16 bfloat16 rows: query and key heads rotated
    (rotate-half), queries to ``q_out``, keys and values into their pages, all from the epilogue."""
    _check_qkv_args("linear_small_qkv", act, w, q_out, k_pages, v_pages, cos, sin, positions, row_req, block_table, nh)
    m, k = act.shape
    _, nkvh, page_size, dh = k_pages.shape
    lib = _build.load("linear_small")
    _check("linear_small", lib.jk_linear_small_qkv(
        _ptr(act), _ptr(w), _c_int(m), _c_int(k), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(cos), _ptr(sin),
        _ptr(positions), _ptr(row_req), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size), _c_int(nh),
        _c_int(nkvh), _c_int(dh), _c_int(_sm_count(act.device)), _stream()))
    return q_out


SUMSQ_FIXED = float(1 << 26)      # the fixed-point scale of the row sums of squares (csrc/linear_small.cu)


def linear_small_norm_supports(m: int, n: int, k: int) -> bool:
    """Whether the products of a chain without norm kernels take this shape (the tile kernel's reach)."""
    return bool(_build.load("linear_small").jk_linear_small_norm_supports(_c_int(m), _c_int(n), _c_int(k)))


def linear_small_norm(act: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_F32,
                      in_sumsq: Optional[torch.Tensor] = None, in_eps: float = 0.0, xb: Optional[torch.Tensor] = None,
                      next_w: Optional[torch.Tensor] = None, out_sumsq: Optional[torch.Tensor] = None,
                      scale: float = 1.0) -> torch.Tensor:
    """A few-row product of a chain in which RMSNorm has no kernel of its own.  With ``in_sumsq`` (int64 [M],
    fixed point: sum of squares times ``SUMSQ_FIXED``) the activations are x * norm weight without the 1 / rms,
    which the rows of the product get before the epilogue (EPI_F32 or EPI_SWIGLU).  ``EPI_RESIDUAL``: ``out`` is
    the float32 residual stream, ``out += scale * product``; ``xb`` receives bfloat16(out * next_w) and
    ``out_sumsq`` (zeroed by the caller) this product's sums of squares of the new rows."""
    _need(act, "act", torch.bfloat16); _need(w, "w", torch.bfloat16)
    _need(out, "out", torch.bfloat16 if epilogue == EPI_SWIGLU else torch.float32)
    m, k = act.shape
    n = w.shape[0] // (2 if epilogue == EPI_SWIGLU else 1)
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise KernelError(f"linear_small_norm: act {tuple(act.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    for name, t, dt in (("in_sumsq", in_sumsq, torch.int64), ("out_sumsq", out_sumsq, torch.int64), ("xb", xb, torch.bfloat16),
                        ("next_w", next_w, torch.float32)):
        if t is not None:
            _need(t, name, dt)
    if (in_sumsq is not None and in_sumsq.numel() < m) or (out_sumsq is not None and out_sumsq.numel() < m) \
            or (xb is not None and tuple(xb.shape) != (m, n)) or (next_w is not None and next_w.numel() != n):
        raise KernelError("linear_small_norm: a norm array has the wrong size")
    lib = _build.load("linear_small")
    _check("linear_small", lib.jk_linear_small_norm(
        _ptr(act), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k), _c_int(out.stride(0)), _c_int(epilogue),
        _ptr(in_sumsq), _c_float(in_eps), _ptr(xb), _ptr(next_w), _ptr(out_sumsq), _c_float(scale),
        _ptr(gemm_status(act.device)), _c_int(_sm_count(act.device)), _stream()))
    return out


def linear_small_qkv_norm(act: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor,
                          v_pages: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                          positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor, nh: int,
                          in_sumsq: torch.Tensor, in_eps: float) -> torch.Tensor:
    """``linear_small_qkv`` for activations that came without their norm's 1 / rms (see ``linear_small_norm``)."""
    _check_qkv_args("linear_small_qkv_norm", act, w, q_out, k_pages, v_pages, cos, sin, positions, row_req, block_table, nh)
    _need(in_sumsq, "in_sumsq", torch.int64)
    m, k = act.shape
    _, nkvh, page_size, dh = k_pages.shape
    lib = _build.load("linear_small")
    _check("linear_small", lib.jk_linear_small_qkv_norm(
        _ptr(act), _ptr(w), _c_int(m), _c_int(k), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(cos), _ptr(sin),
        _ptr(positions), _ptr(row_req), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size), _c_int(nh),
        _c_int(nkvh), _c_int(dh), _ptr(in_sumsq), _c_float(in_eps), _c_int(_sm_count(act.device)), _stream()))
    return q_out


def _check_qkv_args(what, act, w, q_out, k_pages, v_pages, cos, sin, positions, row_req, block_table, nh) -> None:
    for name, t in (("act", act), ("w", w), ("q_out", q_out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _need(t, name, torch.bfloat16)
    for name, t in (("positions", positions), ("row_req", row_req), ("block_table", block_table)):
        _need(t, name, torch.int32)
    m, k = act.shape
    _, nkvh, page_size, dh = k_pages.shape
    if w.shape != ((nh + 2 * nkvh) * dh, k) or q_out.numel() < m * nh * dh or v_pages.shape != k_pages.shape:
        raise KernelError(f"{what}: act {tuple(act.shape)}, w {tuple(w.shape)}, pages {tuple(k_pages.shape)}")
    if positions.numel() < m or row_req.numel() < m:
        raise KernelError(f"{what}: positions or row_req hold fewer entries than rows")
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32)
        if cos.shape[1] != dh // 2 or sin.shape != cos.shape:
            raise KernelError(f"{what}: cos/sin tables must be [positions, head_dim/2]")


def gemm_tcgen05_qkv_supports(dh: int) -> bool:
    """Head sizes for which the tcgen05 product can rotate and store [q | k | v] in its epilogue."""
    return dh in (64, 128)


def gemm_tcgen05_qkv(act: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor,
                     v_pages: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor, nh: int) -> torch.Tensor:
    """The fused [q | k | v] projection of bfloat16 rows: ``act @ w^T`` with query and key heads rotated
    (rotate-half; cos/sin ``[positions, dh/2]`` float32 or None), queries written to ``q_out`` and keys and
    values into their pages through ``block_table``, all from the product's epilogue."""
    _check_qkv_args("gemm_tcgen05_qkv", act, w, q_out, k_pages, v_pages, cos, sin, positions, row_req, block_table, nh)
    m, k = act.shape
    _, nkvh, page_size, dh = k_pages.shape
    lib = _build.load("gemm_tcgen05")
    _check("gemm_tcgen05", lib.jk_gemm_tcgen05_qkv(
        _ptr(act), _ptr(w), _c_int(m), _c_int(k), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(cos), _ptr(sin),
        _ptr(positions), _ptr(row_req), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size), _c_int(nh),
        _c_int(nkvh), _c_int(dh), _ptr(gemm_status(act.device)), _c_int(_sm_count(act.device)), _stream()))
    return q_out


TG_F32, TG_BF16, TG_RESIDUAL, TG_SWIGLU = 0, 1, 2, 3
_tg_status = {}


def gemm_status(device) -> torch.Tensor:
    """The word in which a kernel records a wait that ran out (0: none).  It lies in pinned host memory, which the
    device reaches under the same address: a kernel that gives up writes across, and the host reads it without a copy."""
    key = str(device)
    if key not in _tg_status:
        _tg_status[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _tg_status[key]


def check_gemm_status(device) -> None:
    """Wait for the device's work, read the status words; raise if a kernel gave up waiting."""
    torch.cuda.synchronize(device)
    small = _build._loaded.get("linear_small")
    if small is not None:
        fault = small.jk_linear_small_take_fault()
        if fault > 0:
            raise KernelError(f"linear_small: a bounded wait for a tile of weights ran out or shared memory was misaligned "
                              f"(code {fault}); the step's results are not valid")
    key = str(device)
    if key in _tg_status:
        code = int(_tg_status[key].item())
        if code:
            _tg_status[key].zero_()
            if code == 4:
                raise KernelError("linear_small: a row's sum of squares is beyond the range of the fixed-point counters "
                                  "(activations of several thousand on average); the step's results are not valid; "
                                  "JK_NO_FUSED_NORM=1 keeps the norm kernels, which have no such limit")
            raise KernelError(f"gemm_tcgen05: a bounded wait ran out (role {code}: 1 TMA, 2 MMA, 3 epilogue); "
                              "the step's results are not valid")


def gemm_tcgen05_supports(m: int, n: int, k: int) -> bool:
    """K must keep rows 16-byte aligned for TMA; everything else is free (the same rule as the library's
    ``jk_gemm_tcgen05_supports``; answered here so that asking does not compile the module)."""
    return m >= 1 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_tcgen05_pairs(mode: int) -> int:
    """Which products run on pairs of blocks (clusters of two sharing one 256 x 256 tile, ``cta_group::2``):
    0 none, 1 those whose tiles make more than one wave (the default), 2 all of more than 128 rows.  Returns
    the mode before (-1: the environment's or the default had not been read yet)."""
    return _build.load("gemm_tcgen05").jk_gemm_tcgen05_set_pairs(ctypes.c_int(mode))


def gemm_tcgen05(act: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = TG_F32,
                 scale: float = 1.0) -> torch.Tensor:
    """out (op)= act @ w^T on the tcgen05 tensor cores, operands by TMA.  Epilogues: TG_F32 / TG_BF16 store,
    TG_RESIDUAL ``out += scale * product`` (float32, in place), TG_SWIGLU ``w`` is [2N, K] (gate rows, up rows)
    and ``out`` is bfloat16 [M, N] = silu(gate) * up."""
    _need(act, "act", torch.bfloat16); _need(w, "w", torch.bfloat16)
    _need(out, "out", torch.bfloat16 if epilogue in (TG_BF16, TG_SWIGLU) else torch.float32, contiguous=False)
    m, k = act.shape
    n = w.shape[0] // (2 if epilogue == TG_SWIGLU else 1)
    if w.shape[1] != k or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_tcgen05: act {tuple(act.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lib = _build.load("gemm_tcgen05")
    _check("gemm_tcgen05", lib.jk_gemm_tcgen05(_ptr(act), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k),
                                               _c_int(out.stride(0)), _c_int(epilogue), _c_float(scale),
                                               _ptr(gemm_status(act.device)), _c_int(_sm_count(act.device)), _stream()))
    return out


def gemm_skinny_supports(m: int, n: int, k: int) -> bool:
    """Up to 128 activation rows; K must keep rows 16-byte aligned for TMA."""
    return 1 <= m <= 128 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_skinny(act: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = TG_F32, scale: float = 1.0) -> torch.Tensor:
    """The product of few activation rows (decode batches, short portions) on the tcgen05 tensor cores with the
    weights on the MMA's M side, so that the kernel streams W once at memory speed: TG_F32 ``out = product``
    (float32), TG_RESIDUAL ``out += scale * product`` (float32, blocks split K and add their partial sums),
    TG_SWIGLU ``w`` is [2N, K] and ``out`` bfloat16 = silu(gate) * up."""
    if epilogue not in (TG_F32, TG_RESIDUAL, TG_SWIGLU):
        raise KernelError(f"gemm_skinny: epilogue {epilogue}")
    _need(act, "act", torch.bfloat16); _need(w, "w", torch.bfloat16)
    _need(out, "out", torch.bfloat16 if epilogue == TG_SWIGLU else torch.float32, contiguous=False)
    m, k = act.shape
    n = w.shape[0] // (2 if epilogue == TG_SWIGLU else 1)
    if w.shape[1] != k or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_skinny: act {tuple(act.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lib = _build.load("gemm_tcgen05")
    _check("gemm_tcgen05", lib.jk_gemm_skinny(_ptr(act), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k),
                                              _c_int(out.stride(0)), _c_int(epilogue), _c_float(scale),
                                              _ptr(gemm_status(act.device)), _c_int(_sm_count(act.device)), _stream()))
    return out


_SMS = {}


def _sm_count(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[key]


def attention_rows(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                   positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor, ntok: int,
                   nh: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of ``ntok`` query rows over the paged cache, one warp per (row, head)."""
    _need(q, "q"); _need(k_pages, "k_pages"); _need(v_pages, "v_pages"); _need(out, "out")
    _need(positions, "positions", torch.int32); _need(row_req, "row_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("attention: q, pages and out must have one type")
    _, nkvh, page_size, dh = k_pages.shape
    if q.numel() < ntok * nh * dh or out.numel() < ntok * nh * dh:
        raise KernelError("attention: q or out is too small")
    lib = _build.load("attention")
    _check("attention", lib.jk_attention_rows(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _c_int(dtype_code(q.dtype)), _ptr(positions),
        _ptr(row_req), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size), _c_int(ntok),
        _c_int(nh), _c_int(nkvh), _c_int(dh), _c_float(scale), _c_int(window or 0), _stream()))
    return out


def attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                     rows: Optional[torch.Tensor], nrows: int, positions: torch.Tensor, row_req: torch.Tensor,
                     block_table: torch.Tensor, nh: int, scale: float, window: int, splits: int,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 attention of rows that bring few queries per request (decoded tokens, short portions):
    the key range of every (row, key/value head) is cut into ``splits`` blocks whose partial results
    a second kernel merges.  ``rows`` lists the rows to work on (None: rows 0..nrows-1)."""
    for name, t in (("q", q), ("k_pages", k_pages), ("v_pages", v_pages), ("out", out)):
        _need(t, name, torch.bfloat16)
    _need(positions, "positions", torch.int32); _need(row_req, "row_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _, nkvh, page_size, dh = k_pages.shape
    lib = _build.load("attention")
    lib.jk_attention_decode_scratch_floats.restype = ctypes.c_longlong
    need = lib.jk_attention_decode_scratch_floats(_c_int(nrows), _c_int(nh), _c_int(dh), _c_int(splits))
    if need and scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if need:
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"attention_decode: scratch holds {scratch.numel()} floats, {need} needed")
    _check("attention", lib.jk_attention_decode(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch if need else None), _ptr(rows), _c_int(nrows),
        _ptr(positions), _ptr(row_req), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size),
        _c_int(nh), _c_int(nkvh), _c_int(dh), _c_float(scale), _c_int(window or 0), _c_int(splits), _stream()))
    if need and splits > 1:
        global launch_count
        launch_count += 1          # the merge kernel
    return out


def attention_prefill_supports(dh: int) -> bool:
    return bool(_build.load("attention").jk_attention_prefill_supports(_c_int(dh)))


TILE_ROWS = _host.attention_tile_rows()      # rows of a query tile in the tile lists that the prefill attention kernels take


def attention_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                      tiles: torch.Tensor, ntiles: int, req_start: torch.Tensor, req_pos: torch.Tensor,
                      block_table: torch.Tensor, nh: int, scale: float, window: int = 0) -> torch.Tensor:
    """bfloat16 tensor-core (mma.sync) attention of requests that bring many rows: ``tiles[i] = (batch
    entry, first row)`` names TILE_ROWS-row tiles of query rows."""
    for name, t in (("q", q), ("k_pages", k_pages), ("v_pages", v_pages), ("out", out)):
        _need(t, name, torch.bfloat16)
    for name, t in (("tiles", tiles), ("req_start", req_start), ("req_pos", req_pos), ("block_table", block_table)):
        _need(t, name, torch.int32)
    _, nkvh, page_size, dh = k_pages.shape
    if tiles.numel() < 2 * ntiles:
        raise KernelError("attention_prefill: the tile list is shorter than ntiles")
    lib = _build.load("attention")
    _check("attention", lib.jk_attention_prefill(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), _c_int(ntiles), _c_int(TILE_ROWS), _ptr(req_start),
        _ptr(req_pos), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(page_size), _c_int(nh), _c_int(nkvh),
        _c_int(dh), _c_float(scale), _c_int(window or 0), _stream()))
    return out


def attention_tcgen05_supports(dh: int, page_size: int) -> bool:
    """Head sizes 64 and 128 with pages that divide a tile of 128 keys and fill whole groups of 8 rows
    (``jk::attention_tcgen05_takes`` of csrc/host_rules.h; asking does not compile the kernel's module)."""
    return _host.attention_tcgen05_takes(dh, page_size)


def attention_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                      tiles: torch.Tensor, ntiles: int, ntok: int, req_start: torch.Tensor, req_pos: torch.Tensor,
                      block_table: torch.Tensor, nh: int, scale: float, window: int = 0) -> torch.Tensor:
    """The same attention of TILE_ROWS-row query tiles on the tcgen05 tensor cores (TMA operands, both
    products with accumulators in tensor memory); head sizes 64 and 128, pages that divide 128."""
    for name, t in (("q", q), ("k_pages", k_pages), ("v_pages", v_pages), ("out", out)):
        _need(t, name, torch.bfloat16)
    for name, t in (("tiles", tiles), ("req_start", req_start), ("req_pos", req_pos), ("block_table", block_table)):
        _need(t, name, torch.int32)
    num_pages, nkvh, page_size, dh = k_pages.shape
    if tiles.numel() < 2 * ntiles or q.numel() < ntok * nh * dh:
        raise KernelError("attention_tcgen05: the tile list or q is too short")
    lib = _build.load("attention_tcgen05")
    _check("attention_tcgen05", lib.jk_attention_tcgen05(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), _c_int(ntiles), _c_int(ntok), _ptr(req_start),
        _ptr(req_pos), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(num_pages), _c_int(page_size), _c_int(nh),
        _c_int(nkvh), _c_int(dh), _c_float(scale), _c_int(window or 0), _ptr(gemm_status(q.device)), _stream()))
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    n, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("argmax: rows must be contiguous")
    lib = _build.load("sampling")
    lib.jk_argmax_scratch_bytes.restype = ctypes.c_longlong
    need = lib.jk_argmax_scratch_bytes(_c_int(n), _c_int(v))
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _check("sampling", lib.jk_argmax(_ptr(logits), _c_ll(logits.stride(0)), _c_int(n), _c_int(v), _ptr(out),
                                     _ptr(scratch), _stream()))
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, topk: torch.Tensor, topp: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(topk, "topk", torch.int32)
    _need(topp, "topp", torch.float32); _need(uniform, "uniform", torch.float32)
    n, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: rows must be contiguous")
    if min(temperature.numel(), topk.numel(), topp.numel(), uniform.numel(), out.numel()) < n:
        raise KernelError("sample: a per-row array is shorter than the number of rows")
    lib = _build.load("sampling")
    _check("sampling", lib.jk_sample(_ptr(logits), _c_ll(logits.stride(0)), _c_int(n), _c_int(v), _ptr(temperature),
                                     _ptr(topk), _ptr(topp), _ptr(uniform), _ptr(out), _stream()))
    return out


def build_all(verbose: bool = True):
    return _build.build_all(verbose)
