"""The standard decoder stack run from native code: one call per step instead of a dozen per layer.

``NativeRunner`` hands the kernel modules' entry points and the model's weights, tables and cache pages to
``csrc/runner.cu`` once, and per step fills one small struct with the step's device arrays.  The native
function launches the same kernels, with the same routing, as ``Model.forward`` over the parts does; it is a
faster way to issue them (a step of a 52-layer model costs the host about half a millisecond instead of
nine), not another implementation of the model.  It takes a model only if every layer is the standard
arrangement (pre-norm block, rotary attention without bias, SwiGLU, RMSNorm) in bfloat16 with the default
run order; anything else (toy parts, float32, sizes the small-row kernels refuse) runs through the parts.

(The reference's counterpart is the per-device worker thread that runs ``inferDeviceBatch``,
src/models/jiuge/jiuge.cpp:126-305, fed through ``inferBatch``: :307-330.)
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import kernels
from ..kernels import build as _build
from ..parts import StepContext


class _Fns(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "embed", "add_rmsnorm", "swiglu", "rope_kv", "linear_small", "linear_small_qkv", "gemm_tcgen05",
        "gemm_tcgen05_qkv", "attention_decode", "attention_prefill", "attention_tcgen05",
        "err_elementwise", "err_linear_small", "err_gemm_tcgen05", "err_attention", "err_attention_tcgen05",
        "linear_small_supports", "linear_small_qkv_supports", "gemm_skinny",
        "linear_small_norm_supports", "linear_small_norm", "linear_small_qkv_norm", "argmax", "sample", "err_sampling")]


class _Model(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int) for n in (
        "layers", "hidden", "heads", "kv_heads", "head_dim", "intermediate", "vocab",
        "page_size", "max_blocks", "num_pages", "window",
        "sms", "tcgen05_min_rows", "tcgen05_min_tiles", "tcgen05_min_fill_pct", "skinny_min_blocks", "fused_norms", "attention_tcgen05", "embed_dtype")]
                + [(n, ctypes.c_float) for n in ("embed_scale", "residual_scale", "logit_scale", "softmax_scale", "final_eps")]
                + [(n, ctypes.c_void_p) for n in ("embedding", "lm_head", "final_norm", "cos_table", "sin_table", "status")])


class _Layer(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("w_qkv", "w_o", "w_gate_up", "w_down", "norm1", "norm2")]
                + [("eps1", ctypes.c_float), ("eps2", ctypes.c_float)]
                + [("k_pages", ctypes.c_void_p), ("v_pages", ctypes.c_void_p)])


class _Step(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int) for n in ("ntok", "nreq", "n_want", "n_tiles", "n_short", "splits")]
                + [(n, ctypes.c_void_p) for n in ("tokens", "positions", "row_req", "req_start", "req_pos", "want_rows",
                                                  "short_rows", "tiles", "block_table", "logits")])


class _Scratch(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("x", "h", "qkv", "q", "o", "delta", "gate_up", "act", "hw",
                                                "decode_scratch", "workspace")]
                + [("workspace_bytes", ctypes.c_longlong), ("sumsq", ctypes.c_void_p)])


def _addr(lib, name: str) -> int:
    return ctypes.cast(getattr(lib, name), ctypes.c_void_p).value


class NativeRunner:
    """See the module's docstring.  ``NativeRunner.build(engine)`` returns a runner or None (with the reason
    in ``NativeRunner.why_not``)."""

    why_not: str = ""

    @classmethod
    def build(cls, engine) -> Optional["NativeRunner"]:
        reason = cls._ineligible(engine)
        if reason:
            cls.why_not = reason
            return None
        return cls(engine)

    @staticmethod
    def _ineligible(engine) -> str:
        from ..parts.attention import Attention
        from ..parts.block import PreNormBlock
        from ..parts.feed_forward import SwiGLU
        from ..parts.norm import RMSNorm
        from ..parts.rope import RotaryTables
        rt, model, spec = engine.runtime, engine.model, engine.spec
        if rt.dtype != torch.bfloat16:
            return "the native runner is built for bfloat16"
        if rt.plain_attention or rt.library_products_only or rt.legacy_tensor_cores:
            return "a runtime switch asks for another kernel"
        if len(engine.cache.groups) != 1 or engine.cache.dtype != torch.bfloat16:
            return "more than one cache group"
        for i, e in enumerate(spec.order):
            if (e.layer, e.cache, e.writes_cache) != (i, i, True):
                return "the run order is not one pass over the layers"
        if len(spec.order) != len(model.layers):
            return "the run order is not one pass over the layers"
        first = model.layers[0]
        for blk in model.layers:
            if type(blk) is not PreNormBlock or type(blk.mixer) is not Attention or type(blk.feed_forward) is not SwiGLU \
                    or type(blk.mixer_norm) is not RMSNorm or type(blk.ffn_norm) is not RMSNorm:
                return "a layer is not the standard arrangement"
            a, a0 = blk.mixer, first.mixer
            if a.b_qkv is not None:
                return "attention has a bias"
            if a.position is not None and (type(a.position) is not RotaryTables or a.position.interleaved):
                return "the position encoding is not rotate-half rotary"
            if (a.position is None) != (a0.position is None):
                return "layers differ in their position encoding"
            same = ("num_heads", "num_kv_heads", "head_dim", "softmax_scale", "window")
            if any(getattr(a.spec, k) != getattr(a0.spec, k) for k in same) or blk.spec.residual_scale != first.spec.residual_scale:
                return "layers differ in their sizes"
            if a.position is not None and (a.position.cos.data_ptr() != a0.position.cos.data_ptr()
                                           and not torch.equal(a.position.cos, a0.position.cos)):
                return "layers differ in their rotary tables"
        if type(model.final_norm) is not RMSNorm:
            return "the final norm is not RMSNorm"
        s = first.mixer.spec
        d, di, dh = spec.hidden_size, first.feed_forward.spec.intermediate_size, s.head_dim
        page = engine.cache.page_size
        if not (dh % 8 == 0 and dh <= 256 and (kernels.attention_prefill_supports(dh)
                                               or kernels.attention_tcgen05_supports(dh, page))):
            return "no tensor-core attention kernel for this head size"
        nq = (s.num_heads + 2 * s.num_kv_heads) * dh
        small = [(nq, d), (d, s.num_heads * dh), (di, d), (d, di), (spec.vocab_size, d)]
        # every product of few rows has a home: the small-row kernels, or (K too long for their shared memory)
        # the few-rows tcgen05 kernel
        if any(k % 32 for _, k in small) or dh % 16 \
                or not all(kernels.linear_small_supports(16, n, k) or kernels.gemm_skinny_supports(16, n, k) for n, k in small) \
                or not kernels.linear_small_qkv_supports(16, d, dh):
            return "a product is outside what the small-row kernels take"
        if model.embedding.dtype != torch.bfloat16 or model.lm_head.dtype != torch.bfloat16:
            return "the embedding is not bfloat16"
        return ""

    def __init__(self, engine):
        # no reference back to the engine: a cycle would leave the engine (and the CUDA graphs it holds) to
        # the cyclic collector, which may then destroy those graphs in the middle of another capture
        rt, model, spec, cache = engine.runtime, engine.model, engine.spec, engine.cache
        self.runtime, self.max_step_tokens, self.vocab_size = rt, engine.max_step_tokens, spec.vocab_size
        dev = rt.device
        self.lib = _build.load("runner")
        self.lib.jk_runner_last_error.restype = ctypes.c_char_p
        first = model.layers[0]
        a = first.mixer.spec
        d, di, dh = spec.hidden_size, first.feed_forward.spec.intermediate_size, a.head_dim
        nq = (a.num_heads + 2 * a.num_kv_heads) * dh
        self._products = [(nq, d, "f32"), (d, a.num_heads * dh, "residual"), (di, d, "swiglu"), (d, di, "residual"),
                          (spec.vocab_size, d, "f32")]
        self._attention_tcgen05 = kernels.attention_tcgen05_supports(dh, cache.page_size)
        self._bound_tcgen05 = None
        self._bind()
        self.dims = (d, di, a.num_heads, a.num_kv_heads, dh)
        pos = first.mixer.position
        k0 = cache.views[0].k_pages
        self._model = _Model(
            layers=len(model.layers), hidden=d, heads=a.num_heads, kv_heads=a.num_kv_heads, head_dim=dh, intermediate=di,
            vocab=spec.vocab_size, page_size=cache.page_size, max_blocks=cache.max_blocks, num_pages=k0.shape[0],
            window=a.window or 0, sms=kernels._sm_count(dev), tcgen05_min_rows=rt.tcgen05_min_rows,
            tcgen05_min_tiles=rt.tcgen05_min_tiles, tcgen05_min_fill_pct=rt.tcgen05_min_fill_pct,
            skinny_min_blocks=rt.skinny_min_blocks or 0,
            fused_norms=1 if rt.fused_norms else 0,
            attention_tcgen05=1 if self._attention_tcgen05 else 0,
            embed_dtype=kernels.dtype_code(model.embedding.dtype), embed_scale=spec.embed_scale,
            residual_scale=first.spec.residual_scale, logit_scale=spec.logit_scale, softmax_scale=a.softmax_scale,
            final_eps=model.final_norm.spec.eps, embedding=model.embedding.data_ptr(), lm_head=model.lm_head.data_ptr(),
            final_norm=model.final_norm.weight.data_ptr(), cos_table=pos.cos.data_ptr() if pos else 0,
            sin_table=pos.sin.data_ptr() if pos else 0, status=kernels.gemm_status(dev).data_ptr())
        self._routing = (rt.tcgen05_min_rows, rt.tcgen05_min_tiles, rt.tcgen05_min_fill_pct, rt.skinny_min_blocks, rt.fused_norms)
        self._layers = (_Layer * len(model.layers))()
        for i, blk in enumerate(model.layers):
            view = cache.views[spec.order[i].cache]
            self._layers[i] = _Layer(
                w_qkv=blk.mixer.w_qkv.data_ptr(), w_o=blk.mixer.w_o.data_ptr(), w_gate_up=blk.feed_forward.w_gate_up.data_ptr(),
                w_down=blk.feed_forward.w_down.data_ptr(), norm1=blk.mixer_norm.weight.data_ptr(),
                norm2=blk.ffn_norm.weight.data_ptr(), eps1=blk.mixer_norm.spec.eps, eps2=blk.ffn_norm.spec.eps,
                k_pages=view.k_pages.data_ptr(), v_pages=view.v_pages.data_ptr())
        T = engine.max_step_tokens
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        b16 = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device=dev)
        self._buffers = dict(x=f32(T, d), h=b16(T, d), qkv=f32(T, nq), q=b16(T, a.num_heads * dh), o=b16(T, a.num_heads * dh),
                             delta=f32(T, d), gate_up=f32(T, 2 * di), act=b16(T, di), hw=b16(T, d),
                             workspace=torch.empty(32 << 20, dtype=torch.uint8, device=dev))
        self._max_positions = a.position.max_positions if a.position else 1 << 20
        # The split-key attention's scratch, sized once for the worst step: captured decode steps keep its address,
        # so it must never move (rows x heads x splits x (head size + 2) floats; more rows mean fewer splits).
        sms, worst = kernels._sm_count(dev), 1
        for rows in range(1, T + 1):
            splits = kernels.attention_decode_splits(rows, a.num_kv_heads, a.num_heads // a.num_kv_heads,
                                                     a.window or self._max_positions, sms, dh)
            if splits > 1:
                worst = max(worst, rows * a.num_heads * splits * (dh + 2))
        self._decode_scratch = f32(worst)
        self._sumsq = torch.zeros(2 * len(model.layers), 16, dtype=torch.int64, device=dev)
        self._scratch = _Scratch(workspace_bytes=32 << 20, decode_scratch=self._decode_scratch.data_ptr(),
                                 sumsq=self._sumsq.data_ptr(),
                                 **{k: v.data_ptr() for k, v in self._buffers.items()})
        self.launches = 0

    def _bind(self) -> None:
        """Hand the kernel modules' entry points to the native side.  The tcgen05 product is bound (and so
        compiled) only if a step of this engine can reach it under the runtime's routing, the tcgen05
        attention only for the head and page sizes it is built for."""
        rt = self.runtime
        rows = self.max_step_tokens
        need_tc = any(rt.takes_tcgen05(rows, n, k)
                      or "skinny" in (rt.few_rows_route(min(16, rows), n, k, kind), rt.few_rows_route(min(128, rows), n, k, kind))
                      for n, k, kind in self._products)
        if self._bound_tcgen05 is not None and (self._bound_tcgen05 or not need_tc):
            return
        names = ["elementwise", "linear_small", "attention", "sampling"] + (["gemm_tcgen05"] if need_tc else []) \
            + (["attention_tcgen05"] if self._attention_tcgen05 else [])
        mods = {m: _build.load(m) for m in names}
        get = lambda module, name: _addr(mods[module], name) if module in mods else None
        fns = _Fns(
            embed=get("elementwise", "jk_embed"), add_rmsnorm=get("elementwise", "jk_add_rmsnorm"),
            swiglu=get("elementwise", "jk_swiglu"), rope_kv=get("elementwise", "jk_rope_kv"),
            linear_small=get("linear_small", "jk_linear_small"), linear_small_qkv=get("linear_small", "jk_linear_small_qkv"),
            gemm_tcgen05=get("gemm_tcgen05", "jk_gemm_tcgen05"), gemm_tcgen05_qkv=get("gemm_tcgen05", "jk_gemm_tcgen05_qkv"),
            gemm_skinny=get("gemm_tcgen05", "jk_gemm_skinny"),
            linear_small_supports=get("linear_small", "jk_linear_small_supports"),
            linear_small_qkv_supports=get("linear_small", "jk_linear_small_qkv_supports"),
            linear_small_norm_supports=get("linear_small", "jk_linear_small_norm_supports"),
            linear_small_norm=get("linear_small", "jk_linear_small_norm"),
            linear_small_qkv_norm=get("linear_small", "jk_linear_small_qkv_norm"),
            attention_decode=get("attention", "jk_attention_decode"), attention_prefill=get("attention", "jk_attention_prefill"),
            attention_tcgen05=get("attention_tcgen05", "jk_attention_tcgen05"),
            err_elementwise=get("elementwise", "jk_elementwise_last_error"),
            err_linear_small=get("linear_small", "jk_linear_small_last_error"),
            err_gemm_tcgen05=get("gemm_tcgen05", "jk_gemm_tcgen05_last_error"),
            err_attention=get("attention", "jk_attention_last_error"),
            err_attention_tcgen05=get("attention_tcgen05", "jk_attention_tcgen05_last_error"),
            # the C interface of the same library (csrc/model_api.h) samples through these
            argmax=get("sampling", "jk_argmax"), sample=get("sampling", "jk_sample"),
            err_sampling=get("sampling", "jk_sampling_last_error"))
        self._check(self.lib.jk_runner_bind(ctypes.byref(fns)))
        self._bound_tcgen05 = need_tc

    def _check(self, rc: int) -> None:
        if rc:
            raise kernels.KernelError(self.lib.jk_runner_last_error().decode(errors="replace") or f"the native runner returned {rc}")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Logits (float32 ``[n_want, vocab]``) of the step that ``ctx`` describes."""
        rt = self.runtime
        now = (rt.tcgen05_min_rows, rt.tcgen05_min_tiles, rt.tcgen05_min_fill_pct, rt.skinny_min_blocks, rt.fused_norms)
        if now != self._routing:       # a test moved the thresholds
            self._routing = now
            self._model.tcgen05_min_fill_pct = rt.tcgen05_min_fill_pct
            self._model.fused_norms = 1 if rt.fused_norms else 0
            self._model.tcgen05_min_rows, self._model.tcgen05_min_tiles = rt.tcgen05_min_rows, rt.tcgen05_min_tiles
            self._model.skinny_min_blocks = rt.skinny_min_blocks or 0
            self._bind()
        d, di, nh, nkvh, dh = self.dims
        T = ctx.ntok
        if T > self.max_step_tokens:
            raise kernels.KernelError(f"the native runner holds buffers for {self.max_step_tokens} rows, the step has {T}")
        splits = 1
        if ctx.n_short:
            splits = kernels.attention_decode_splits(ctx.n_short, nkvh, nh // nkvh, self._model.window or self._max_positions,
                                                     kernels._sm_count(rt.device), dh)
            if splits > 1 and ctx.n_short * nh * splits * (dh + 2) > self._decode_scratch.numel():
                raise kernels.KernelError("the split-key attention needs more scratch than was sized for the largest step")
        n_want = ctx.want_rows.numel()
        logits = torch.empty(n_want, self.vocab_size, dtype=torch.float32, device=rt.device)
        table = ctx.block_tables[0]
        step = _Step(ntok=T, nreq=ctx.nreq, n_want=n_want, n_tiles=ctx.n_tiles, n_short=ctx.n_short, splits=splits,
                     tokens=ctx.tokens.data_ptr(), positions=ctx.positions.data_ptr(), row_req=ctx.row_req.data_ptr(),
                     req_start=ctx.req_start.data_ptr(), req_pos=ctx.req_pos.data_ptr(), want_rows=ctx.want_rows.data_ptr(),
                     short_rows=ctx.short_rows.data_ptr() if ctx.short_rows is not None else 0,
                     tiles=ctx.tiles.data_ptr() if ctx.tiles is not None and ctx.n_tiles else 0,
                     block_table=table.data_ptr(), logits=logits.data_ptr())
        self._check(self.lib.jk_runner_forward(ctypes.byref(self._model), self._layers, ctypes.byref(step),
                                               ctypes.byref(self._scratch), kernels._stream()))
        self.launches = self.lib.jk_runner_launches()
        return logits
