"""A model as launch records, and the code that replays them.

Every part says what it does to a step ONCE, when the model is built, by emitting launch records into a ``Program``
(``part.plan(program, ...)``): one record per operation of its layer kind, naming the buffers it reads and writes, its
weights and its constants (``RunnerOp`` of csrc/runner.h).  A step then replays the records with one native call
(``jk_runner_run`` of csrc/runner.cu), which also decides, from the step's size and the precision, which kernel runs
each record.  The records of this architecture's parts are written by emitters on the native side
(``jk_emit_attention`` ...), which the C interface calls as well; a part of another kind may emit any records that say
what it does, or none: a part without ``plan`` is run by its own ``forward`` between two runs of records (a *host
step*), so every model has a program and a part that uses existing operations runs natively without any native code
of its own.

The reference's counterpart is the hand-written layer loop of ``inferDeviceBatch`` (src/models/jiuge/jiuge.cpp:195-258).
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..kernels import build as _build
from ..kernels import host as _host

_i, _f, _p, _ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

SLOTS = ("x", "delta", "h", "q", "o", "act", "hw", "logits", "tmp", "decode")       # RunnerSlot of csrc/runner.h
SLOT = {name: i for i, name in enumerate(SLOTS)}
OP_NAMES = {1: "embed", 2: "norm", 3: "qkv", 4: "attention", 5: "residual", 6: "gate_up", 7: "linear"}
MAX_GROUPS = 8
MAX_LISTS = 8


class RunnerOp(ctypes.Structure):
    _fields_ = ([(n, _i) for n in ("kind", "in_slot", "out_slot", "wanted_rows", "n", "k", "heads", "kv_heads", "head_dim", "window",
                                   "interleaved", "writes_cache", "cache_group", "list_short", "list_tiles", "w_dtype",
                                   "max_positions")]
                + [(n, _f) for n in ("eps", "scale", "softmax_scale")]
                + [(n, _p) for n in ("w", "vec", "cos_table", "sin_table", "k_pages", "v_pages")]
                + [("num_pages", _i)])


class Routing(ctypes.Structure):
    _fields_ = [(n, _i) for n in ("sms", "tcgen05_min_rows", "tcgen05_min_tiles", "tcgen05_min_fill_pct", "skinny_min_blocks",
                                  "library_only")]


class RunnerEnv(ctypes.Structure):
    _fields_ = ([(n, _i) for n in ("dtype", "page_size", "max_blocks", "fused_norms", "plain_attention", "legacy_tensor_cores")]
                + [("routing", Routing), ("status", _p)])


class RunnerStep(ctypes.Structure):
    _fields_ = ([(n, _i) for n in ("ntok", "nreq", "n_want", "context")]
                + [(n, _p) for n in ("tokens", "positions", "row_req", "req_start", "req_pos", "want_rows")]
                + [("block_tables", _p * MAX_GROUPS), ("lists", _p * MAX_LISTS), ("list_n", _i * MAX_LISTS)])


class RunnerBuffers(ctypes.Structure):
    _fields_ = [("slot", _p * len(SLOTS)), ("bytes", _ll * len(SLOTS)), ("workspace", _p), ("workspace_bytes", _ll),
                ("sumsq", _p), ("sumsq_rows", _i)]


class _Fns(ctypes.Structure):
    _fields_ = [(n, _p) for n in (
        "embed", "add_rmsnorm", "residual_add", "swiglu", "rope_kv", "gemm_f32", "linear_small", "linear_small_qkv", "gemm_tcgen05",
        "gemm_tcgen05_qkv", "attention_rows", "attention_decode", "attention_prefill", "attention_prefill_supports",
        "attention_tcgen05", "err_elementwise", "err_linear_small", "err_gemm_tcgen05", "err_attention", "err_attention_tcgen05",
        "linear_small_supports", "linear_small_qkv_supports", "gemm_skinny", "linear_small_norm_supports", "linear_small_norm",
        "linear_small_qkv_norm", "argmax", "sample", "err_sampling")]


def _addr(lib, name: str) -> int:
    return ctypes.cast(getattr(lib, name), ctypes.c_void_p).value


_bound: Dict[str, bool] = {"base": False, "gemm_tcgen05": False, "attention_tcgen05": False}


def runner_lib(gemm_tcgen05: bool = False, attention_tcgen05: bool = False) -> ctypes.CDLL:
    """The native step's library with the kernel modules' entry points handed over.  The tcgen05 modules are bound (and so
    compiled) only when asked for: a model whose steps never reach them never builds them."""
    lib = _build.load("runner")
    want = {"base": True, "gemm_tcgen05": gemm_tcgen05, "attention_tcgen05": attention_tcgen05}
    if all(_bound[k] or not want[k] for k in want):
        return lib
    lib.jk_runner_last_error.restype = ctypes.c_char_p
    names = ["elementwise", "linear_small", "attention", "sampling"] + (["gemm_tcgen05"] if gemm_tcgen05 else []) \
        + (["attention_tcgen05"] if attention_tcgen05 else [])
    mods = {m: _build.load(m) for m in names}
    get = lambda module, name: _addr(mods[module], name) if module in mods else None
    fns = _Fns(
        embed=get("elementwise", "jk_embed"), add_rmsnorm=get("elementwise", "jk_add_rmsnorm"),
        residual_add=get("elementwise", "jk_residual_add"), swiglu=get("elementwise", "jk_swiglu"),
        rope_kv=get("elementwise", "jk_rope_kv"), gemm_f32=get("elementwise", "jk_gemm_f32"),
        linear_small=get("linear_small", "jk_linear_small"), linear_small_qkv=get("linear_small", "jk_linear_small_qkv"),
        gemm_tcgen05=get("gemm_tcgen05", "jk_gemm_tcgen05"), gemm_tcgen05_qkv=get("gemm_tcgen05", "jk_gemm_tcgen05_qkv"),
        gemm_skinny=get("gemm_tcgen05", "jk_gemm_skinny"),
        linear_small_supports=get("linear_small", "jk_linear_small_supports"),
        linear_small_qkv_supports=get("linear_small", "jk_linear_small_qkv_supports"),
        linear_small_norm_supports=get("linear_small", "jk_linear_small_norm_supports"),
        linear_small_norm=get("linear_small", "jk_linear_small_norm"),
        linear_small_qkv_norm=get("linear_small", "jk_linear_small_qkv_norm"),
        attention_rows=get("attention", "jk_attention_rows"), attention_decode=get("attention", "jk_attention_decode"),
        attention_prefill=get("attention", "jk_attention_prefill"),
        attention_prefill_supports=get("attention", "jk_attention_prefill_supports"),
        attention_tcgen05=get("attention_tcgen05", "jk_attention_tcgen05"),
        err_elementwise=get("elementwise", "jk_elementwise_last_error"),
        err_linear_small=get("linear_small", "jk_linear_small_last_error"),
        err_gemm_tcgen05=get("gemm_tcgen05", "jk_gemm_tcgen05_last_error"),
        err_attention=get("attention", "jk_attention_last_error"),
        err_attention_tcgen05=get("attention_tcgen05", "jk_attention_tcgen05_last_error"),
        # the C interface of the same library (csrc/model_api.h) samples through these
        argmax=get("sampling", "jk_argmax"), sample=get("sampling", "jk_sample"),
        err_sampling=get("sampling", "jk_sampling_last_error"))
    if lib.jk_runner_bind(ctypes.byref(fns)):
        from ..kernels import KernelError
        raise KernelError(lib.jk_runner_last_error().decode(errors="replace"))
    for k in want:
        _bound[k] = _bound[k] or want[k]
    return lib


def check_struct_sizes(lib) -> None:
    """The ctypes mirrors above against the structs of csrc/runner.h, by size."""
    sizes = (ctypes.c_int * 5)()
    lib.jk_runner_struct_sizes(sizes)
    mine = [ctypes.sizeof(t) for t in (RunnerOp, RunnerEnv, RunnerStep, RunnerBuffers, _Fns)]
    if list(sizes) != mine:
        raise RuntimeError(f"the records' layout differs between Python {mine} and csrc/runner.h {list(sizes)}")


class HostIO:
    """What a host step sees of a step's buffers: torch views of the slots for the rows of this step."""

    def __init__(self, runner: "ProgramRunner", rows: int):
        self._runner, self.rows = runner, rows

    def view(self, slot: str, width: int, dtype: Optional[torch.dtype] = None, rows: Optional[int] = None) -> torch.Tensor:
        """``[rows, width]`` of a slot (the activations' type unless said otherwise; ``x`` and ``delta`` are float32)."""
        rows = self.rows if rows is None else rows
        if dtype is None:
            dtype = torch.float32 if slot in ("x", "delta", "logits", "tmp", "decode") else self._runner.runtime.dtype
        raw = self._runner.slot_tensor(slot)
        need = rows * width * torch.empty((), dtype=dtype).element_size()
        if need > raw.numel():
            raise ValueError(f"slot {slot} holds {raw.numel()} bytes, {rows} rows of {width} need {need}")
        return raw[:need].view(dtype).view(rows, width)


class Program:
    """The model's operations in order: runs of native records, and host steps between them."""

    def __init__(self, runtime, hidden_size: int, page_size: int, max_blocks: int, capacity: int = 64):
        self.runtime, self.hidden_size = runtime, hidden_size
        self.page_size, self.max_blocks = page_size, max_blocks
        self.lib = _build.load("runner")
        self._cap = capacity
        self.ops = (RunnerOp * capacity)()
        self.count = 0
        self.items: List[Tuple] = []          # ("ops", first, count) | ("host", fn)
        self.keep: List[object] = []          # tensors that the records point into
        self.lists: Dict[str, int] = {}       # name of a work list -> its index in a step's lists
        self.list_owners: List[type] = []     # mixer classes whose work lists the steps must carry
        check_struct_sizes(self.lib)

    # ---- emitting ----------------------------------------------------------------------------------------------------
    def _room(self, n: int) -> ctypes.c_void_p:
        if self.count + n > self._cap:
            self._cap = max(2 * self._cap, self.count + n)
            grown = (RunnerOp * self._cap)()
            ctypes.memmove(grown, self.ops, ctypes.sizeof(RunnerOp) * self.count)
            self.ops = grown
        return ctypes.byref(self.ops, ctypes.sizeof(RunnerOp) * self.count)

    def _emitted(self, n: int) -> None:
        if self.items and self.items[-1][0] == "ops":
            _, first, count = self.items[-1]
            self.items[-1] = ("ops", first, count + n)
        else:
            self.items.append(("ops", self.count, n))
        self.count += n

    def emit(self, emitter: str, *args, keep=()) -> None:
        """Call a native emitter (``jk_emit_*`` of csrc/runner.cu) that writes its records at the program's end."""
        fn = getattr(self.lib, emitter)
        self._emitted(fn(self._room(8), *args))
        self.keep.extend(keep)

    def host(self, fn: Callable) -> None:
        """A step of the model that its own Python code runs: ``fn(ctx, io)`` with ``io`` a ``HostIO``.  The stream is
        whole when it is called (no product waits for its addition) and must be whole when it returns."""
        self.items.append(("host", fn))

    def work_lists(self, owner: type, names) -> List[int]:
        """Indices, in a step's lists, of the work lists that the mixer class ``owner`` fills for every step."""
        if owner not in self.list_owners:
            self.list_owners.append(owner)
            for n in names:
                if len(self.lists) >= MAX_LISTS:
                    raise ValueError(f"a step carries at most {MAX_LISTS} work lists")
                self.lists[f"{owner.__name__}.{n}"] = len(self.lists)
        return [self.lists[f"{owner.__name__}.{n}"] for n in names]

    # ---- reading ------------------------------------------------------------------------------------------------------
    @property
    def native_only(self) -> bool:
        return all(kind == "ops" for kind, *_ in self.items)

    def launch_list(self) -> List[str]:
        """The program in words, one entry per record or host step."""
        out = []
        for item in self.items:
            if item[0] == "host":
                out.append("host:" + getattr(item[1], "__qualname__", repr(item[1])))
            else:
                out.extend(OP_NAMES.get(self.ops[i].kind, "?") for i in range(item[1], item[1] + item[2]))
        return out


def _dtype_code(dtype: torch.dtype) -> int:
    from .. import kernels
    return kernels.dtype_code(dtype)


class ProgramRunner:
    """Buffers for steps of up to ``max_rows`` rows, and the call that replays a program over them."""

    WORKSPACE_BYTES = 32 << 20

    def __init__(self, program: Program, max_rows: int, max_want: Optional[int] = None, one_by_one: bool = False):
        from .. import kernels
        self.program, self.runtime = program, program.runtime
        rt = self.runtime
        self.max_rows, self.max_want = max_rows, max_want or max_rows
        self.one_by_one = one_by_one
        self.env = rt.env(program.page_size, program.max_blocks)
        need_gemm = bool(program.lib.jk_runner_needs_gemm_tcgen05(ctypes.byref(self.env), program.ops, program.count, max_rows))
        need_attn = rt.dtype == torch.bfloat16 and not rt.legacy_tensor_cores and any(
            program.ops[i].kind == 4 and _host.attention_tcgen05_takes(program.ops[i].head_dim, program.page_size)
            for i in range(program.count))
        self.lib = runner_lib(need_gemm, need_attn)
        self.lib.jk_runner_last_error.restype = ctypes.c_char_p
        sizes = (_ll * len(SLOTS))()
        self._check(self.lib.jk_runner_slot_bytes(ctypes.byref(self.env), program.ops, program.count, max_rows, self.max_want, sizes))
        sizes[SLOT["x"]] = max(sizes[SLOT["x"]], 4 * max_rows * program.hidden_size)         # host steps see the stream too
        sizes[SLOT["h"]] = max(sizes[SLOT["h"]], 4 * max_rows * program.hidden_size)
        sizes[SLOT["logits"]] = 0                                                           # made per step: the caller keeps them
        self._slots = [torch.empty(max(int(b), 16), dtype=torch.uint8, device=rt.device) for b in sizes]
        self._workspace = torch.empty(self.WORKSPACE_BYTES, dtype=torch.uint8, device=rt.device)
        self._sumsq = torch.zeros(max(1, program.count), 16, dtype=torch.int64, device=rt.device)
        self.buffers = RunnerBuffers(workspace=self._workspace.data_ptr(), workspace_bytes=self.WORKSPACE_BYTES,
                                     sumsq=self._sumsq.data_ptr(), sumsq_rows=max(1, program.count))
        for s, t in enumerate(self._slots):
            self.buffers.slot[s] = t.data_ptr()
            self.buffers.bytes[s] = t.numel()
        self.launches = 0
        self._routing_key = rt.routing_key()

    def slot_tensor(self, name: str) -> torch.Tensor:
        return self._slots[SLOT[name]]

    def _check(self, rc: int) -> None:
        if rc:
            from ..kernels import KernelError
            raise KernelError(self.lib.jk_runner_last_error().decode(errors="replace") or f"the native step returned {rc}")

    def forward(self, ctx, vocab_size: int) -> torch.Tensor:
        """Run the program for the step that ``ctx`` describes; float32 logits ``[wanted rows, vocab]``."""
        from .. import kernels
        rt, prog = self.runtime, self.program
        if rt.routing_key() != self._routing_key:       # a test moved a threshold or a switch
            self._routing_key = rt.routing_key()
            self.env = rt.env(prog.page_size, prog.max_blocks)
            need_gemm = bool(prog.lib.jk_runner_needs_gemm_tcgen05(ctypes.byref(self.env), prog.ops, prog.count, self.max_rows))
            runner_lib(need_gemm, _bound["attention_tcgen05"])
        T = ctx.ntok
        if T > self.max_rows:
            raise kernels.KernelError(f"the step's buffers hold {self.max_rows} rows, the step has {T}")
        n_want = ctx.want_rows.numel()
        logits = torch.empty(n_want, vocab_size, dtype=torch.float32, device=rt.device)
        self.buffers.slot[SLOT["logits"]] = logits.data_ptr()
        self.buffers.bytes[SLOT["logits"]] = logits.numel() * 4
        step = RunnerStep(ntok=T, nreq=ctx.nreq, n_want=n_want, context=ctx.context,
                          tokens=ctx.tokens.data_ptr(), positions=ctx.positions.data_ptr(), row_req=ctx.row_req.data_ptr(),
                          req_start=ctx.req_start.data_ptr(), req_pos=ctx.req_pos.data_ptr(), want_rows=ctx.want_rows.data_ptr())
        for g, table in enumerate(ctx.block_tables):
            step.block_tables[g] = table.data_ptr()
        for name, index in prog.lists.items():
            view, n = ctx.lists[name]
            step.lists[index] = view.data_ptr() if view is not None else None
            step.list_n[index] = n
        stream = kernels._stream()
        self.launches = 0
        items = prog.items
        for idx, item in enumerate(items):
            if item[0] == "host":
                before = kernels.launch_count
                item[1](ctx, HostIO(self, T))
                self.launches += kernels.launch_count - before
                continue
            _, first, count = item
            flush = 1 if idx + 1 < len(items) else 0
            if self.one_by_one:
                # every record a call of its own (with the stream made whole after each): no record can share work with
                # its neighbours, which is the unfused way of running the same program
                for i in range(first, first + count):
                    self._check(self.lib.jk_runner_run(ctypes.byref(self.env), prog.ops, i, 1, ctypes.byref(step),
                                                       ctypes.byref(self.buffers), 1, stream))
                    self.launches += self.lib.jk_runner_launches()
            else:
                self._check(self.lib.jk_runner_run(ctypes.byref(self.env), prog.ops, first, count, ctypes.byref(step),
                                                   ctypes.byref(self.buffers), flush, stream))
                self.launches += self.lib.jk_runner_launches()
        return logits


def step_lists_for(owners, ctx, device) -> Dict[str, tuple]:
    """The work lists that the mixer classes ``owners`` ask for, made for a hand-built step context (the engine makes
    them inside its metadata buffer; a part run alone gets them here)."""
    import numpy as np
    starts, B = list(ctx.host_req_start), ctx.nreq
    lens = [starts[i + 1] - starts[i] for i in range(B)]
    pos = list(ctx.host_req_pos)
    out = {}
    for owner in owners:
        caps = owner.step_list_capacity(ctx.ntok, B)
        arrays = {n: np.zeros(max(1, c), dtype=np.int32) for n, c in caps.items()}
        for name, (count, identity) in owner.fill_step_lists(B, B, lens, pos, arrays).items():
            view = None if identity else torch.from_numpy(arrays[name]).to(device)
            out[f"{owner.__name__}.{name}"] = (view, count)
    return out


def run_part_alone(runtime, plan, ctx, h: torch.Tensor, hidden_size: int, page_size: int = 16) -> torch.Tensor:
    """A mixer or feed-forward by itself: its records (emitted by ``plan(program)`` with a residual scale of 1) run
    over the activations ``h`` into a stream of zeros, which is then the part's output, float32 ``[T, hidden]``.
    For tests of a part alone and for blocks arranged by hand; a model runs its parts' records in one program."""
    T = h.shape[0]
    max_blocks = ctx.block_tables[0].shape[1] if ctx is not None and ctx.block_tables else 1
    program = Program(runtime, hidden_size, page_size, max_blocks, capacity=8)
    plan(program)
    runner = ProgramRunner(program, max_rows=T)
    io = HostIO(runner, T)
    io.view("h", h.shape[1]).copy_(h)
    x = io.view("x", hidden_size)
    x.zero_()
    if ctx is None:             # a part that looks at no batch (a feed-forward): rows only
        from .base import StepContext
        z = torch.zeros(max(T, 2), dtype=torch.int32, device=runtime.device)
        ctx = StepContext(ntok=T, nreq=1, tokens=z, positions=z, row_req=z, req_start=z, req_pos=z, slot_ids=z,
                          block_tables=[], want_rows=z[:0], n_want=0, host_req_start=[0, T], host_req_pos=[0])
    if any(name not in ctx.lists for name in program.lists):
        ctx.lists.update(step_lists_for(program.list_owners, ctx, runtime.device))
    from .. import kernels
    step = RunnerStep(ntok=T, nreq=ctx.nreq, n_want=0, context=ctx.context, tokens=ctx.tokens.data_ptr(),
                      positions=ctx.positions.data_ptr(), row_req=ctx.row_req.data_ptr(), req_start=ctx.req_start.data_ptr(),
                      req_pos=ctx.req_pos.data_ptr(), want_rows=None)
    for g, table in enumerate(ctx.block_tables):
        step.block_tables[g] = table.data_ptr()
    for name, index in program.lists.items():
        view, n = ctx.lists[name]
        step.lists[index] = view.data_ptr() if view is not None else None
        step.list_n[index] = n
    runner._check(runner.lib.jk_runner_run(ctypes.byref(runner.env), program.ops, 0, program.count, ctypes.byref(step),
                                          ctypes.byref(runner.buffers), 1, kernels._stream()))
    kernels.launch_count += runner.lib.jk_runner_launches()
    return x.clone()
