"""Weights by tensor name.

A model's parts declare the tensors they own (name, shape, role); the union is
the manifest.  ``check_manifest`` compares it with what a checkpoint holds and
raises ONE error that lists every missing tensor, every unexpected one and every
wrong shape.  A ``WeightSource`` then hands tensors to the parts on the device.

Storage rule: floating-point tensors stored in 16 bits are kept in bfloat16,
integer tables become int32, and a tensor stored in 32 bits stays in 32 bits.
The *compute* type of a matrix is the engine's: in bfloat16 mode a matrix stored
wider is rounded once at load, because the tensor-core products take 16-bit
operands; in float32 mode everything floating is widened (exactly) to float32.
Vectors (norm weights) are used in float32 in both modes, as the reference keeps
them (scripts/jiuge.py:145-146).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, TensorInfo, index_directory, read_tensor

MATRIX = "matrix"     # operand of a matrix product: compute dtype
VECTOR = "vector"     # norm weights, biases: float32
TABLE = "table"       # integer tables: int32
KEEP = "keep"         # as stored (16-bit floats as bfloat16, 32-bit stays)


@dataclass(frozen=True)
class TensorDecl:
    shape: Tuple[int, ...]
    role: str = MATRIX
    optional: bool = False
    init: str = "normal"      # random-weights mode: "normal" N(0, std) or "ones" 1 + N(0, norm_std)


class WeightError(ValueError):
    """The checkpoint does not hold what the model needs."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"checkpoint {where} does not fit the model:".replace("  ", " ")]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


class UnusedTensorsWarning(UserWarning):
    """The checkpoint holds tensors that the model does not use."""


def check_manifest(manifest: Mapping[str, TensorDecl], found: Mapping[str, Tuple[int, ...]],
                   where: str = "", strict: bool = False) -> None:
    """Compare what the model's parts declare with what the checkpoint holds.  Missing tensors and wrong shapes
    raise ONE ``WeightError`` that lists them all.  Tensors that no part declared are left alone with an
    ``UnusedTensorsWarning`` that names them, as the reference reads every key of a checkpoint and uses what it
    needs (scripts/jiuge.py:400-407; checkpoints carry such extras, e.g. ``rotary_emb.inv_freq``); with
    ``strict=True`` they are part of the error."""
    missing = [n for n, d in manifest.items() if n not in found and not d.optional]
    unexpected = sorted(n for n in found if n not in manifest)
    wrong = [(n, manifest[n].shape, tuple(found[n])) for n in manifest
             if n in found and tuple(found[n]) != tuple(manifest[n].shape)]
    if missing or wrong or (strict and unexpected):
        raise WeightError(sorted(missing), unexpected, sorted(wrong), where)
    if unexpected:
        shown = ", ".join(unexpected[:8]) + (", ..." if len(unexpected) > 8 else "")
        warnings.warn(f"checkpoint {where} holds {len(unexpected)} tensors that the model does not use: {shown}".replace("  ", " "),
                      UnusedTensorsWarning, stacklevel=2)


def stored_dtype(dtype: torch.dtype) -> torch.dtype:
    """The type a tensor is kept in, by the storage rule above."""
    if dtype in (torch.float16, torch.bfloat16):
        return torch.bfloat16
    if dtype in (torch.float32, torch.float64):
        return torch.float32
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise ValueError(f"unsupported tensor type {dtype}")


def _to_role(t: torch.Tensor, role: str, compute: torch.dtype) -> torch.Tensor:
    if role == TABLE:
        return t.to(torch.int32)
    if role == VECTOR:
        return t.to(torch.float32)
    if role == MATRIX:
        return t.to(compute)
    keep = stored_dtype(t.dtype)
    if compute == torch.float32 and keep == torch.bfloat16:
        keep = torch.float32
    return t.to(keep)


class WeightSource:
    """Hands out tensors by name, on ``device``, in the type their role asks for."""

    def __init__(self, compute_dtype: torch.dtype, device):
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)

    def plan(self, manifest: Mapping[str, TensorDecl]) -> None:
        """Told once, before the parts are built, which tensors will be asked for and in which role."""

    def close(self) -> None:
        """Told once the parts are built: nothing more will be asked for."""

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        raise NotImplementedError

    def get_rows(self, names: Sequence[str], role: str = MATRIX) -> torch.Tensor:
        """The named tensors one below the other (along their first dimension) as ONE tensor: how a part asks for
        a fused matrix ([q | k | v], [gate | up]).  A source that can place the pieces directly overrides this."""
        if len(names) == 1:
            return self.get(names[0], role)
        return torch.cat([self.get(n, role) for n in names], dim=0).contiguous()


def _target_dtype(stored: torch.dtype, role: str, compute: torch.dtype) -> torch.dtype:
    """The type a tensor stored as ``stored`` is handed out in (what ``_to_role`` produces)."""
    if role == TABLE:
        return torch.int32
    if role == VECTOR:
        return torch.float32
    if role == MATRIX:
        return compute
    keep = stored_dtype(stored)
    return torch.float32 if (compute == torch.float32 and keep == torch.bfloat16) else keep


class Float16RoundedWarning(UserWarning):
    """A float16 checkpoint runs in the bfloat16 engine: its matrices lose three bits of mantissa."""


class FileWeights(WeightSource):
    """Tensors of the ``*.safetensors`` files of a model folder.

    On a CUDA device all tensors live in ONE device allocation (an arena sized from the manifest in ``plan``): a fused
    matrix is one slice of it and each checkpoint tensor is copied straight to its rows, so nothing is concatenated
    on the device and no tensor has an allocation of its own.  Bytes travel through two pinned staging buffers of
    fixed size that take turns: the file is read into one while the other's asynchronous copy is in flight.  (The
    reference allocates and copies tensor by tensor, blocking, under a global lock: src/tensor/tensor.cpp:142-167.)
    """

    STAGING_BYTES = 32 << 20
    ALIGN = 256

    def __init__(self, model_dir: str, compute_dtype: torch.dtype, device):
        super().__init__(compute_dtype, device)
        self.model_dir = model_dir
        self.index: Dict[str, TensorInfo] = index_directory(model_dir)
        self._arena: Optional[torch.Tensor] = None
        self._arena_used = 0
        self._staging: List[torch.Tensor] = []
        self._events: List[Optional[object]] = [None, None]
        self._turn = 0
        self._warned_f16 = False
        self.arena_bytes = 0          # size of the arena; outside_arena counts tensors that did not fit it
        self.outside_arena = 0

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: i.shape for n, i in self.index.items()}

    def has(self, name: str) -> bool:
        return name in self.index

    # ---- the arena ---------------------------------------------------------------------------------------
    def plan(self, manifest: Mapping[str, TensorDecl]) -> None:
        if self.device.type != "cuda" or self._arena is not None:
            return
        total = 0
        for name, decl in manifest.items():
            info = self.index.get(name)
            if info is not None:
                size = _numel(info.shape) * _itemsize(_target_dtype(info.dtype, decl.role, self.compute_dtype))
                total += -(-size // self.ALIGN) * self.ALIGN + self.ALIGN      # a fused matrix starts aligned once
        self._arena = torch.empty(max(total, self.ALIGN), dtype=torch.uint8, device=self.device)
        self.arena_bytes = self._arena.numel()

    def _alloc(self, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        size = _numel(shape) * _itemsize(dtype)
        begin = -(-self._arena_used // self.ALIGN) * self.ALIGN
        if self._arena is None or begin + size > self._arena.numel():
            self.outside_arena += 1
            return torch.empty(shape, dtype=dtype, device=self.device)
        self._arena_used = begin + size
        return self._arena[begin:begin + size].view(dtype).view(shape)

    def close(self) -> None:
        """Wait for the copies in flight and let the staging buffers go."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._staging, self._events = [], [None, None]

    # ---- bytes: file -> pinned staging -> device -----------------------------------------------------------
    def _stream(self, info: TensorInfo, dst: torch.Tensor) -> None:
        """The tensor's stored bytes into ``dst`` (contiguous, of the stored type and shape)."""
        if not info.nbytes:
            return
        if self.device.type != "cuda":
            dst.copy_(read_tensor(info))
            return
        if not self._staging:
            self._staging = [torch.empty(self.STAGING_BYTES, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        raw = dst.view(-1).view(torch.uint8)
        with open(info.path, "rb") as f:
            f.seek(info.begin)
            done = 0
            while done < info.nbytes:
                n = min(self.STAGING_BYTES, info.nbytes - done)
                turn, self._turn = self._turn, self._turn ^ 1
                if self._events[turn] is not None:
                    self._events[turn].synchronize()          # its last copy has left the buffer
                buf = self._staging[turn]
                got = f.readinto(memoryview(buf.numpy())[:n])
                if got != n:
                    raise SafetensorsError(f"{info.path}: short read of {info.name} ({done + got} of {info.nbytes} bytes)")
                raw[done:done + n].copy_(buf[:n], non_blocking=True)
                if self._events[turn] is None:
                    self._events[turn] = torch.cuda.Event()
                self._events[turn].record()
                done += n

    def _load_into(self, info: TensorInfo, dst: torch.Tensor, role: str) -> None:
        if info.dtype == dst.dtype:
            self._stream(info, dst)
            return
        if info.dtype == torch.float16 and dst.dtype == torch.bfloat16 and not self._warned_f16:
            self._warned_f16 = True
            warnings.warn(f"checkpoint {self.model_dir} stores {info.name} (and maybe more) in float16; the bfloat16 engine "
                          "rounds such matrices to bfloat16 (8 bits of mantissa instead of 11), where the reference keeps "
                          "float16; dtype float32 runs them exactly", Float16RoundedWarning, stacklevel=4)
        tmp = torch.empty(info.shape, dtype=info.dtype, device=self.device)
        self._stream(info, tmp)
        dst.copy_(tmp)          # converts on the device; the order of the stream keeps tmp alive until then

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        return self.get_rows([name], role)

    def get_rows(self, names: Sequence[str], role: str = MATRIX) -> torch.Tensor:
        infos = [self.index[n] for n in names]
        rest = infos[0].shape[1:]
        if any(i.shape[1:] != rest or not i.shape for i in infos[1:]) or (len(infos) > 1 and not infos[0].shape):
            raise ValueError(f"tensors {list(names)} cannot be stacked: shapes {[i.shape for i in infos]}")
        dtype = _target_dtype(infos[0].dtype, role, self.compute_dtype)
        if len(infos) == 1:
            out = self._alloc(infos[0].shape, dtype)
            self._load_into(infos[0], out, role)
            return out
        out = self._alloc((sum(i.shape[0] for i in infos),) + tuple(rest), dtype)
        row = 0
        for info in infos:
            self._load_into(info, out[row:row + info.shape[0]], role)
            row += info.shape[0]
        return out


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class DictWeights(WeightSource):
    """Tensors given in memory (tests, and models built from a random generator)."""

    def __init__(self, tensors: Mapping[str, torch.Tensor], compute_dtype: torch.dtype, device):
        super().__init__(compute_dtype, device)
        self.tensors = dict(tensors)

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: tuple(t.shape) for n, t in self.tensors.items()}

    def has(self, name: str) -> bool:
        return name in self.tensors

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        t = self.tensors[name]
        if t.dtype == torch.float16:
            t = t.float() if (role == VECTOR or self.compute_dtype == torch.float32) else t.to(torch.bfloat16)
        return _to_role(t.to(self.device), role, self.compute_dtype).contiguous()
