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

from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .safetensors_io import TensorInfo, index_directory, read_tensor

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


def check_manifest(manifest: Mapping[str, TensorDecl], found: Mapping[str, Tuple[int, ...]],
                   where: str = "") -> None:
    missing = [n for n, d in manifest.items() if n not in found and not d.optional]
    unexpected = [n for n in found if n not in manifest]
    wrong = [(n, manifest[n].shape, tuple(found[n])) for n in manifest
             if n in found and tuple(found[n]) != tuple(manifest[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong), where)


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

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        raise NotImplementedError


class FileWeights(WeightSource):
    """Tensors of the ``*.safetensors`` files of a model folder."""

    def __init__(self, model_dir: str, compute_dtype: torch.dtype, device):
        super().__init__(compute_dtype, device)
        self.model_dir = model_dir
        self.index: Dict[str, TensorInfo] = index_directory(model_dir)

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: i.shape for n, i in self.index.items()}

    def has(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        info = self.index[name]
        host = read_tensor(info, pin=self.device.type == "cuda")
        if host.dtype == torch.float16:       # 16-bit: bfloat16 in the bfloat16 engine, widened exactly in float32
            host = host.float() if (role == VECTOR or self.compute_dtype == torch.float32) else host.to(torch.bfloat16)
        dev = host.to(self.device, non_blocking=False)
        return _to_role(dev, role, self.compute_dtype).contiguous()


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
