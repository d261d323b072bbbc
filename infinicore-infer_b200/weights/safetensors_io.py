"""Reading and writing the safetensors container, by tensor name.

Layout of a file: an unsigned 64-bit little-endian header length N, N bytes of
JSON mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header), then the raw little-endian data.
The reference reads such files through the ``safetensors`` package
(scripts/jiuge.py:400-407); here the header is parsed directly, so that a tensor's
shape and type are known before a single byte of data is read.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int      # absolute byte offset in the file
    nbytes: int
    path: str


def read_header(path: str) -> Dict[str, TensorInfo]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
    out: Dict[str, TensorInfo] = {}
    base = 8 + n
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        if rec["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {rec['dtype']}")
        dtype = _DTYPES[rec["dtype"]]
        shape = tuple(int(s) for s in rec["shape"])
        begin, end = (int(x) for x in rec["data_offsets"])
        numel = 1
        for s in shape:
            numel *= s
        want = numel * torch.empty((), dtype=dtype).element_size()
        if end - begin != want or base + end > size or begin < 0:
            raise SafetensorsError(
                f"{path}: tensor {name} of shape {shape} {rec['dtype']} needs {want} bytes, "
                f"its offsets [{begin}, {end}) give {end - begin} (file data: {size - base} bytes)")
        out[name] = TensorInfo(name, dtype, shape, base + begin, want, path)
    return out


def read_tensor(info: TensorInfo, pin: bool = False) -> torch.Tensor:
    """Read one tensor's bytes straight into a (pinned, if asked) host tensor."""
    t = torch.empty(info.shape, dtype=info.dtype, pin_memory=pin)
    if info.nbytes:
        flat = t.view(-1) if t.dim() else t.reshape(1)
        raw = memoryview(flat.view(torch.uint8).numpy())
        with open(info.path, "rb") as f:
            f.seek(info.begin)
            got = f.readinto(raw)
        if got != info.nbytes:
            raise SafetensorsError(f"{info.path}: short read of {info.name} ({got} of {info.nbytes} bytes)")
    return t


def write_file(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order: List[str] = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {name}: dtype {t.dtype}")
        flat = t.view(-1) if t.dim() else t.reshape(1)
        raw = flat.view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)      # data begins on an 8-byte boundary
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def index_directory(model_dir: str) -> Dict[str, TensorInfo]:
    """Headers of every ``*.safetensors`` file of a folder, in sorted file order."""
    files = sorted(p for p in os.listdir(model_dir) if p.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors file in {model_dir}")
    out: Dict[str, TensorInfo] = {}
    for p in files:
        out.update(read_header(os.path.join(model_dir, p)))
    return out
