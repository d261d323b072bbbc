"""Random-weights mode: a model from a configuration and a seed.

``write_model_folder`` writes ``config.json`` and ``model.safetensors`` so that the
folder loads through the ordinary path.  ``DeviceRandomWeights`` makes the same kind of
tensors directly on the GPU, for shapes whose weights would be gigabytes on the host.
The reference has no such mode; matrices are N(0, std), norm weights 1 + N(0, norm_std).
Each tensor's values depend on the seed and its own name only.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping

import torch

from .loader import MATRIX, TABLE, VECTOR, TensorDecl, WeightSource, _to_role
from .safetensors_io import write_file


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
    return g


def _make(name: str, decl: TensorDecl, seed: int, std: float, norm_std: float, device="cpu") -> torch.Tensor:
    g = _generator(seed, name, device)
    if decl.role == TABLE:
        return torch.randint(0, 2 ** 15, decl.shape, generator=g, device=device, dtype=torch.int32)
    x = torch.randn(decl.shape, generator=g, device=device, dtype=torch.float32)
    if decl.init == "ones":
        return 1.0 + norm_std * x
    return std * x


def random_tensors(manifest: Mapping[str, TensorDecl], seed: int, std: float = 0.02,
                   norm_std: float = 0.01, matrix_dtype: torch.dtype = torch.bfloat16,
                   include_optional: bool = False) -> Dict[str, torch.Tensor]:
    """Host tensors for every declared name; matrices in ``matrix_dtype``, vectors in float32."""
    out = {}
    for name, decl in manifest.items():
        if decl.optional and not include_optional:
            continue
        t = _make(name, decl, seed, std, norm_std)
        out[name] = t.to(matrix_dtype) if decl.role == MATRIX else t
    return out


def write_model_folder(config, out_dir: str, seed: int, std: float = 0.02, norm_std: float = 0.01,
                       matrix_dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration)."""
    from ..parts.model import model_manifest
    os.makedirs(out_dir, exist_ok=True)
    spec = config.model_spec()
    tensors = random_tensors(model_manifest(spec), seed, std, norm_std, matrix_dtype,
                             include_optional=not spec.tie_embeddings)
    write_file(os.path.join(out_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    return out_dir


class DeviceRandomWeights(WeightSource):
    """Random tensors made on the device when a part asks for them."""

    def __init__(self, manifest: Mapping[str, TensorDecl], seed: int, compute_dtype, device,
                 std: float = 0.02, norm_std: float = 0.01, untied: bool = False):
        super().__init__(compute_dtype, device)
        self.manifest = dict(manifest)
        self.seed, self.std, self.norm_std, self.untied = seed, std, norm_std, untied

    def shapes(self):
        return {n: d.shape for n, d in self.manifest.items() if not d.optional or self.untied}

    def has(self, name: str) -> bool:
        return name in self.manifest and (not self.manifest[name].optional or self.untied)

    def get(self, name: str, role: str = MATRIX) -> torch.Tensor:
        decl = self.manifest[name]
        t = _make(name, decl, self.seed, self.std, self.norm_std, device=self.device)
        if decl.role == MATRIX:
            t = t.to(torch.bfloat16)       # what a 16-bit checkpoint would hold
        return _to_role(t, role, self.compute_dtype).contiguous()
