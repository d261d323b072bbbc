"""The engine through its C interface (``csrc/model_api.h``), for programs without Python.

``NativeModel`` is a thin ctypes wrapper over that interface: it reads a model folder with the package's
own configuration and weight readers, hands the host tensors to ``jkCreateModel`` and then only calls
``jkCreateKVCache`` / ``jkInferBatch`` / ``jkForwardBatch`` / ``jkDropKVCache``.  The kernel modules are
found by the C side itself in the build folder (``dlopen``), as a C program would find them.  The step
is the native runner's, so the model has to be one the runner takes: bfloat16, the standard block of
this architecture (the Python engine covers everything else).

The reference's counterpart is scripts/libinfinicore_infer.py (the ctypes declarations of its C
interface) together with the calls of scripts/jiuge.py:430-520.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import build as _build


class _Meta(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("nlayer", "d", "nh", "nkvh", "dh", "di", "dctx", "dvoc")] \
        + [(n, ctypes.c_float) for n in ("epsilon", "theta", "embed_scale", "residual_scale", "logit_scale")] \
        + [("end_token", ctypes.c_int32)]


class _Weights(ctypes.Structure):
    _fields_ = [("norm_dtype", ctypes.c_int32), ("input_embd", ctypes.c_void_p), ("output_norm", ctypes.c_void_p),
                ("output_embd", ctypes.c_void_p)] \
        + [(n, ctypes.POINTER(ctypes.c_void_p)) for n in ("attn_norm", "attn_qkv", "attn_o", "ffn_norm", "ffn_gate_up",
                                                          "ffn_down", "attn_qkv_b")]


class _Options(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int32), ("page_size", ctypes.c_int32), ("cache_tokens", ctypes.c_int64),
                ("max_step_tokens", ctypes.c_int32), ("kernel_dir", ctypes.c_char_p)]


class NativeModelError(RuntimeError):
    pass


def _u32(values) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(values, dtype=np.uint32))


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


class NativeModel:
    """A model created through the C interface from host tensors named as in the checkpoint."""

    def __init__(self, config, tensors: Dict[str, torch.Tensor], device: int = 0, page_size: int = 64,
                 cache_tokens: Optional[int] = None, max_step_tokens: int = 2048, strict: bool = False):
        spec = config.model_spec()
        blocks = [spec.layers[e.layer] for e in spec.order]
        a, f = blocks[0].mixer, blocks[0].feed_forward
        L = len(blocks)
        self.lib = _build.load("runner")
        lib = self.lib
        lib.jkLastError.restype = ctypes.c_char_p
        lib.jkCreateModel.restype = ctypes.c_void_p
        lib.jkCreateKVCache.restype = ctypes.c_void_p
        lib.jkDuplicateKVCache.restype = ctypes.c_void_p
        lib.jkFreePages.restype = ctypes.c_int64
        for fn in (lib.jkCreateKVCache, lib.jkFreePages, lib.jkLastLaunches, lib.jkDestroyModel):
            fn.argtypes = [ctypes.c_void_p]
        lib.jkDuplicateKVCache.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32]
        lib.jkDropKVCache.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.jkDropKVCache.restype = None
        lib.jkDestroyModel.restype = None

        # The same checks and the same packing as the Python engine's: the manifest of the model's parts decides what
        # the checkpoint must hold, and the parts' own ``pack`` functions fuse q | k | v and gate | up.
        from ..parts import model_manifest, part_class
        from ..weights import VECTOR, DictWeights, check_manifest
        check_manifest(model_manifest(spec), {n: tuple(t.shape) for n, t in tensors.items()}, strict=strict)
        source = DictWeights(tensors, torch.bfloat16, "cpu")
        keep: List[torch.Tensor] = []          # what the pointers below point into

        def mat(t: torch.Tensor) -> int:
            keep.append(t)
            return t.data_ptr()

        packed = []
        for e in spec.order:
            b, p = spec.layers[e.layer], spec.layer_prefix.format(e.layer)
            one = dict(part_class("mixer", b.mixer).pack(b.mixer, source, p + b.mixer_prefix))
            one.update(part_class("feed_forward", b.feed_forward).pack(b.feed_forward, source, p + b.ffn_prefix))
            one["norm1"] = source.get(p + b.mixer_norm_prefix + "weight", VECTOR)
            one["norm2"] = source.get(p + b.ffn_norm_prefix + "weight", VECTOR)
            packed.append(one)

        def per_layer(key: str) -> ctypes.Array:
            return (ctypes.c_void_p * L)(*[mat(one[key]) for one in packed])

        embd = mat(source.get(spec.embed_name))
        tied = not source.has(spec.lm_head_name)
        w = _Weights(
            norm_dtype=0, input_embd=embd, output_norm=mat(source.get(spec.final_norm_prefix + "weight", VECTOR)),
            output_embd=embd if tied else mat(source.get(spec.lm_head_name)),
            attn_norm=per_layer("norm1"), attn_qkv=per_layer("w_qkv"), attn_o=per_layer("w_o"),
            ffn_norm=per_layer("norm2"), ffn_gate_up=per_layer("w_gate_up"), ffn_down=per_layer("w_down"))
        if a.bias:
            w.attn_qkv_b = (ctypes.c_void_p * L)(*[mat(one["b_qkv"].float().contiguous()) for one in packed])
        meta = _Meta(nlayer=L, d=spec.hidden_size, nh=a.num_heads, nkvh=a.num_kv_heads, dh=a.head_dim,
                     di=f.intermediate_size, dctx=spec.max_positions, dvoc=spec.vocab_size, epsilon=blocks[0].mixer_norm.eps,
                     theta=a.position.theta if a.position is not None else 0.0, embed_scale=spec.embed_scale,
                     residual_scale=blocks[0].residual_scale, logit_scale=spec.logit_scale,
                     end_token=spec.eos_token_ids[0] if spec.eos_token_ids else 0)
        opt = _Options(device=device, page_size=page_size, cache_tokens=cache_tokens or spec.max_positions,
                       max_step_tokens=max_step_tokens, kernel_dir=_build.build_dir().encode())
        self.vocab_size, self.page_size = spec.vocab_size, page_size
        names = ctypes.create_string_buffer(256)
        if lib.jkKernelModules(ctypes.byref(meta), ctypes.byref(opt), names, 256):
            raise NativeModelError(self._message())
        for module in names.value.decode().split(","):      # compiled here, loaded by the C side from the folder
            _build.build(module)
        self.handle = lib.jkCreateModel(ctypes.byref(meta), ctypes.byref(w), ctypes.byref(opt))
        if not self.handle:
            raise NativeModelError(self._message())

    @classmethod
    def from_folder(cls, model_dir: str, **kwargs) -> "NativeModel":
        from ..config import read_config
        from ..weights.safetensors_io import index_directory, read_tensor
        config = read_config(model_dir)
        tensors = {name: read_tensor(info) for name, info in index_directory(model_dir).items()}
        return cls(config, tensors, **kwargs)

    def _message(self) -> str:
        return self.lib.jkLastError().decode(errors="replace") or "the C interface failed without a message"

    # ---- caches ---------------------------------------------------------------------------------------
    def create_kv_cache(self) -> int:
        return self.lib.jkCreateKVCache(self.handle)

    def duplicate_kv_cache(self, cache: int, seq_len: int) -> int:
        c = self.lib.jkDuplicateKVCache(self.handle, cache, seq_len)
        if not c:
            raise NativeModelError(self._message())
        return c

    def drop_kv_cache(self, cache: int) -> None:
        self.lib.jkDropKVCache(self.handle, cache)

    @property
    def free_pages(self) -> int:
        return self.lib.jkFreePages(self.handle)

    @property
    def last_launches(self) -> int:
        return self.lib.jkLastLaunches(self.handle)

    # ---- batches --------------------------------------------------------------------------------------
    def _batch(self, tokens: Sequence[Sequence[int]], positions: Sequence[int], caches: Sequence[int]):
        flat = _u32([t for ts in tokens for t in ts])
        lens, pos = _u32([len(ts) for ts in tokens]), _u32(positions)
        handles = (ctypes.c_void_p * len(caches))(*caches)
        return flat, lens, pos, handles

    def forward_batch(self, tokens: Sequence[Sequence[int]], positions: Sequence[int], caches: Sequence[int]) -> np.ndarray:
        """float32 logits of every row, ``[total tokens, vocab]``."""
        flat, lens, pos, handles = self._batch(tokens, positions, caches)
        out = np.empty((flat.size, self.vocab_size), dtype=np.float32)
        rc = self.lib.jkForwardBatch(ctypes.c_void_p(self.handle), _ptr(flat, ctypes.c_uint32), ctypes.c_uint32(flat.size),
                                     _ptr(lens, ctypes.c_uint32), ctypes.c_uint32(len(caches)), _ptr(pos, ctypes.c_uint32),
                                     handles, _ptr(out, ctypes.c_float))
        if rc:
            raise NativeModelError(self._message())
        return out

    def infer_batch(self, tokens: Sequence[Sequence[int]], positions: Sequence[int], caches: Sequence[int],
                    temperature: Optional[Sequence[float]] = None, topk: Optional[Sequence[int]] = None,
                    topp: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None) -> List[int]:
        """One new token per request."""
        flat, lens, pos, handles = self._batch(tokens, positions, caches)
        n = len(caches)
        temp = np.ascontiguousarray(np.asarray(temperature if temperature is not None else [0.0] * n, dtype=np.float32))
        k = _u32(topk if topk is not None else [0] * n)
        p = np.ascontiguousarray(np.asarray(topp if topp is not None else [1.0] * n, dtype=np.float32))
        s = np.ascontiguousarray(np.asarray(seeds if seeds is not None else [0] * n, dtype=np.uint64))
        out = np.zeros(n, dtype=np.uint32)
        rc = self.lib.jkInferBatch(ctypes.c_void_p(self.handle), _ptr(flat, ctypes.c_uint32), ctypes.c_uint32(flat.size),
                                   _ptr(lens, ctypes.c_uint32), ctypes.c_uint32(n), _ptr(pos, ctypes.c_uint32), handles,
                                   _ptr(temp, ctypes.c_float), _ptr(k, ctypes.c_uint32), _ptr(p, ctypes.c_float),
                                   _ptr(s, ctypes.c_uint64), _ptr(out, ctypes.c_uint32))
        if rc:
            raise NativeModelError(self._message())
        return [int(t) for t in out]

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.jkDestroyModel(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
