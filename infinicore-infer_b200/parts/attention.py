"""Causal softmax attention over the paged cache: the mixer of this architecture.

Per layer, in the reference's order (src/models/jiuge/jiuge.cpp:200-236): the fused
query/key/value product, rotary encoding of query and key heads, keys and values into the
cache at the rows' positions, softmax(q k^T / sqrt(dh)) v over the request's cached
positions under the causal mask, then the output product.  Query head h reads key/value
head h // (num_heads / num_kv_heads) (jiuge.cpp:210-211).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import PagedKV
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import part_class, register


@register("mixer", "attention")
class Attention:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, q, kv = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        decls = {
            "q_proj.weight": TensorDecl((q, d)), "k_proj.weight": TensorDecl((kv, d)),
            "v_proj.weight": TensorDecl((kv, d)), "o_proj.weight": TensorDecl((d, q)),
        }
        if spec.bias:
            decls.update({"q_proj.bias": TensorDecl((q,), VECTOR), "k_proj.bias": TensorDecl((kv,), VECTOR),
                          "v_proj.bias": TensorDecl((kv,), VECTOR)})
        return decls

    @staticmethod
    def cache_need(spec):
        return PagedKV(spec.num_kv_heads, spec.head_dim, spec.window)

    @staticmethod
    def pack(spec, weights, prefix: str) -> Dict[str, Optional[torch.Tensor]]:
        """The layer's tensors as the kernels take them: one fused [q | k | v] matrix with the checkpoint's rows
        in the checkpoint's order (scripts/jiuge.py:217-240 concatenates the same way, but also permutes the rows
        of q and k inside each head for its adjacent-pair rotary operator; here the rows stay and the rotation pairs
        row j with row j + head_dim/2, which is the same function), the output matrix, the fused bias or None.
        Every holder of these weights (this part, the C interface's wrapper) packs through this one function."""
        out = {"w_qkv": weights.get_rows([prefix + n + "_proj.weight" for n in "qkv"], MATRIX),
               "w_o": weights.get(prefix + "o_proj.weight", MATRIX), "b_qkv": None}
        if spec.bias:
            out["b_qkv"] = weights.get_rows([prefix + n + "_proj.bias" for n in "qkv"], VECTOR)
        return out

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        packed = self.pack(spec, weights, prefix)
        self.w_qkv, self.w_o, self.b_qkv = packed["w_qkv"], packed["w_o"], packed["b_qkv"]
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, weights, prefix, runtime)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    # ---- work lists: what this mixer asks every step to carry -----------------------------------------------------
    # Requests that bring few rows to a step go to the split-key decode kernels row by row, the others to the prefill
    # kernels in tiles of query rows; the rule and the numbers are jk::attention_work_lists of csrc/host_rules.h.
    LISTS = ("short_rows", "tiles")

    @staticmethod
    def step_list_capacity(T: int, B: int) -> Dict[str, int]:
        from ..kernels import host
        short, tiles = host.attention_list_capacity(T, B)
        return {"short_rows": short, "tiles": tiles}

    @staticmethod
    def fill_step_lists(B: int, pad_B: int, lens, starts, arrays) -> Dict[str, tuple]:
        """Fill ``arrays[name]`` (int32 numpy views of the step's metadata buffer); returns name -> (entries, whether
        the list is simply the rows 0..entries-1, which the kernels take without a list)."""
        from ..kernels import host
        n_short, n_tiles = host.attention_work_lists(B, pad_B, lens, starts, arrays["short_rows"], arrays["tiles"])
        rows = sum(lens) + (pad_B - B)
        return {"short_rows": (n_short, n_short == rows), "tiles": (n_tiles, False)}

    def plan(self, program, view, writes_cache: bool = True, residual_scale: float = 1.0) -> None:
        """Three records: the fused q | k | v product with rotation and cache write (h -> q), the attention over the
        cache (q -> o), the output product added into the stream times ``residual_scale``."""
        import ctypes
        s, pos = self.spec, self.position
        i, f, p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
        short, tiles = program.work_lists(Attention, self.LISTS)
        ptr = lambda t: p(t.data_ptr() if t is not None else 0)
        max_positions = getattr(pos, "max_positions", None) or (pos.cos.shape[0] if pos is not None else 1 << 20)
        program.emit("jk_emit_attention", ptr(self.w_qkv), ptr(self.b_qkv), ptr(self.w_o), i(s.hidden_size), i(s.num_heads),
                     i(s.num_kv_heads), i(s.head_dim), i(s.window or 0), f(s.softmax_scale), f(residual_scale),
                     ptr(pos.cos if pos is not None else None), ptr(pos.sin if pos is not None else None),
                     i(1 if (pos is not None and pos.interleaved) else 0), i(max_positions), ptr(view.k_pages), ptr(view.v_pages),
                     i(view.k_pages.shape[0]), i(view.group_index), i(1 if writes_cache else 0), i(short), i(tiles),
                     keep=(self.w_qkv, self.b_qkv, self.w_o, pos, view.k_pages, view.v_pages))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]`` (the output product, not yet scaled)."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan(program, view, writes_cache, 1.0), ctx, h,
                              self.spec.hidden_size, page_size=view.page_size)
