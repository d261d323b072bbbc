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

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        from .. import kernels
        s, rt = self.spec, self.runtime
        T = ctx.ntok
        q = rt.empty(T, s.num_heads * s.head_dim)
        table = ctx.block_tables[view.group_index]
        pos = self.position
        n, k = self.w_qkv.shape
        # the product's epilogue can rotate and write q and the cache itself: no float32 copy of the
        # product, no rotary kernel (the tcgen05 kernel for many rows, the small-row kernel for few)
        fusable = (rt.dtype == torch.bfloat16 and self.b_qkv is None and writes_cache
                   and not (pos and pos.interleaved) and not rt.library_products_only)
        if fusable and rt.takes_tcgen05(T, n, k) and kernels.gemm_tcgen05_qkv_supports(s.head_dim):
            kernels.gemm_tcgen05_qkv(h, self.w_qkv, q, view.k_pages, view.v_pages, pos.cos if pos else None,
                                     pos.sin if pos else None, ctx.positions, ctx.row_req, table, s.num_heads)
        elif fusable and T <= 16 and kernels.linear_small_qkv_supports(T, k, s.head_dim):
            kernels.linear_small_qkv(h, self.w_qkv, q, view.k_pages, view.v_pages, pos.cos if pos else None,
                                     pos.sin if pos else None, ctx.positions, ctx.row_req, table, s.num_heads)
        else:
            qkv = rt.linear(h, self.w_qkv, out_dtype=torch.float32)
            kernels.rope_kv(qkv, self.b_qkv, ctx.positions, ctx.row_req, table, view.page_size,
                            pos.cos if pos else None, pos.sin if pos else None,
                            pos.interleaved if pos else False, q, view.k_pages, view.v_pages,
                            T, s.num_heads, s.num_kv_heads, s.head_dim, write_cache=writes_cache)
        o = rt.empty(T, s.num_heads * s.head_dim)
        self._attend(q, o, view, table, ctx)
        return rt.product(o, self.w_o)       # the block adds it to the residual stream

    def _attend(self, q, o, view, table, ctx) -> None:
        """float32: one warp per (row, head), the same arithmetic whatever the batch.  bfloat16: rows of
        requests with few rows go to the split-key decode kernel, tiles of the others to a tensor-core
        kernel (tcgen05 where it is built for the head and page size, else mma.sync); head sizes neither
        is built for take the row kernel."""
        from .. import kernels
        s, T = self.spec, ctx.ntok
        fast = (self.runtime.dtype == torch.bfloat16 and not self.runtime.plain_attention
                and (ctx.n_short or ctx.n_tiles) and s.head_dim % 8 == 0 and s.head_dim <= 256)
        if fast and ctx.n_tiles and not (kernels.attention_prefill_supports(s.head_dim)
                                         or kernels.attention_tcgen05_supports(s.head_dim, view.page_size)):
            fast = False
        if not fast:
            kernels.attention_rows(q, view.k_pages, view.v_pages, o, ctx.positions, ctx.row_req, table, T,
                                   s.num_heads, s.softmax_scale, s.window or 0)
            return
        if ctx.n_tiles:
            if not self.runtime.legacy_tensor_cores and kernels.attention_tcgen05_supports(s.head_dim, view.page_size):
                kernels.attention_tcgen05(q, view.k_pages, view.v_pages, o, ctx.tiles, ctx.n_tiles, T, ctx.req_start,
                                          ctx.req_pos, table, s.num_heads, s.softmax_scale, s.window or 0)
            else:
                kernels.attention_prefill(q, view.k_pages, view.v_pages, o, ctx.tiles, ctx.n_tiles, ctx.req_start,
                                          ctx.req_pos, table, s.num_heads, s.softmax_scale, s.window or 0)
        if ctx.n_short:
            splits = kernels.attention_decode_splits(ctx.n_short, s.num_kv_heads, s.num_heads // s.num_kv_heads,
                                                     s.window or (s.position.max_positions if s.position else 1 << 20),
                                                     kernels._sm_count(q.device), s.head_dim)
            kernels.attention_decode(q, view.k_pages, view.v_pages, o, ctx.short_rows, ctx.n_short, ctx.positions,
                                     ctx.row_req, table, s.num_heads, s.softmax_scale, s.window or 0, splits)
