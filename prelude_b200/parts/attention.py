"""Grouped-query softmax attention over a paged key/value cache.

One merged q/k/v projection, optional per-head RMSNorm of q and k, the position
encoding, the write of k and v into the layer's pages, attention over the
pages, and the output projection
(crates/prelude-core/src/models/qwen3.rs:45-131 for the shapes and the merged
projection, 161-231 for the order of operations).  The inner width is
num_heads * head_dim, which need not equal the hidden size (qwen3.rs:54-57).

With ``write_cache=False`` the call projects q only and reads the pages that an
earlier layer wrote.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import AttentionSpec
from ..ops import kernels as K
from ..ops.attention import paged_attention
from ..ops.linear import linear, qkv_heads
from ..weights.loader import TensorReq
from .registry import KvPagesNeed, RunContext, make_part, register_part


@register_part("mixer", "attention")
class Attention:
    def __init__(self, spec: AttentionSpec, prefix: str):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not divide over {spec.num_kv_heads} key/value heads")
        self.spec, self.prefix = spec, prefix
        self.position = make_part("position", spec.position, prefix)
        self.q_cols = spec.num_heads * spec.head_dim
        self.kv_cols = spec.num_kv_heads * spec.head_dim
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_norm = self.k_norm = None

    def parts(self):
        return (self.position,)

    # -- weights ----------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {
            f"{p}.q_proj.weight": TensorReq((self.q_cols, s.hidden_size)),
            f"{p}.k_proj.weight": TensorReq((self.kv_cols, s.hidden_size)),
            f"{p}.v_proj.weight": TensorReq((self.kv_cols, s.hidden_size)),
            f"{p}.o_proj.weight": TensorReq((s.hidden_size, self.q_cols)),
        }
        if s.bias:
            req.update({
                f"{p}.q_proj.bias": TensorReq((self.q_cols,), "bias"),
                f"{p}.k_proj.bias": TensorReq((self.kv_cols,), "bias"),
                f"{p}.v_proj.bias": TensorReq((self.kv_cols,), "bias"),
                f"{p}.o_proj.bias": TensorReq((s.hidden_size,), "bias"),
            })
        if s.qk_norm_eps is not None:
            req[f"{p}.q_norm.weight"] = TensorReq((s.head_dim,), "norm")
            req[f"{p}.k_norm.weight"] = TensorReq((s.head_dim,), "norm")
        req.update(self.position.tensors())
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        # q, k and v rows one below the other: one product instead of three (qwen3.rs:89-106)
        self.w_qkv = torch.cat([mat("q_proj.weight"), mat("k_proj.weight"), mat("v_proj.weight")], dim=0).contiguous()
        self.w_o = mat("o_proj.weight").contiguous()
        if s.bias:
            self.b_qkv = torch.cat([vec("q_proj.bias"), vec("k_proj.bias"), vec("v_proj.bias")]).contiguous()
            self.b_o = vec("o_proj.bias")
        if s.qk_norm_eps is not None:
            self.q_norm, self.k_norm = vec("q_norm.weight"), vec("k_norm.weight")
        self.position.load(get, ctx)

    def activation_bytes_per_token(self, elem: int) -> int:
        """The merged projection, q, the attention output (twice: the layers share one buffer, a step keeps one)."""
        return (2 * self.q_cols + 2 * self.kv_cols + 2 * self.q_cols) * elem + self.spec.hidden_size * elem

    # -- cache ------------------------------------------------------------------
    def cache_need(self) -> KvPagesNeed:
        return KvPagesNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    # -- one step -----------------------------------------------------------------
    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        table = batch.block_tables[cache.group]
        # the projection, the per-head norms, the rotation and the cache write: one call, which for a prompt step's
        # many rows is one kernel (the product with the rest in its epilogue), else the product and a kernel behind it
        q = qkv_heads(
            x, self.w_qkv, self.b_qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm, self.k_norm,
            s.qk_norm_eps if s.qk_norm_eps is not None else 0.0, self.position.cos, self.position.sin,
            self.position.rotary_dim, bool(getattr(self.position, "interleaved", False)), batch.positions,
            batch.table_row_of_token, table, cache.k_pages, cache.v_pages, write_cache, batch.status,
            out=batch.workspace("attention_q", (batch.n_tokens, s.num_heads, s.head_dim), x.dtype))
        o = paged_attention(q, cache.k_pages, cache.v_pages, batch, cache.group, s.softmax_scale, s.window,
                            out=batch.workspace("attention_out", (batch.n_tokens, s.num_heads, s.head_dim), x.dtype))
        return linear(o.view(batch.n_tokens, self.q_cols), self.w_o, self.b_o)
