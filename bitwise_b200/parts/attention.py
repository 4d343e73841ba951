"""Grouped-query attention with rotary positions over the paged cache.

Per step (src/model.cpp:281-300): the fused projection ``[q | k | v] = xn Wqkv^T`` (rows
of q_proj, k_proj, v_proj stacked in this order, src/model.cpp:150-153), rotation of q
and k, the write of k and v of EVERY row of the step into the cache, then attention that
reads only the cache (also for the step's own rows, which is what makes a row's result
independent of how the prompt was cut), the output projection and the residual sum.
Head h reads key/value head ``h // (heads / kv_heads)`` (src/kernels.cpp:346,361); the
score scale ``1 / sqrt(head_dim)`` is applied after the dot product (src/kernels.cpp:319,347).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..weights.loader import MATRIX, ParamSpec
from .base import Mixer, PagedKVNeed, PagedKVView, PositionEncoding, StepContext, register_mixer


class GQAAttention(Mixer):
    # Kernels only.  What forward and the launchers decide on the host depends on the step's
    # sizes (rows, sequences, query tiles) and on ctx.max_keys, the rounded bound on the context;
    # the stepper keeps a captured step under exactly these.
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int,
                 position: Optional[PositionEncoding] = None, window: Optional[int] = None,
                 names=("q_proj", "k_proj", "v_proj", "o_proj")):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key/value heads")
        if head_dim % 16:
            raise ValueError(f"head size {head_dim} is not a multiple of 16 (the kernels' step)")
        self.width, self.heads, self.kv_heads, self.head_dim = width, heads, kv_heads, head_dim
        self.q_dim, self.kv_dim = heads * head_dim, kv_heads * head_dim
        self.position = position
        self.window = window
        self.names = names
        self.scale = 1.0 / math.sqrt(head_dim)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.head_dim, self.window)

    def query_tile_rows(self, ops=None):
        """Heights of the query tiles this mixer's attention kernels want (rows of one sequence
        per thread block); the stepper prepares tiles of every height asked for."""
        if ops is not None and hasattr(ops, "attention_tile_heights"):
            return list(ops.attention_tile_heights(self.heads, self.kv_heads, self.head_dim))
        return [max(1, 64 // (self.heads // self.kv_heads))]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        q, k, v, o = self.names
        return [ParamSpec(f"{prefix}.{q}.weight", (self.q_dim, self.width), MATRIX),
                ParamSpec(f"{prefix}.{k}.weight", (self.kv_dim, self.width), MATRIX),
                ParamSpec(f"{prefix}.{v}.weight", (self.kv_dim, self.width), MATRIX),
                ParamSpec(f"{prefix}.{o}.weight", (self.width, self.q_dim), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        q, k, v, o = self.names
        self.w_qkv = torch.cat([state[f"{prefix}.{q}.weight"], state[f"{prefix}.{k}.weight"],
                                state[f"{prefix}.{v}.weight"]], dim=0).contiguous()
        self.w_o = state[f"{prefix}.{o}.weight"]

    def param_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, cache: PagedKVView) -> None:
        ops, n = ctx.ops, ctx.n
        qkv = ctx.workspace.rows("qkv", n, self.q_dim + 2 * self.kv_dim, ctx.act_dtype)
        tables = self.position.rotary_tables(x.device) if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        fuses = getattr(ops, "fuses_rope", None)
        if fuses and fuses(n, self.width, self.heads, self.kv_heads, self.head_dim):
            # a step of few rows: the projection rotates and stores its outputs itself
            ops.linear_rope_cache(xn, self.w_qkv, qkv, ctx.pos, ctx.row_seq, cos, sin, cache.block_table, cache.k,
                                  cache.v, self.heads, self.kv_heads, self.head_dim, write_kv=cache.writable)
        else:
            ops.linear(xn, self.w_qkv, qkv)
            ops.rope_cache(qkv, ctx.pos, ctx.row_seq, cos, sin, cache.block_table, cache.k, cache.v,
                           self.heads, self.kv_heads, self.head_dim, write_kv=cache.writable)
        attn = ctx.workspace.rows("attn", n, self.q_dim, ctx.act_dtype)
        ops.attention(qkv, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.pos, attn, self.heads,
                      self.kv_heads, self.head_dim, self.window or 0, ctx.max_keys, self.scale, batch=ctx)
        ops.linear(attn, self.w_o, x, residual=x)


register_mixer("gqa_attention", GQAAttention)
