"""The dense SwiGLU feed-forward: ``h = silu(xn Wg^T) * (xn Wu^T)``, ``x += h Wd^T``
(src/model.cpp:301-305; src/kernels.cpp:291-298).  gate_proj and up_proj are stacked by
rows into one matrix so that one product yields rows laid out [gate | up]
(src/model.cpp:162-164).  SiLU is the only activation the reference has; no biases."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import MATRIX, ParamSpec
from .base import FeedForward, StepContext, register_feed_forward


class SwiGLU(FeedForward):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, intermediate: int, names=("gate_proj", "up_proj", "down_proj")):
        self.width, self.intermediate = width, intermediate
        self.names = names
        self.w_gate_up: Optional[torch.Tensor] = None  # rows [gate | up], or interleaved when fused
        self.w_down: Optional[torch.Tensor] = None
        self.fused = False  # gate/up product and SwiGLU in one kernel

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        g, u, d = self.names
        return [ParamSpec(f"{prefix}.{g}.weight", (self.intermediate, self.width), MATRIX),
                ParamSpec(f"{prefix}.{u}.weight", (self.intermediate, self.width), MATRIX),
                ParamSpec(f"{prefix}.{d}.weight", (self.width, self.intermediate), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        g, u, d = self.names
        self.w_gate_up = torch.cat([state[f"{prefix}.{g}.weight"], state[f"{prefix}.{u}.weight"]], 0).contiguous()
        self.w_down = state[f"{prefix}.{d}.weight"]

    def param_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def prepare(self, ops) -> None:
        """Kernels that apply SwiGLU in the epilogue of the gate/up product want the two
        matrices interleaved in blocks of 64 rows."""
        if not self.fused and getattr(ops, "fuses_swiglu", None) and ops.fuses_swiglu(self.width, self.intermediate):
            gate, up = self.w_gate_up[:self.intermediate], self.w_gate_up[self.intermediate:]
            self.w_gate_up = ops.interleave_gate_up(gate, up)
            self.fused = True

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor) -> None:
        ops, n = ctx.ops, ctx.n
        h = ctx.workspace.rows("ffn_h", n, self.intermediate, ctx.act_dtype)
        if self.fused:
            ops.linear_swiglu(xn, self.w_gate_up, h)
        else:
            gate_up = ctx.workspace.rows("gate_up", n, 2 * self.intermediate, ctx.act_dtype)
            ops.linear(xn, self.w_gate_up, gate_up)
            ops.swiglu(gate_up, h)
        ops.linear(h, self.w_down, x, residual=x)


register_feed_forward("swiglu", SwiGLU)
