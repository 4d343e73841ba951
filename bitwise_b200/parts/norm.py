"""RMSNorm: y = (x * inv) * w, inv = 1 / sqrt(mean(x^2) + eps), no offset on the weight
(src/kernels.cpp:264-271).  The statistic is always computed in 32-bit."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, ParamSpec
from .base import Norm, StepContext, register_norm


class RMSNorm(Norm):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, eps: float):
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [ParamSpec(prefix + ".weight", (self.width,), KEEP32, init="ones")]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        self.weight = state[prefix + ".weight"]

    def param_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx: StepContext, x, out, rows=None) -> None:
        ctx.ops.rmsnorm(x, self.weight, self.eps, out, rows)


register_norm("rmsnorm", RMSNorm)
