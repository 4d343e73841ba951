"""Token embedding and output head.

Embedding: a row copy, widened to the 32-bit stream (src/model.cpp:233-239,274); no
scaling of embeddings.  Head: gather the rows whose logits are wanted, final norm on those
rows only, one product with lm_head, or with the embedding table when the model ties them
(src/model.cpp:170-171,308-321); logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import MATRIX, ParamSpec
from .base import Norm, Part, StepContext


class TokenEmbedding(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, vocab: int, width: int, name: str = "embed_tokens"):
        self.vocab, self.width, self.name = vocab, width, name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [ParamSpec(f"{prefix}.{self.name}.weight", (self.vocab, self.width), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        self.table = state[f"{prefix}.{self.name}.weight"]

    def param_bytes(self) -> int:
        return self.table.numel() * self.table.element_size()

    def forward(self, ctx: StepContext, x: torch.Tensor) -> None:
        ctx.ops.embed_rows(self.table, ctx.tokens, x)


class OutputHead(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, vocab: int, width: int, norm: Norm, tied_to: Optional[TokenEmbedding] = None,
                 norm_name: str = "model.norm", head_name: str = "lm_head"):
        self.vocab, self.width = vocab, width
        self.norm, self.tied_to = norm, tied_to
        self.norm_name, self.head_name = norm_name, head_name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str = "") -> List[ParamSpec]:
        specs = self.norm.param_specs(self.norm_name)
        if self.tied_to is None:
            specs.append(ParamSpec(f"{self.head_name}.weight", (self.vocab, self.width), MATRIX))
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str = "") -> None:
        self.norm.load_params(state, self.norm_name)
        self.weight = self.tied_to.table if self.tied_to is not None else state[f"{self.head_name}.weight"]

    def param_bytes(self) -> int:
        own = 0 if self.tied_to is not None else self.weight.numel() * self.weight.element_size()
        return own + self.norm.param_bytes()

    def forward(self, ctx: StepContext, x: torch.Tensor) -> Optional[torch.Tensor]:
        c = ctx.num_logit_rows
        if c == 0:
            return None
        last = ctx.workspace.rows("head_in", c, self.width, ctx.act_dtype)
        self.norm.forward(ctx, x, last, rows=ctx.logit_rows)
        logits = ctx.workspace.rows("logits", c, self.vocab, torch.float32, growable=True)
        ctx.ops.linear(last, self.weight, logits)
        return logits
