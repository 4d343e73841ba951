"""The arrangement of a layer: pre-norm residual block.

``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:281-305).  The
block owns nothing but its four parts and the sub-names under which their tensors are
found; which mixer and which feed-forward it holds is decided where the model is assembled,
layer by layer.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights.loader import ParamSpec
from .base import FeedForward, Mixer, Norm, Part, StepContext


class PreNormBlock(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm,
                 names: Dict[str, str]):
        self.width = width
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.names = names  # keys: mixer_norm, mixer, ffn_norm, feed_forward

    def _children(self, prefix: str):
        return [(self.mixer_norm, f"{prefix}.{self.names['mixer_norm']}"),
                (self.mixer, f"{prefix}.{self.names['mixer']}"),
                (self.ffn_norm, f"{prefix}.{self.names['ffn_norm']}"),
                (self.feed_forward, f"{prefix}.{self.names['feed_forward']}")]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [s for part, p in self._children(prefix) for s in part.param_specs(p)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        for part, p in self._children(prefix):
            part.load_params(state, p)

    def param_bytes(self) -> int:
        return sum(part.param_bytes() for part, _ in self._children(""))

    def cache_need(self):
        return self.mixer.cache_need()

    def prepare(self, ops) -> None:
        for part, _ in self._children(""):
            part.prepare(ops)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        """Run the block on the float32 stream ``x`` in place."""
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        self.mixer_norm.forward(ctx, x, xn)
        self.mixer.forward(ctx, xn, x, cache)
        self.ffn_norm.forward(ctx, x, xn)
        self.feed_forward.forward(ctx, xn, x)
