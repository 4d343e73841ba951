"""A decoder assembled from parts: embedding, a list of blocks, a run order, a head.

``blocks`` holds the layers (each with weights of its own).  ``schedule`` is the order in
which they run, as data: a list of :class:`LayerRun`.  A run names the block it executes
and the cache entry it uses; a block may appear in several runs, and a run may use the
cache entry that an earlier run owns (it then reads that cache and stores nothing).  The
plain Llama stack of the reference (src/model.cpp:279-306) is the schedule
``[run(0), run(1), ...]`` with one cache entry per run.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import PositionEncoding, StepContext
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights.loader import ParamSpec


@dataclass(frozen=True)
class LayerRun:
    block: int   # index into DecoderModel.blocks
    cache: int   # index of the cache entry this run uses
    owns_cache: bool = True  # False: reads an entry that another run writes


def sequential_schedule(num_layers: int) -> List[LayerRun]:
    return [LayerRun(i, i, True) for i in range(num_layers)]


class DecoderModel:
    def __init__(self, config, embedding: TokenEmbedding, blocks: Sequence, head: OutputHead,
                 schedule: Optional[Sequence[LayerRun]] = None,
                 position_encodings: Sequence[PositionEncoding] = (),
                 block_prefix: str = "model.layers.{}", embed_prefix: str = "model"):
        self.config = config
        self.embedding = embedding
        self.blocks = list(blocks)
        self.head = head
        self.schedule = list(schedule) if schedule is not None else sequential_schedule(len(self.blocks))
        self.position_encodings = list(position_encodings)
        self.block_prefix, self.embed_prefix = block_prefix, embed_prefix
        self.dtype: Optional[str] = None
        self.device = None
        self._check_schedule()

    def _check_schedule(self) -> None:
        owners: Dict[int, int] = {}
        for i, run in enumerate(self.schedule):
            if not (0 <= run.block < len(self.blocks)):
                raise ValueError(f"run {i} names block {run.block}; the model has {len(self.blocks)}")
            if run.owns_cache:
                if run.cache in owners:
                    raise ValueError(f"cache entry {run.cache} is owned by runs {owners[run.cache]} and {i}")
                owners[run.cache] = i
        for i, run in enumerate(self.schedule):
            if not run.owns_cache:
                if run.cache not in owners or owners[run.cache] > i:
                    raise ValueError(f"run {i} reads cache entry {run.cache}, which no earlier run owns")
                a = self.blocks[self.schedule[owners[run.cache]].block].cache_need()
                b = self.blocks[run.block].cache_need()
                if a != b:
                    raise ValueError(f"run {i} reads a cache of another shape ({b} vs {a})")
        self.cache_entries = sorted(owners)
        if self.cache_entries != list(range(len(self.cache_entries))):
            raise ValueError("cache entries must be numbered 0..n-1 without gaps")

    # -- what the cache manager needs to know -----------------------------------------
    def cache_needs(self) -> List[object]:
        """The need of every cache entry, indexed by entry."""
        needs = [None] * len(self.cache_entries)
        for run in self.schedule:
            if run.owns_cache:
                needs[run.cache] = self.blocks[run.block].cache_need()
        return needs

    # -- parameters --------------------------------------------------------------------
    def param_specs(self) -> List[ParamSpec]:
        specs = self.embedding.param_specs(self.embed_prefix)
        for pe in self.position_encodings:  # encodings with weights of their own (a learned table)
            specs += pe.param_specs(self.embed_prefix)
        for i, b in enumerate(self.blocks):
            specs += b.param_specs(self.block_prefix.format(i))
        specs += self.head.param_specs()
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], dtype: str, device) -> None:
        self.embedding.load_params(state, self.embed_prefix)
        for pe in self.position_encodings:
            pe.load_params(state, self.embed_prefix)
        for i, b in enumerate(self.blocks):
            b.load_params(state, self.block_prefix.format(i))
        self.head.load_params(state)
        self.dtype, self.device = dtype, device

    def ignorable_tensor(self, name: str) -> bool:
        """Stored tensors that the model has no use for: the rotary tables that older exports
        keep as buffers (the engine builds its own from the configuration)."""
        return name.endswith(".rotary_emb.inv_freq")

    def tensor_aliases(self) -> Dict[str, str]:
        """Stored name -> declared tensor it must repeat: a tied head stored a second time."""
        if self.head.tied_to is not None:
            return {f"{self.head.head_name}.weight": f"{self.embed_prefix}.{self.head.tied_to.name}.weight"}
        return {}

    def prepare(self, ops) -> None:
        """Let every part lay out its weights for the kernel library it will run on."""
        for b in self.blocks:
            b.prepare(ops)

    def param_bytes(self) -> int:
        return (self.embedding.param_bytes() + sum(b.param_bytes() for b in self.blocks) + self.head.param_bytes()
                + sum(pe.param_bytes() for pe in self.position_encodings))

    def graph_safe(self) -> bool:
        """True when every part only launches kernels in forward and decides nothing on the host
        beyond what the step's sizes and ``ctx.max_keys`` determine, so that a step's launches
        can be captured into a CUDA graph and replayed for steps with the same sizes."""
        parts = [self.embedding, self.head, self.head.norm] + list(self.position_encodings)
        for b in self.blocks:
            parts += [b, b.mixer, b.feed_forward, b.mixer_norm, b.ffn_norm]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def reserve_positions(self, positions: int) -> None:
        for pe in self.position_encodings:
            if hasattr(pe, "reserve"):
                pe.reserve(positions)

    # -- one step ----------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache_views: Sequence[object]) -> Optional[torch.Tensor]:
        """Run the step's rows through every scheduled layer; returns float32 logits
        [wanted rows, vocab] or None.  ``cache_views[e]`` is the view of cache entry e."""
        x = ctx.workspace.rows("stream", ctx.n, self.embedding.width, torch.float32)
        self.embedding.forward(ctx, x)
        for pe in self.position_encodings:
            pe.on_embed(ctx, x)
        for run in self.schedule:
            view = cache_views[run.cache]
            if not run.owns_cache and hasattr(view, "writable"):
                view = type(view)(**{**view.__dict__, "writable": False})
            self.blocks[run.block].forward(ctx, x, view)
        return self.head.forward(ctx, x)
