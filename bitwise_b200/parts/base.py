"""What a part is, and what a step hands to it.

A model is put together from parts: a mixer (attention here), a feed-forward, norms, a
position encoding, arranged in a block.  A part gets every size and constant through its
constructor, declares the tensors it needs (``param_specs``), takes them
(``load_params``), says what cache it needs (``cache_need``), and runs on the rows of a
step (``forward``).  No part knows which model it is in: names of checkpoint tensors
are given to it as a prefix, and the step's data arrive in a :class:`StepContext`.

The reference has one fixed decoder (src/model.cpp:267-322); the split into parts is this
package's own, so that another mixer or feed-forward can be added beside the present ones.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..weights.loader import ParamSpec


# ---------------------------------------------------------------------------------------
# cache needs

@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values that grow with the position, kept in pages.
    ``window`` = None keeps every key; an integer keeps the last ``window`` positions."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotStateNeed:
    """State of fixed size per request, one slot each: ``shape`` elements of ``dtype``.
    A slot is handed out as the request that held it before left it: the mixer starts its state
    itself at a request's first position (``seq_pos0 == 0``), as pages are not cleared either."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------------------------------
# what a step gives to the parts

@dataclass
class PagedKVView:
    """The cache of one layer run, as a mixer sees it during a step."""
    k: torch.Tensor            # [pages, kv_heads, page, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # int32 [step sequences, max blocks] of the layer's group
    page_size: int
    writable: bool = True      # False: the run reads another run's cache and stores nothing


@dataclass
class SlotStateView:
    state: torch.Tensor        # [slots, *shape]
    seq_slot: torch.Tensor     # int32 [step sequences]


class Workspace:
    """Named scratch tensors with fixed addresses, sized once for the largest step."""

    def __init__(self, device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self._buffers: Dict[str, torch.Tensor] = {}

    def rows(self, name: str, n: int, width: int, dtype: torch.dtype, growable: bool = False) -> torch.Tensor:
        """A [n, width] view of the buffer ``name``.  Fixed buffers are allocated
        [max_rows, width] on first use and never move; a ``growable`` one starts small and
        is replaced by a larger one when a step needs more rows (logits of many positions)."""
        key = f"{name}:{width}:{dtype}"
        buf = self._buffers.get(key)
        if n > self.max_rows:
            raise ValueError(f"step of {n} rows exceeds the workspace of {self.max_rows} rows")
        if buf is None or buf.shape[0] < n:
            cap = self.max_rows
            if growable:
                cap = 8
                while cap < n:
                    cap *= 2
                cap = min(cap, self.max_rows)
            buf = torch.empty((cap, width), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:n]

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    """One step's batch as device arrays, plus the kernel library and scratch space.

    Rows of one sequence are contiguous and in increasing position (src/model.h:78-85).
    """
    ops: object
    workspace: Workspace
    n: int                       # rows (tokens) in this step
    num_seqs: int
    tokens: torch.Tensor         # int32 [n]
    pos: torch.Tensor            # int32 [n] absolute position of each row
    row_seq: torch.Tensor        # int32 [n] index of the row's sequence in this step
    seq_row0: torch.Tensor       # int32 [num_seqs + 1] first row of each sequence
    seq_pos0: torch.Tensor       # int32 [num_seqs] position of each sequence's first row
    seq_slot: torch.Tensor       # int32 [num_seqs] state slot of each sequence
    logit_rows: torch.Tensor     # int32 [c] rows whose logits are wanted
    num_logit_rows: int
    max_keys: int                # bound on pos + 1 over the step's rows, rounded up to ops.key_granule:
                                 # for sizing launches on the host; rows are bounded by ``pos`` on the device
    # query tiles for kernels that tile rows by sequence (sequence, first row, row count)
    tile_seq: Optional[torch.Tensor] = None
    tile_row0: Optional[torch.Tensor] = None
    tile_rows: Optional[torch.Tensor] = None
    num_tiles: int = 0
    # host copies, for parts written without kernels of their own
    host_seq_rows: List[Tuple[int, int]] = field(default_factory=list)  # (first row, rows)
    host_seq_pos0: List[int] = field(default_factory=list)
    host_seq_slot: List[int] = field(default_factory=list)
    # filled by the stepper: query tiles by tile height, and the device block table of each group
    tile_sets: Dict[int, tuple] = field(default_factory=dict)
    block_tables: List[torch.Tensor] = field(default_factory=list)
    cache_views: List[object] = field(default_factory=list)  # one per cache entry, as the model's forward takes them
    wanted_rows: int = 0         # of num_logit_rows, how many belong to requests (the stepper may add rows of no request)

    def query_tiles(self, rows_per_tile: int):
        """(tile_seq, tile_row0, tile_rows, count) for tiles of at most ``rows_per_tile`` rows."""
        return self.tile_sets[rows_per_tile]

    @property
    def act_dtype(self) -> torch.dtype:
        return self.ops.act_dtype


# ---------------------------------------------------------------------------------------
# the interfaces

class Part:
    """Common to every part: parameters by name."""

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return []

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        pass

    def param_bytes(self) -> int:
        return 0

    def prepare(self, ops) -> None:
        """Called once after the parameters are loaded, with the kernel library the model
        will run on: a part may lay its weights out the way those kernels want them."""
        pass


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = norm(x[rows[r]] if rows is given else x[r]); x is the float32 stream."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter the model.  ``on_embed`` may add to the stream after the token
    embedding; ``rotary_tables`` gives (cos, sin) float32 tables [positions, head_dim/2]
    for mixers that rotate queries and keys, or None."""

    def on_embed(self, ctx: StepContext, x: torch.Tensor) -> None:
        pass

    def rotary_tables(self, device):
        return None

    def max_positions(self) -> Optional[int]:
        return None


class Mixer(Part):
    """Mixes information between the positions of a sequence."""

    def cache_need(self):
        return None

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, cache) -> None:
        """Read the normed rows ``xn`` (act dtype), add the mixer's output into the float32
        stream ``x`` in place.  ``cache`` is the view that fits ``cache_need``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor) -> None:
        """Read ``xn``, add the feed-forward's output into ``x`` in place."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# registries of part kinds, so that a configuration can choose parts by name layer by layer

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}


def register_mixer(name: str, cls: type) -> None:
    MIXERS[name] = cls


def register_feed_forward(name: str, cls: type) -> None:
    FEED_FORWARDS[name] = cls


def register_norm(name: str, cls: type) -> None:
    NORMS[name] = cls


def register_position_encoding(name: str, cls: type) -> None:
    POSITION_ENCODINGS[name] = cls
