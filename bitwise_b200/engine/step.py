"""The step function: one batch of (request, its next tokens) through the model.

In the manner of the reference's ``Runner::forward`` (src/model.cpp:267-322) and of the
row building in its engine (src/engine.cpp:386-402): a batch is a flat list of rows, each
a token at a position of some request; portions of prompts stand beside single decoded
tokens, cut anywhere.  Keys and values of every row are stored in the cache before
attention runs, and attention reads the cache only, so the logits at a position do not
depend on how the tokens were cut into steps or on what else is in the batch.  Only the
tokens given are run; logits come back for the wanted rows only.

The host side of a step is one packed int32 buffer (tokens, positions, the row -> sequence
map, per-sequence arrays, the block tables of every cache group, query tiles) copied to
the device in one transfer from pinned memory; every kernel of the step reads its
indices from there, which also keeps the step replayable as a CUDA graph.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import FREED, CacheError, CacheManager
from ..cache.storage import CacheStorage
from ..parts.base import StepContext, Workspace


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(RuntimeError):
    pass


class OutOfPages(StepError):
    pass


def query_tile_rows(model, ops=None) -> List[int]:
    """The distinct query-tile heights that the model's mixers ask for on the kernel library ``ops``."""
    sizes = set()
    for b in model.blocks:
        fn = getattr(b.mixer, "query_tile_rows", None)
        if fn is not None:
            try:
                got = fn(ops)
            except TypeError:  # a mixer that takes no argument
                got = fn()
            sizes.update(int(v) for v in (got if isinstance(got, (list, tuple, set)) else [got]))
    return sorted(sizes) or [16]


class _Layout:
    """Offsets (in int32 elements) of the sections of the packed step buffer."""

    def __init__(self, max_rows: int, max_seqs: int, max_blocks: Sequence[int], tile_rows: Sequence[int]):
        self.max_rows, self.max_seqs = max_rows, max_seqs
        self.max_blocks = list(max_blocks)
        self.tile_rows = list(tile_rows)
        off = 0

        def take(n):
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4  # keep every section 16-byte aligned
            return start

        self.tokens = take(max_rows)
        self.pos = take(max_rows)
        self.row_seq = take(max_rows)
        self.seq_row0 = take(max_seqs + 1)
        self.seq_pos0 = take(max_seqs)
        self.seq_slot = take(max_seqs)
        self.logit_rows = take(max_rows)
        self.patch_rows = take(max_seqs)   # rows whose token the step before sampled, and where it lies
        self.patch_src = take(max_seqs)
        self.tiles = {}
        for tr in self.tile_rows:
            cap = max_rows // tr + max_seqs + 1
            self.tiles[tr] = (take(cap), take(cap), take(cap), cap)
        self.tables = [take(max_seqs * mb) for mb in self.max_blocks]
        self.total = off


class Stepper:
    """Owns the step's device buffers and runs steps for one model and one cache."""

    GRAPH_MAX_ROWS = 256   # steps up to this many rows are replayed as CUDA graphs
    GRAPH_CACHE = 256      # graphs kept (one per batch shape and bound on the context length)
    # A decode step of more than PAD_FROM rows is filled up to a multiple of PAD_TO with rows of
    # no request (token 0 at position 0 of a page and slot that no request ever holds), so that
    # batches whose size drifts as requests come and go meet a graph captured earlier.
    PAD_TO = 8
    PAD_FROM = 8

    def __init__(self, model, manager: CacheManager, storage: CacheStorage, ops, max_rows: int,
                 max_seqs: int, max_tokens_per_request: int, use_graphs: Optional[bool] = None):
        self.model, self.manager, self.storage, self.ops = model, manager, storage, ops
        self.device = model.device
        self.max_rows, self.max_seqs = max_rows, max_seqs
        page = manager.page_size
        mb = (max_tokens_per_request + page - 1) // page
        pad = self.PAD_TO - 1
        self._fill_seq0 = max_seqs + 1  # first sequence index of the filling rows (behind the end mark of seq_row0)
        self.layout = _Layout(max_rows + pad, max_seqs + 1 + pad, [mb] * len(manager.groups), query_tile_rows(model, ops))
        pin = self.device is not None and torch.device(self.device).type == "cuda"
        self.host = torch.zeros(self.layout.total, dtype=torch.int32, pin_memory=pin)
        self._host_np = self.host.numpy()
        self._host_address = self.host.data_ptr()
        import ctypes
        groups = len(self.layout.max_blocks)
        self._rows = manager.new_rows(max_seqs)    # what each row of the block tables in the pinned buffer holds
        self._keys_buf = (ctypes.c_int64 * max_seqs)()
        self._counts_buf = (ctypes.c_int * max_seqs)()
        self._starts_buf = (ctypes.c_int * max_seqs)()
        self._slots_buf = (ctypes.c_int * max_seqs)()
        self._table_offsets = (ctypes.c_int * max(groups, 1))(*self.layout.tables)
        self._max_blocks_buf = (ctypes.c_int * max(groups, 1))(*self.layout.max_blocks)
        self._views: Dict[tuple, dict] = {}        # step sizes -> views of the device buffer
        # the sequences of filling rows sit behind the real ones: their rows of the block tables
        # name the spare page, their slot is the spare slot, and nothing else ever writes there
        L = self.layout
        f0 = self._fill_seq0
        for g, off in enumerate(L.tables):
            rows0 = off + f0 * L.max_blocks[g]
            self._host_np[rows0:rows0 + pad * L.max_blocks[g]] = storage.pad_pages[g] if hasattr(storage, "pad_pages") else 0
        self._host_np[L.seq_slot + f0:L.seq_slot + f0 + pad] = getattr(storage, "pad_slot", 0)
        self._host_np[L.seq_pos0 + f0:L.seq_pos0 + f0 + pad] = 0
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=self.device)
        self.workspace = Workspace(self.device, max_rows + pad)
        self.vocab = model.head.vocab
        model.reserve_positions(mb * page)
        self.steps = 0
        self.h2d_bytes = 0
        self._copy_done = torch.cuda.Event() if pin else None
        self._copy_pending = False
        # Small steps are bound by launch overhead: after a batch shape has been run once
        # eagerly (which allocates every buffer it needs), its kernel sequence is captured
        # into a CUDA graph and replayed.  All indices live in the packed device buffer, so
        # a replay differs from another only by the data copied before it.  Only the serving
        # precision does this (the 32-bit attention sizes its shared memory on the host),
        # and only models whose parts all say they are safe to capture.
        if use_graphs is None:
            use_graphs = pin and getattr(ops, "kind", "") == "bf16"
        self.use_graphs = bool(use_graphs) and getattr(model, "graph_safe", lambda: False)()
        # contexts reach the kernels rounded up to this many keys (1: as they are)
        self.key_granule = max(1, int(getattr(ops, "key_granule", 1)))
        self._graphs: Dict[tuple, tuple] = {}
        self._seen: Dict[tuple, int] = {}
        self.graph_replays = 0

    # -- building the batch ------------------------------------------------------------
    def _section(self, t: torch.Tensor, start: int, n: int) -> torch.Tensor:
        return t[start:start + n]

    def prepare(self, entries: Sequence[StepEntry], patches: Sequence[Tuple[int, int]] = (),
                patch_values: Optional[torch.Tensor] = None) -> Tuple[StepContext, List[Tuple[Hashable, int]]]:
        """Allocate pages, fill the packed buffer, copy it, and return the step's context
        together with (request, new length) for the bookkeeping after the run.  ``patches``:
        (row, index) pairs: the token of that row is ``patch_values[index]`` on the device (what
        the step before sampled and the host has not read)."""
        L, mgr = self.layout, self.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        if self._copy_pending:  # the pinned buffer is rewritten only after its last copy is done
            self._copy_done.synchronize()
            self._copy_pending = False
        if len(entries) > self.max_seqs:
            raise StepError(f"{len(entries)} requests in one step; the stepper was built for {self.max_seqs}")
        seen = set()
        h = self._host_np
        vocab = self.vocab
        num_seqs = len(entries)
        rows_total = 0
        for s, e in enumerate(entries):
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            cnt = len(e.tokens)
            if cnt == 0:
                raise StepError(f"request {e.rid!r} brings no tokens")
            rows_total += cnt
            if rows_total > self.max_rows:
                raise StepError(f"step of more than {self.max_rows} rows")
            toks = e.tokens
            if min(toks) < 0 or max(toks) >= vocab:  # (a token still on the device stands as 0 here)
                bad = next(t for t in toks if not (0 <= t < vocab))
                raise StepError(f"token id {bad} outside the vocabulary of {vocab}")
            for w in e.want:
                if not (0 <= w < cnt):
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its {cnt} tokens")
            if not mgr.has(e.rid):
                mgr.begin(e.rid)
            self._keys_buf[s] = mgr.get(e.rid)._key
            self._counts_buf[s] = cnt
        # Pages and block-table rows, in the library, for all requests at once: every request
        # takes the pages its new tokens need, and its rows of the block tables in the pinned
        # buffer are brought up to date (a request that sits in the same row as in the step
        # before only adds the pages it gained).
        rc = mgr.prepare_rows(self._rows, num_seqs, self._keys_buf, self._counts_buf, self._host_address,
                              self._table_offsets, self._max_blocks_buf, self._starts_buf, self._slots_buf)
        if rc > 0:
            e = entries[rc - 1]
            raise OutOfPages(f"no free page for request {e.rid!r} ({mgr.length(e.rid)} + {len(e.tokens)} tokens)")
        if rc < 0:
            e = entries[-rc - 2]
            raise StepError(f"request {e.rid!r} would hold {mgr.length(e.rid) + len(e.tokens)} tokens; the block "
                            f"table covers {min(L.max_blocks) * mgr.page_size}")
        n = 0
        seq_rows: List[Tuple[int, int]] = []
        seq_pos0: List[int] = self._starts_buf[:num_seqs]
        seq_slot: List[int] = self._slots_buf[:num_seqs]
        after: List[Tuple[Hashable, int]] = []
        logit_rows: List[int] = []
        all_tokens: List[int] = []
        all_pos: List[int] = []
        all_row_seq: List[int] = []
        max_keys = 0
        for s, e in enumerate(entries):
            cnt = len(e.tokens)
            start = seq_pos0[s]
            all_tokens.extend(e.tokens)
            all_pos.extend(range(start, start + cnt))
            all_row_seq.extend([s] * cnt)
            for w in e.want:
                logit_rows.append(n + w)
            seq_rows.append((n, cnt))
            after.append((e.rid, start + cnt))
            max_keys = max(max_keys, start + cnt)
            n += cnt
        # What the kernels get is a bound on the context, rounded up to the library's granule:
        # launchers size grids, scratch and record strides from it, so everything that a launch
        # derives on the host is a function of the rounded value, which is also part of the key
        # under which a step's graph is kept.  Rows are bounded on the device by their own position.
        granule = self.key_granule
        max_keys = (max_keys + granule - 1) // granule * granule
        # filling rows (see PAD_TO): one row each of sequences _fill_seq0, _fill_seq0 + 1, ...
        n_real, c_real = n, len(logit_rows)
        fill = 0
        if self.use_graphs and n == num_seqs and self.PAD_FROM < n <= self.GRAPH_MAX_ROWS and hasattr(self.storage, "pad_pages"):
            fill = (-n) % self.PAD_TO
            for i in range(fill):
                all_tokens.append(0)
                all_pos.append(0)
                all_row_seq.append(self._fill_seq0 + i)
                h[L.seq_row0 + self._fill_seq0 + i] = n
                logit_rows.append(n)
                n += 1
        h[L.tokens:L.tokens + n] = all_tokens
        h[L.pos:L.pos + n] = all_pos
        h[L.row_seq:L.row_seq + n] = all_row_seq
        h[L.seq_row0:L.seq_row0 + num_seqs + 1] = [r[0] for r in seq_rows] + [n]
        h[L.seq_pos0:L.seq_pos0 + num_seqs] = seq_pos0
        h[L.seq_slot:L.seq_slot + num_seqs] = seq_slot
        c = len(logit_rows)
        h[L.logit_rows:L.logit_rows + c] = logit_rows
        # Query tiles, for every tile height in use, listed with the most keys first: a tile's
        # attention takes as long as it has keys, and blocks that start in this order finish
        # together instead of leaving the longest for last.
        tiles = {}
        for tr, (o_seq, o_row0, o_rows, cap) in L.tiles.items():
            listed = []
            for s, (r0, cnt) in enumerate(seq_rows):
                for a in range(0, cnt, tr):
                    rows_here = min(tr, cnt - a)
                    listed.append((-(seq_pos0[s] + a + rows_here), s, r0 + a, rows_here))
            if len(listed) > 1:
                listed.sort()
            for i in range(fill):  # one key each: they come last
                listed.append((-1, self._fill_seq0 + i, n_real + i, 1))
            t = len(listed)
            if t:
                h[o_seq:o_seq + t] = [x[1] for x in listed]
                h[o_row0:o_row0 + t] = [x[2] for x in listed]
                h[o_rows:o_rows + t] = [x[3] for x in listed]
            tiles[tr] = t
        if patches:
            h[L.patch_rows:L.patch_rows + len(patches)] = [r for r, _ in patches]
            h[L.patch_src:L.patch_src + len(patches)] = [i for _, i in patches]
        self.dev.copy_(self.host, non_blocking=True)
        if self._copy_done is not None:
            self._copy_done.record()
            self._copy_pending = True
        if patches:
            d = self.dev
            self.ops.patch_tokens(d[L.tokens:L.tokens + n], d[L.patch_rows:L.patch_rows + len(patches)],
                                  d[L.patch_src:L.patch_src + len(patches)], patch_values, len(patches))
        self.h2d_bytes = self.host.numel() * 4
        # The views of the device buffer depend on the step's sizes only: steps of a shape seen
        # before take them from a small cache (slicing a tensor costs microseconds, a dozen each step).
        shape = (n, num_seqs, c) + tuple(tiles.values())
        views = self._views.get(shape)
        if views is None:
            d = self.dev
            views = dict(
                tokens=d[L.tokens:L.tokens + n], pos=d[L.pos:L.pos + n], row_seq=d[L.row_seq:L.row_seq + n],
                seq_row0=d[L.seq_row0:L.seq_row0 + num_seqs + 1], seq_pos0=d[L.seq_pos0:L.seq_pos0 + num_seqs],
                seq_slot=d[L.seq_slot:L.seq_slot + num_seqs], logit_rows=d[L.logit_rows:L.logit_rows + c],
                tile_sets={tr: (d[o[0]:o[0] + tiles[tr]], d[o[1]:o[1] + tiles[tr]], d[o[2]:o[2] + tiles[tr]],
                                tiles[tr]) for tr, o in L.tiles.items()},
                block_tables=[d[L.tables[g]:L.tables[g] + num_seqs * L.max_blocks[g]].view(num_seqs, L.max_blocks[g])
                              for g in range(len(L.max_blocks))])
            if len(self._views) >= 512:
                self._views.clear()
            self._views[shape] = views
        first_tr = L.tile_rows[0]
        ctx = StepContext(
            ops=self.ops, workspace=self.workspace, n=n, num_seqs=num_seqs,
            tokens=views["tokens"], pos=views["pos"], row_seq=views["row_seq"], seq_row0=views["seq_row0"],
            seq_pos0=views["seq_pos0"], seq_slot=views["seq_slot"], logit_rows=views["logit_rows"],
            num_logit_rows=c, max_keys=max_keys,
            host_seq_rows=seq_rows, host_seq_pos0=seq_pos0, host_seq_slot=seq_slot)
        ctx.wanted_rows = c_real  # logits rows that belong to requests (the rest belong to filling rows)
        ctx.tile_sets = views["tile_sets"]
        ctx.tile_seq, ctx.tile_row0, ctx.tile_rows, ctx.num_tiles = ctx.tile_sets[first_tr]
        ctx.block_tables = views["block_tables"]
        if "cache" not in views:
            views["cache"] = self.storage.views(ctx.block_tables, ctx.seq_slot)
        ctx.cache_views = views["cache"]
        return ctx, after

    # -- running -----------------------------------------------------------------------
    def run(self, entries: Sequence[StepEntry], patches: Sequence[Tuple[int, int]] = (),
            patch_values: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [wanted, vocab] on the device (a view of
        the stepper's buffer, valid until the next step) or None when nothing is wanted."""
        ctx, after = self.prepare(entries, patches, patch_values)
        views = ctx.cache_views
        key = None
        if self.use_graphs and ctx.n <= self.GRAPH_MAX_ROWS:
            # everything a launcher computes on the host is a function of these: the step's sizes,
            # the (rounded) bound on the context and the numbers of query tiles
            # (a step with filling rows is the same step whatever share of its rows is filling)
            seqs = ctx.num_seqs if ctx.wanted_rows == ctx.num_logit_rows else -1
            key = (ctx.n, seqs, ctx.num_logit_rows, ctx.max_keys) + tuple(t[3] for t in ctx.tile_sets.values())
        if key is not None and key in self._graphs:
            graph, logits, launches = self._graphs[key]
            graph.replay()
            self.ops.launches += launches
            self.graph_replays += 1
        elif key is not None and self._seen.get(key, 0) >= 1 and len(self._graphs) < self.GRAPH_CACHE:
            before = self.ops.launches
            graph = torch.cuda.CUDAGraph()
            # No garbage collection while the stream captures: collecting an old stepper
            # destroys its graphs, and destroying a graph during a capture invalidates it.
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    logits = self.model.forward(ctx, views)
            finally:
                if collecting:
                    gc.enable()
            launches = self.ops.launches - before
            self._graphs[key] = (graph, logits, launches)
            graph.replay()
            self.graph_replays += 1
        else:
            logits = self.model.forward(ctx, views)
            if key is not None:
                self._seen[key] = self._seen.get(key, 0) + 1
        for rid, length in after:
            self.manager.advance(rid, length)
        self.steps += 1
        self.last_context = ctx
        if logits is not None and ctx.wanted_rows < ctx.num_logit_rows:
            return logits[:ctx.wanted_rows] if ctx.wanted_rows else None
        return logits

    def finish(self, rid: Hashable) -> None:
        """The request is over: everything it holds goes back."""
        if self.manager.has(rid):
            self.manager.release(rid)
