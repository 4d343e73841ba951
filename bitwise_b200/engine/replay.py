"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: every step goes
through :class:`Stepper`, the step function that generation uses, over a cache pool made
for ``max_tokens`` tokens (so that pages are used again when requests end).  The
reference's nearest analogues are ``logits_chunked`` in its tests
(tests/test_main.cpp:200-217) and ``Model.logits`` (python/bindings.cpp:35-52).

Input: one JSON object a line,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}``.
For a step in which something is wanted the logits at the wanted places are written to
``<out>/<step>.f32`` as little-endian float32 ``[wanted, vocab]``, in the order of the
entries and of ``want``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np
import torch

from ..cache.storage import build_cache
from ..model import _TORCH_DTYPE, Model
from .step import StepEntry, Stepper

MAX_LIVE_REQUESTS = 4


def make_replay_stepper(model: Model, max_tokens: int, page_size: int = 16, max_live: int = MAX_LIVE_REQUESTS,
                        max_rows: Optional[int] = None, use_graphs: Optional[bool] = None) -> Stepper:
    """A stepper over a pool that holds ``max_tokens`` tokens (each live request's count
    rounded up to a multiple of 64; the page size divides 64)."""
    if 64 % page_size:
        raise ValueError(f"page size {page_size} does not divide 64")
    pages = (max_tokens + page_size - 1) // page_size
    manager, storage = build_cache(model.decoder, pages, page_size, max_live, _TORCH_DTYPE[model.dtype],
                                   model.device)
    return Stepper(model.decoder, manager, storage, model.ops, max_rows=max_rows or max(max_tokens, 1),
                   max_seqs=max_live, max_tokens_per_request=max_tokens, use_graphs=use_graphs)


def replay(model: Model, lines: IO[str], out_dir: str, max_tokens: int, page_size: int = 16,
           report: Optional[IO[str]] = None) -> int:
    """Run every step read from ``lines``; returns the number of steps run."""
    report = report if report is not None else sys.stdout
    os.makedirs(out_dir, exist_ok=True)
    stepper = make_replay_stepper(model, max_tokens, page_size)
    count = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if entries:
            logits = stepper.run(entries)
            if logits is not None:
                poll = getattr(model.ops, "failure_poll", None)
                if poll is not None:
                    poll()
                arr = logits.detach().to(torch.float32).cpu().numpy()
                if poll is not None and model.ops.failure_seen():
                    raise RuntimeError(f"step {step}: a kernel gave up a bounded wait; its logits are not written")
                arr.astype("<f4").tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            stepper.finish(rid)
        print(f"done {step}", file=report, flush=True)
        count += 1
    return count
