"""Continuous batching above the step function: admit, cut prompts into portions under a
token budget, decode, finish and free; recompute preemption when pages run out.

The policy is the reference's (src/engine.cpp:304-377), decision for decision:

1. Running requests are served oldest first (by id).  A request needs
   ``len(tokens) - computed`` rows: one for a decode, more for a prompt not yet through or
   being recomputed.  If that exceeds what is left of the step's budget it gets the rest
   of the budget (a portion), or nothing when the budget is spent; it stays running.
2. Its pages are taken one at a time.  When the pool runs dry the YOUNGEST running
   request that is neither already scheduled in this step nor the asker is preempted: all
   its pages go back, ``computed = 0``, and it returns to the waiting queue in id order,
   ahead of newer arrivals, to be recomputed over prompt plus generated tokens later.  With
   no such victim the asker preempts itself.  (src/engine.cpp:166-174,233-237,335-347)
3. Then waiting requests are admitted first-in first-out, only the head of the queue, while
   fewer than ``max_num_seqs`` run and budget is left.  A head that cannot get its pages
   gives back what it took and admission stops for this step; nobody is preempted for a
   newcomer.  (src/engine.cpp:354-376)
4. A request that could never fit is refused when it is added (src/engine.cpp:130-133).

This class decides only; it never touches a device.  ``Engine`` (engine/engine.py) runs
what it plans.
"""
from __future__ import annotations

import bisect
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams


@dataclass
class Sequence:
    """Host state of one request (src/engine.cpp:82-98)."""
    id: int
    tokens: List[int]          # prompt + generated
    prompt_len: int
    params: SamplingParams
    computed: int = 0          # tokens whose keys/values are in the cache
    running: bool = False
    done: bool = False

    @property
    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len


@dataclass
class Planned:
    seq: Sequence
    n: int  # rows to run for it in this step


@dataclass
class SchedulerStats:
    preemptions: int = 0
    admitted: int = 0


class Scheduler:
    def __init__(self, manager: CacheManager, max_batched_tokens: int, max_num_seqs: int):
        if max_batched_tokens <= 0 or max_num_seqs <= 0:
            raise ValueError("max_batched_tokens and max_num_seqs must be positive")
        self.manager = manager
        self.max_batched_tokens = max_batched_tokens
        self.max_num_seqs = max_num_seqs
        self.running: List[Sequence] = []       # sorted by id
        self.waiting: Deque[Sequence] = deque()  # first in, first out; preempted ones re-enter in id order
        self.stats = SchedulerStats()
        self.preempted_log: List[int] = []      # ids in the order they were preempted
        self.on_preempt = None                  # callback(seq) before its pages go back

    # -- queue operations --------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def idle(self) -> bool:
        return not self.running and not self.waiting

    def _release(self, seq: Sequence) -> None:
        if self.manager.has(seq.id):
            self.manager.release(seq.id)
        seq.computed = 0

    def preempt(self, seq: Sequence) -> None:
        if self.on_preempt is not None:
            self.on_preempt(seq)
        self._release(seq)
        seq.running = False
        self.running.remove(seq)
        pos = 0
        while pos < len(self.waiting) and self.waiting[pos].id < seq.id:
            pos += 1
        self.waiting.insert(pos, seq)
        self.stats.preemptions += 1
        self.preempted_log.append(seq.id)

    def finish(self, seq: Sequence) -> None:
        """The request is over (done or cancelled): pages and slot go back, queues forget it."""
        self._release(seq)
        if seq.running:
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        seq.running = False
        seq.done = True

    def _pick_victim(self, protect: List[Sequence]) -> Optional[Sequence]:
        for s in reversed(self.running):
            if s not in protect:
                return s
        return None

    # -- one step's plan ---------------------------------------------------------------
    def plan(self) -> List[Planned]:
        budget = self.max_batched_tokens
        plan: List[Planned] = []
        scheduled: List[Sequence] = []
        for s in list(self.running):
            if not s.running:
                continue  # preempted earlier in this loop
            need = len(s.tokens) - s.computed
            n = need
            if n == 0:
                continue
            if n > budget:
                if budget <= 0:
                    continue
                n = budget
            ok = self.manager.ensure(s.id, s.computed + n)
            while not ok:
                victim = self._pick_victim(scheduled + [s])
                if victim is None:
                    break
                self.preempt(victim)
                ok = self.manager.ensure(s.id, s.computed + n)
            if not ok:
                self.preempt(s)
                continue
            plan.append(Planned(s, n))
            scheduled.append(s)
            budget -= n
        while self.waiting and len(self.running) < self.max_num_seqs:
            if budget <= 0:
                break
            s = self.waiting[0]
            need = len(s.tokens) - s.computed
            n = min(need, budget)
            if not self.manager.has(s.id):
                if self.manager.free_slots() == 0:
                    break
                self.manager.begin(s.id)
            if not self.manager.ensure(s.id, s.computed + n):
                self._release(s)
                break
            self.waiting.popleft()
            s.running = True
            bisect.insort(self.running, s, key=lambda q: q.id)
            self.stats.admitted += 1
            if n > 0:
                plan.append(Planned(s, n))
                budget -= n
        return plan
