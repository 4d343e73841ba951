"""Continuous batching above the step function: admit, cut prompts into portions under a
token budget, decode, finish and free; recompute preemption when pages run out.

The decisions are taken in C++ (``Scheduler`` in csrc/host_runtime.cpp, next to the cache
manager it asks for pages); this class owns the requests' tokens, tells the library before
every plan how many tokens each running request has and how many of them are computed, and
mirrors what the plan did (rows to run, requests preempted or admitted) back onto the
``Sequence`` objects.

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

Nothing here touches a device.  ``Engine`` (engine/engine.py) runs what is planned.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

from .. import host
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
    # An engine that runs a step ahead of its reads: the index in ``tokens`` of a sampled token
    # that the host has not read yet (a stand-in until then; -1: none), where it lies in the
    # sampler's output, and whether the request has left the scheduler because its last token
    # is sampled (it is closed when that token is read).
    pending: int = -1
    pending_src: int = -1
    closing: bool = False

    @property
    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len


@dataclass
class Planned:
    seq: Sequence
    n: int  # rows to run for it in this step


class SchedulerStats:
    def __init__(self, scheduler: "Scheduler"):
        self._s = scheduler

    @property
    def preemptions(self) -> int:
        return int(self._s._lib.bw_sched_stat(self._s._h, 0))

    @property
    def admitted(self) -> int:
        return int(self._s._lib.bw_sched_stat(self._s._h, 1))


class SchedulerError(RuntimeError):
    pass


class Scheduler:
    def __init__(self, manager: CacheManager, max_batched_tokens: int, max_num_seqs: int):
        if max_batched_tokens <= 0 or max_num_seqs <= 0:
            raise ValueError("max_batched_tokens and max_num_seqs must be positive")
        self._lib = host.lib()
        self.manager = manager
        self.max_batched_tokens = max_batched_tokens
        self.max_num_seqs = max_num_seqs
        self._h = self._lib.bw_sched_create(manager._h, max_batched_tokens, max_num_seqs)
        if not self._h:
            raise SchedulerError(host.last_error())
        self._seqs: Dict[int, Sequence] = {}     # the library's key -> request
        self._key: Dict[int, int] = {}           # request id -> key
        cap = max(64, 2 * max_num_seqs + 16)
        self._ids = (ctypes.c_int64 * cap)()
        self._ints = (ctypes.c_int * cap)()
        self._ints2 = (ctypes.c_int * cap)()
        self._cap = cap
        self.stats = SchedulerStats(self)
        self.preempted_log: List[int] = []       # ids in the order they were preempted
        # callback(seq, slot) for a request that has just been preempted: ``slot`` is the state
        # slot it held (its contents stay untouched until the step that follows runs)
        self.on_preempt: Optional[Callable[[Sequence, int], None]] = None

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bw_sched_destroy(self._h)
            self._h = None

    def _grow(self, n: int) -> None:
        if n > self._cap:
            self._cap = 2 * n
            self._ids = (ctypes.c_int64 * self._cap)()
            self._ints = (ctypes.c_int * self._cap)()
            self._ints2 = (ctypes.c_int * self._cap)()

    # -- queue operations --------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        key = self.manager.key_of(seq.id)
        self.manager.hold_key(seq.id)
        if self._lib.bw_sched_add(self._h, key, int(seq.id), len(seq.tokens), seq.computed) < 0:
            raise SchedulerError(host.last_error())
        self._seqs[key] = seq
        self._key[seq.id] = key

    def _listed(self, fn) -> List[Sequence]:
        n = fn(self._h, self._ids, self._cap)
        if n > self._cap:
            self._grow(n)
            n = fn(self._h, self._ids, self._cap)
        return [self._seqs[self._ids[i]] for i in range(n)]

    @property
    def running(self) -> List[Sequence]:
        """Running requests, oldest first."""
        return self._listed(self._lib.bw_sched_running)

    @property
    def waiting(self) -> List[Sequence]:
        """Waiting requests in the order they will be admitted."""
        return self._listed(self._lib.bw_sched_waiting)

    def idle(self) -> bool:
        return not self._seqs

    def _mirror_preempted(self) -> None:
        n = self._lib.bw_sched_preempted(self._h, self._ids, self._ints, self._cap)
        gone = []
        for i in range(min(n, self._cap)):
            seq = self._seqs[self._ids[i]]
            seq.computed = 0
            seq.running = False
            gone.append((seq, self._ints[i]))
        self.manager.sync_with_library([s.id for s, _ in gone])
        for seq, slot in gone:
            self.preempted_log.append(seq.id)
            if self.on_preempt is not None:
                self.on_preempt(seq, slot)

    def preempt(self, seq: Sequence) -> None:
        self._push([seq])
        if self._lib.bw_sched_preempt(self._h, self._key[seq.id]) < 0:
            raise SchedulerError(host.last_error())
        self._mirror_preempted()

    def finish(self, seq: Sequence) -> None:
        """The request is over (done or cancelled): pages and slot go back, queues forget it."""
        key = self._key.pop(seq.id)
        if self._lib.bw_sched_finish(self._h, key) < 0:
            raise SchedulerError(host.last_error())
        del self._seqs[key]
        seq.computed = 0
        seq.running = False
        seq.done = True
        self.manager.sync_with_library([seq.id])
        self.manager.drop_key(seq.id)

    def _push(self, seqs: List[Sequence]) -> None:
        n = len(seqs)
        self._grow(n)
        for i, s in enumerate(seqs):
            self._ids[i] = self._key[s.id]
            self._ints[i] = len(s.tokens)
            self._ints2[i] = s.computed
        if n and self._lib.bw_sched_update_many(self._h, n, self._ids, self._ints, self._ints2) < 0:
            raise SchedulerError(host.last_error())

    # -- one step's plan ---------------------------------------------------------------
    def plan(self) -> List[Planned]:
        # the library learns how far every request has come (tokens are appended and rows
        # computed on this side), then decides
        self._push(list(self._seqs.values()))
        waiting_head = self.waiting[:1]
        n = self._lib.bw_sched_plan(self._h)
        self._grow(n)
        self._mirror_preempted()
        n = self._lib.bw_sched_plan_entries(self._h, self._ids, self._ints, self._cap)
        plan = [Planned(self._seqs[self._ids[i]], self._ints[i]) for i in range(n)]
        # requests that the plan admitted hold pages and a slot now; a head that could not be
        # admitted gave back what it took
        self.manager.sync_with_library([p.seq.id for p in plan] + [s.id for s in waiting_head])
        running = self.running
        for s in running:
            if not s.running:
                s.running = True
        if len(running) > len(plan):  # a running request with nothing to do this step may not be listed
            self.manager.sync_with_library([s.id for s in running])
        return plan
