"""``Engine``: requests in, tokens out, through the scheduler and the step function.

The surface follows the reference's engine and its Python binding (src/engine.h:96-113;
python/bindings.cpp:110-125): ``add_request(prompt, params) -> id``, ``step() ->
[StepEvent]``, ``cancel``, ``idle``, ``result(id)``, ``stats``, ``free_blocks``,
``num_running``, ``num_waiting``, ``now``.  ``EngineConfig`` keeps the reference's names
where it has them (``num_blocks``, ``max_batched_tokens``, ``max_num_seqs``,
``fingerprint_logits``; src/engine.h:38-50) and adds ``block_size`` (the reference fixes
16, src/block_manager.h:20).  Prefix caching, speculative decoding, static batching and
fault injection are not part of this engine.

One step (src/engine.cpp:304-488): plan, build one batch, run it, sample the rows whose
request reached its last known token (on the device, keyed by the position the new token
will take), append, finish and free.  The logits fingerprint of a request
(src/engine.cpp:18-29,246) is chained on the device in the request's state slot.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..cache.storage import FINGERPRINT_SEED, build_cache
from ..model import _TORCH_DTYPE, Model
from ..sampling.rng import counter_uniform
from ..sampling.sampler import SamplingParams
from .scheduler import Planned, Scheduler, Sequence
from .step import StepEntry, Stepper


@dataclass
class EngineConfig:
    num_blocks: int = 512
    block_size: int = 16
    max_batched_tokens: int = 256
    max_num_seqs: int = 32
    fingerprint_logits: bool = True
    max_model_len: Optional[int] = None  # longest request (prompt + output); default: what the pool holds
    # Run a step ahead of the reads (CUDA devices; None: on where possible): ``step()`` launches
    # the next step before it reads the tokens of the one before, which go from the sampler into
    # the next step's batch on the device; the events a call returns are those of the step before.
    lookahead: Optional[bool] = None


@dataclass
class RequestResult:
    tokens: List[int] = field(default_factory=list)
    finished: bool = False
    cancelled: bool = False
    logits_fingerprint: int = FINGERPRINT_SEED
    preemptions: int = 0
    arrival: float = 0.0
    first_token: float = -1.0
    finish: float = -1.0
    token_times: List[float] = field(default_factory=list)


@dataclass
class StepEvent:
    id: int
    tokens: List[int]
    finished: bool


@dataclass
class _Launched:
    """A step that runs on the device and whose tokens the host has not read."""
    turn: int
    sampled: list          # [sequence, index in the sampler's output, state slot, index of the token in seq.tokens,
                           #  whether it is the request's last token by count]
    tokens_copied: object  # event: the sampled tokens are in pinned memory
    started: float


PENDING = -1  # stands in ``Sequence.tokens`` for a sampled token that has not been read


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_rows: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    forward_seconds: float = 0.0


def _signed64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


class Engine:
    def __init__(self, model: Model, config: Optional[EngineConfig] = None):
        self.model = model
        self.config = config or EngineConfig()
        c = self.config
        self.manager, self.storage = build_cache(model.decoder, c.num_blocks, c.block_size, c.max_num_seqs,
                                                 _TORCH_DTYPE[model.dtype], model.device)
        pool_tokens = c.num_blocks * c.block_size
        self.max_len = min(c.max_model_len or pool_tokens, pool_tokens)
        self.stepper = Stepper(model.decoder, self.manager, self.storage, model.ops,
                               max_rows=c.max_batched_tokens, max_seqs=c.max_num_seqs,
                               max_tokens_per_request=self.max_len)
        self.scheduler = Scheduler(self.manager, c.max_batched_tokens, c.max_num_seqs)
        self.scheduler.on_preempt = self._save_fingerprint
        self.vocab = model.decoder.head.vocab
        self.eos_id = getattr(model.config, "eos_token_id", -1)
        self.seqs: Dict[int, Sequence] = {}
        self.results: Dict[int, RequestResult] = {}
        self.stats = EngineStats()
        self._next_id = 0
        self._start = time.perf_counter()
        dev = model.device
        pin = torch.device(dev).type == "cuda"
        m = c.max_num_seqs
        # sampler inputs of a step, one pinned buffer: uniforms (f64), temperatures (f32), slots (i32);
        # two sets that take turns, for an engine that runs a step ahead of its reads
        self._lookahead = pin and c.lookahead is not False
        self._samp_hosts = [torch.zeros(m * 16, dtype=torch.uint8, pin_memory=pin) for _ in range(2)]
        self._samp_devs = [torch.zeros(m * 16, dtype=torch.uint8, device=dev) for _ in range(2)]
        self._tok_devs = [torch.zeros(m, dtype=torch.int32, device=dev) for _ in range(2)]
        self._tok_hosts = [torch.zeros(m, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._tok_events = [torch.cuda.Event(), torch.cuda.Event()] if pin else [None, None]
        self._turn = 0
        self._inflight: Optional[_Launched] = None
        self._use_turn(0)
        self.d2h_bytes = 0
        self._fp_live = set()  # requests whose fingerprint chain sits in their current slot
        # The fingerprint of a row is a serial chain over its logits (a fifth of a millisecond for
        # 49,152 of them) that nothing of the next step needs: on a CUDA device it runs on a
        # stream of its own over a copy of the sampled rows, beside the next step.  Two sets of
        # buffers take turns; events order copy -> hash -> the copy after next.
        self._fp_stream = torch.cuda.Stream(device=dev) if pin and c.fingerprint_logits else None
        self._fp_rows = [None, None]
        self._fp_slots = [torch.zeros(m, dtype=torch.int32, device=dev) for _ in range(2)] if self._fp_stream else []
        self._fp_copied = [torch.cuda.Event(), torch.cuda.Event()] if self._fp_stream else []
        self._fp_hashed = [None, None]
        self._fp_turn = 0
        self._fp_last = None  # event of the newest hash
        # what the slots held after each step's hashes, for an engine that reads a step late
        self._fp_snap = ([torch.zeros(self.storage.fingerprints.numel(), dtype=torch.int64, pin_memory=True)
                          for _ in range(2)] if self._fp_stream is not None and self._lookahead else None)

    def _use_turn(self, turn: int) -> None:
        m = self.config.max_num_seqs
        self._samp_host, self._samp_dev = self._samp_hosts[turn], self._samp_devs[turn]
        self._u_h, self._t_h, self._s_h = self._samp_views(self._samp_host, m)
        self._u_d, self._t_d, self._s_d = self._samp_views(self._samp_dev, m)
        self._tok_dev, self._tok_host = self._tok_devs[turn], self._tok_hosts[turn]

    @staticmethod
    def _samp_views(buf: torch.Tensor, m: int):
        return (buf[:m * 8].view(torch.float64), buf[m * 8:m * 12].view(torch.float32),
                buf[m * 12:m * 16].view(torch.int32))

    # -- the reference's surface -----------------------------------------------------------
    def now(self) -> float:
        return time.perf_counter() - self._start

    def add_request(self, prompt: Seq[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        if any(t < 0 or t >= self.vocab for t in prompt):
            raise ValueError("token id out of range")
        worst = len(prompt) + params.max_new_tokens + 1
        if worst > self.config.num_blocks * self.config.block_size or worst > self.max_len + 1:
            raise ValueError("request can never fit in the KV cache")
        seq = Sequence(self._next_id, prompt, len(prompt), params)
        self._next_id += 1
        self.seqs[seq.id] = seq
        self.results[seq.id] = RequestResult(arrival=self.now())
        self.scheduler.add(seq)
        return seq.id

    def cancel(self, rid: int) -> None:
        seq = self.seqs.get(rid)
        if seq is None or seq.done:
            return
        self._finish(seq, cancelled=True)

    def idle(self) -> bool:
        return self.scheduler.idle() and self._inflight is None

    @property
    def num_running(self) -> int:
        return len(self.scheduler.running)

    @property
    def num_waiting(self) -> int:
        return len(self.scheduler.waiting)

    @property
    def free_blocks(self) -> int:
        return self.manager.min_available()

    def result(self, rid: int) -> RequestResult:
        return self.results[rid]

    # -- internals -------------------------------------------------------------------------
    def _fingerprint_rows(self, logits: torch.Tensor, c: int, turn: Optional[int] = None) -> int:
        """Chain the hash of the c sampled rows into their requests' slots."""
        ops = self.model.ops
        if self._fp_stream is None:
            ops.fingerprint_rows(logits, self._s_d[:c], self.storage.fingerprints)
            return 0
        if turn is None:  # the two sets of buffers take turns; an engine that runs ahead names its own turn
            turn = self._fp_turn
            self._fp_turn ^= 1
        main = torch.cuda.current_stream()
        if self._fp_hashed[turn] is not None:
            main.wait_event(self._fp_hashed[turn])  # the hash that last read these buffers is done
        rows = self._fp_rows[turn]
        if rows is None or rows.shape[0] < c:
            rows = self._fp_rows[turn] = torch.empty((max(c, 8), self.vocab), dtype=torch.float32, device=logits.device)
        rows[:c].copy_(logits)
        self._fp_slots[turn][:c].copy_(self._s_d[:c])
        self._fp_copied[turn].record(main)
        with torch.cuda.stream(self._fp_stream):
            self._fp_stream.wait_event(self._fp_copied[turn])
            ops.fingerprint_rows(rows[:c], self._fp_slots[turn][:c], self.storage.fingerprints)
            if self._fp_snap is not None:
                self._fp_snap[turn].copy_(self.storage.fingerprints, non_blocking=True)
            done = self._fp_hashed[turn] or torch.cuda.Event()
            done.record(self._fp_stream)
            self._fp_hashed[turn] = done
            self._fp_last = done
        return turn

    def _read_fingerprint(self, slot: int) -> int:
        if self._fp_stream is not None:
            self._fp_stream.synchronize()  # every hash launched so far has been chained in
        return int(self.storage.fingerprints[slot].item()) & ((1 << 64) - 1)

    def _save_fingerprint(self, seq: Sequence, slot: int) -> None:
        """A request was preempted and lost its slot: bring its fingerprint to the host (the
        slot's contents stay as they were until the coming step runs)."""
        if self.config.fingerprint_logits and seq.id in self._fp_live and slot >= 0:
            self.results[seq.id].logits_fingerprint = self._read_fingerprint(slot)
        self._fp_live.discard(seq.id)
        self.results[seq.id].preemptions += 1

    def _finish(self, seq: Sequence, cancelled: bool) -> None:
        self._save_fingerprint_final(seq)
        self.scheduler.finish(seq)
        r = self.results[seq.id]
        r.finished, r.cancelled, r.finish = True, cancelled, self.now()
        del self.seqs[seq.id]

    def _save_fingerprint_final(self, seq: Sequence) -> None:
        if self._fp_snap is not None:
            self._fp_live.discard(seq.id)  # the result's fingerprint is brought up to date with every token read
            return
        if self.config.fingerprint_logits and seq.id in self._fp_live and self.manager.has(seq.id):
            slot = self.manager.get(seq.id).slot
            self.results[seq.id].logits_fingerprint = self._read_fingerprint(slot)
        self._fp_live.discard(seq.id)

    def step(self) -> List[StepEvent]:
        """Plan and run one step.  With ``lookahead`` the step is launched and the events of the
        step BEFORE it are returned (its tokens are read while this one runs)."""
        if self._lookahead:
            return self._step_ahead()
        events: List[StepEvent] = []
        self.stats.steps += 1
        plan = self.scheduler.plan()
        self.stats.preemptions = self.scheduler.stats.preemptions
        if not plan:
            return events
        entries: List[StepEntry] = []
        sampled: List[Planned] = []
        for p in plan:
            s = p.seq
            last = s.computed + p.n == len(s.tokens)
            entries.append(StepEntry(s.id, s.tokens[s.computed:s.computed + p.n], [p.n - 1] if last else []))
            if last:
                sampled.append(p)
            if p.n == 1 and s.computed == len(s.tokens) - 1 and s.generated > 0:
                self.stats.decode_rows += 1
            else:
                self.stats.prefill_tokens += p.n
            if self.config.fingerprint_logits and s.id not in self._fp_live:
                # a request that just got its slot: start (or, after preemption, continue) its chain
                slot = self.manager.get(s.id).slot
                self.storage.fingerprints[slot] = _signed64(self.results[s.id].logits_fingerprint)
                self._fp_live.add(s.id)
        t0 = time.perf_counter()
        logits = self.stepper.run(entries)
        c = len(sampled)
        if c:
            for i, p in enumerate(sampled):
                s = p.seq
                self._u_h[i] = counter_uniform(s.params.seed, len(s.tokens))
                self._t_h[i] = s.params.temperature
                self._s_h[i] = self.manager.get(s.id).slot
            self._samp_dev.copy_(self._samp_host, non_blocking=True)
            ops = self.model.ops
            ops.sample_rows(logits, self._t_d[:c], self._u_d[:c], self._tok_dev[:c])
            if self.config.fingerprint_logits:
                self._fingerprint_rows(logits, c)
            self._tok_host[:c].copy_(self._tok_dev[:c], non_blocking=True)
            if torch.device(self.model.device).type == "cuda":
                # the word that a kernel raises when it gave up a bounded wait rides along with
                # the tokens: a step whose kernels did not finish their work must not be used
                poll = getattr(ops, "failure_poll", None)
                if poll is not None:
                    poll()
                torch.cuda.current_stream().synchronize()
                if poll is not None and ops.failure_seen():
                    from ..kernels.ops import DeviceFailure
                    raise DeviceFailure("a kernel gave up a bounded wait; the results of this step and of the "
                                        "steps since the last sampled token are not valid")
            self.d2h_bytes = c * 4
        self.stats.forward_seconds += time.perf_counter() - t0
        toks = self._tok_host[:c].tolist() if c else []
        cursor = 0
        finished: List[Sequence] = []
        for p in plan:
            s = p.seq
            s.computed += p.n
            if s.computed != len(s.tokens):
                continue
            token = int(toks[cursor])
            cursor += 1
            r = self.results[s.id]
            s.tokens.append(token)
            r.tokens.append(token)
            t = self.now()
            if r.first_token < 0:
                r.first_token = t
            r.token_times.append(t)
            self.stats.generated_tokens += 1
            done = (not s.params.ignore_eos and token == self.eos_id) or s.generated >= s.params.max_new_tokens
            events.append(StepEvent(s.id, [token], done))
            if done:
                finished.append(s)
        for s in finished:
            self._finish(s, cancelled=False)
        return events

    # -- a step ahead of the reads ----------------------------------------------------------
    def _step_ahead(self) -> List[StepEvent]:
        self.stats.steps += 1
        plan = self.scheduler.plan()
        self.stats.preemptions = self.scheduler.stats.preemptions
        launched = self._launch(plan) if plan else None
        before, self._inflight = self._inflight, launched
        return self._collect(before) if before is not None else []

    def _launch(self, plan: List[Planned]) -> _Launched:
        turn = self._turn
        self._turn ^= 1
        values_before = self._tok_dev  # the sampler's output of the step before
        self._use_turn(turn)
        entries: List[StepEntry] = []
        sampled: List[Planned] = []
        patches = []
        row = 0
        fresh_slots = []
        for p in plan:
            s = p.seq
            toks = s.tokens[s.computed:s.computed + p.n]
            if s.computed <= s.pending < s.computed + p.n:  # the token is still on the device
                toks[s.pending - s.computed] = 0
                patches.append((row + s.pending - s.computed, s.pending_src))
            last = s.computed + p.n == len(s.tokens)
            entries.append(StepEntry(s.id, toks, [p.n - 1] if last else []))
            if last:
                sampled.append(p)
            if p.n == 1 and s.computed == len(s.tokens) - 1 and s.generated > 0:
                self.stats.decode_rows += 1
            else:
                self.stats.prefill_tokens += p.n
            if self.config.fingerprint_logits and s.id not in self._fp_live:
                fresh_slots.append((self.manager.get(s.id).slot, _signed64(self.results[s.id].logits_fingerprint)))
                self._fp_live.add(s.id)
            row += p.n
        if fresh_slots:
            # a request that just got its slot starts (or, after preemption, continues) its chain
            # there; the slot's last holder may still be hashed on the other stream
            if self._fp_last is not None:
                torch.cuda.current_stream().wait_event(self._fp_last)
            for slot, value in fresh_slots:
                self.storage.fingerprints[slot] = value
        started = time.perf_counter()
        logits = self.stepper.run(entries, patches, values_before)
        record = []
        c = len(sampled)
        if c:
            ops = self.model.ops
            for i, p in enumerate(sampled):
                s = p.seq
                slot = self.manager.get(s.id).slot
                self._u_h[i] = counter_uniform(s.params.seed, len(s.tokens))
                self._t_h[i] = s.params.temperature
                self._s_h[i] = slot
                record.append([s, i, slot, len(s.tokens), False])
            self._samp_dev.copy_(self._samp_host, non_blocking=True)
            ops.sample_rows(logits, self._t_d[:c], self._u_d[:c], self._tok_dev[:c])
            if self.config.fingerprint_logits:
                self._fingerprint_rows(logits, c, turn)
            self._tok_host[:c].copy_(self._tok_dev[:c], non_blocking=True)
            poll = getattr(ops, "failure_poll", None)
            if poll is not None:
                poll()
            self.d2h_bytes = c * 4
        self._tok_events[turn].record()
        for p in plan:
            p.seq.computed += p.n
        for rec in record:
            s, i, _, at, _ = rec
            s.tokens.append(PENDING)
            s.pending, s.pending_src = at, i
            if s.generated >= s.params.max_new_tokens:
                # its last token is sampled: it leaves the scheduler now (its pages go back in the
                # step the reference gives them back in) and is closed when the token is read
                rec[4] = True
                s.closing = True
                self.scheduler.finish(s)
        return _Launched(turn, record, self._tok_events[turn], started)

    def _collect(self, step: _Launched) -> List[StepEvent]:
        step.tokens_copied.synchronize()
        ops = self.model.ops
        if getattr(ops, "failure_seen", None) is not None and ops.failure_seen():
            from ..kernels.ops import DeviceFailure
            raise DeviceFailure("a kernel gave up a bounded wait; the results of the last steps are not valid")
        self.stats.forward_seconds += time.perf_counter() - step.started
        events: List[StepEvent] = []
        if not step.sampled:
            return events
        toks = self._tok_hosts[step.turn][:len(step.sampled)].tolist()
        snap = None
        if self._fp_snap is not None:
            self._fp_hashed[step.turn].synchronize()
            snap = self._fp_snap[step.turn]
        for s, i, slot, at, final in step.sampled:
            r = self.results[s.id]
            if r.finished:
                continue  # cancelled meanwhile, or ended by an end-of-sequence token a step earlier
            token = int(toks[i])
            s.tokens[at] = token
            if s.pending == at:
                s.pending = -1
            r.tokens.append(token)
            if snap is not None:
                r.logits_fingerprint = int(snap[slot]) & ((1 << 64) - 1)
            t = self.now()
            if r.first_token < 0:
                r.first_token = t
            r.token_times.append(t)
            self.stats.generated_tokens += 1
            done = final or (not s.params.ignore_eos and token == self.eos_id)
            events.append(StepEvent(s.id, [token], done))
            if not done:
                continue
            if s.closing:  # it has left the scheduler already (with this token, or with the stand-in after it)
                self._fp_live.discard(s.id)
                r.finished, r.finish = True, t
                del self.seqs[s.id]
            else:
                del s.tokens[at + 1:]  # the stand-in of the step that runs now, whose row is of no use
                s.pending = -1
                self._finish(s, cancelled=False)
        return events

    def generate(self, prompts: Seq[Seq[int]], params: Optional[SamplingParams] = None,
                 max_steps: int = 1_000_000) -> List[List[int]]:
        """Convenience: run the given prompts to the end and return their generated tokens."""
        if isinstance(params, (list, tuple)):
            plist = list(params)
        else:
            plist = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, q) for p, q in zip(prompts, plist)]
        steps = 0
        while not self.idle():
            self.step()
            steps += 1
            if steps > max_steps:
                raise RuntimeError("the engine did not go idle (step limit reached)")
        return [self.results[i].tokens for i in ids]
