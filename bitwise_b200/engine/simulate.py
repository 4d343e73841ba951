"""Randomised traces against requests run alone: the reference's simulator
(sim/simulate.cpp:81-217) for this engine.

Each trace is a seeded random workload (1 to 10 requests, random prompts, arrival steps,
greedy or sampled decoding, 1 to 24 new tokens, an optional cancel step) on an engine whose
configuration is drawn at random too (token budget 4 to 64, 1 to 8 running requests, a pool
of the minimum size plus 0 to 12 pages, so that preemption and recompute happen).  The
oracle: every request that was not cancelled yields exactly the tokens, and the logits
fingerprint, that it yields alone on an idle engine; the engine goes idle within a step
limit (no hang) and holds every page again afterwards (no leak).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from ..sampling.sampler import SamplingParams
from .engine import Engine, EngineConfig

STEP_LIMIT = 20000  # sim/simulate.cpp:168


@dataclass
class Outcome:
    traces: int = 0
    requests_checked: int = 0
    token_mismatch: int = 0
    fingerprint_mismatch: int = 0
    hangs: int = 0
    leaks: int = 0
    preemptions: int = 0
    first_bad_trace: int = -1

    @property
    def violations(self) -> int:
        return self.token_mismatch + self.fingerprint_mismatch + self.hangs + self.leaks


def _solo(model, prompt, sp, block_size, cache: Dict) -> Tuple[List[int], int]:
    key = (tuple(prompt), sp.temperature, sp.seed, sp.max_new_tokens)
    if key not in cache:
        blocks = (len(prompt) + sp.max_new_tokens + 1 + block_size - 1) // block_size + 1
        e = Engine(model, EngineConfig(num_blocks=blocks, block_size=block_size,
                                       max_batched_tokens=max(len(prompt), 1), max_num_seqs=1))
        rid = e.add_request(prompt, sp)
        steps = 0
        while not e.idle() and steps < STEP_LIMIT:
            e.step()
            steps += 1
        cache[key] = (list(e.result(rid).tokens), e.result(rid).logits_fingerprint)
    return cache[key]


def run_traces(model, traces: int = 100, seed: int = 1, only_trace: int = -1, verbose: bool = False,
               block_size: int = 16, max_prompt: int = 48) -> Outcome:
    out = Outcome()
    vocab = model.decoder.head.vocab
    solo_cache: Dict = {}
    for t in range(traces):
        if only_trace >= 0 and t != only_trace:
            continue
        rng = np.random.default_rng([seed, t])
        reqs = []
        for _ in range(int(rng.integers(1, 11))):
            prompt = rng.integers(0, vocab, int(rng.integers(1, max_prompt + 1))).tolist()
            sp = SamplingParams(temperature=float(rng.choice([0.0, 0.0, 0.8, 1.2])), seed=int(rng.integers(0, 1 << 30)),
                                max_new_tokens=int(rng.integers(1, 25)), ignore_eos=True)
            cancel = int(rng.integers(1, 30)) if rng.random() < 0.15 else -1
            reqs.append((prompt, sp, int(rng.integers(0, 12)), cancel))
        need = max((len(p) + sp.max_new_tokens + 1 + block_size - 1) // block_size for p, sp, _, _ in reqs)
        cfg = EngineConfig(num_blocks=need + int(rng.integers(0, 13)), block_size=block_size,
                           max_batched_tokens=int(rng.integers(4, 65)), max_num_seqs=int(rng.integers(1, 9)))
        eng = Engine(model, cfg)
        ids: Dict[int, int] = {}
        cancelled = set()
        step = 0
        hang = False
        while len(ids) < len(reqs) or not eng.idle():
            for i, (prompt, sp, arrive, cancel) in enumerate(reqs):
                if arrive <= step and i not in ids:
                    ids[i] = eng.add_request(prompt, sp)
                if cancel >= 0 and arrive + cancel == step and i in ids and not eng.result(ids[i]).finished:
                    eng.cancel(ids[i])
                    cancelled.add(i)
            eng.step()
            step += 1
            if step > STEP_LIMIT:
                hang = True
                break
        bad = False
        if hang:
            out.hangs += 1
            bad = True
        else:
            for i, rid in ids.items():
                if i in cancelled:
                    continue
                toks, fp = _solo(model, reqs[i][0], reqs[i][1], block_size, solo_cache)
                res = eng.result(rid)
                out.requests_checked += 1
                if res.tokens != toks:
                    out.token_mismatch += 1
                    bad = True
                elif res.logits_fingerprint != fp:
                    out.fingerprint_mismatch += 1
                    bad = True
            if eng.free_blocks != cfg.num_blocks or not eng.manager.all_free():
                out.leaks += 1
                bad = True
        out.preemptions += eng.stats.preemptions
        out.traces += 1
        if bad and out.first_bad_trace < 0:
            out.first_bad_trace = t
        if verbose:
            print(f"trace {t}: {len(reqs)} requests, {step} steps, {eng.stats.preemptions} preemptions, "
                  f"blocks {cfg.num_blocks}, budget {cfg.max_batched_tokens}, seqs {cfg.max_num_seqs}"
                  + (" VIOLATION" if bad else ""), flush=True)
    return out
