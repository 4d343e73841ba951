"""The scheduler, the cache manager and the engine's bookkeeping against the reference's own
Engine, decision for decision.

tests/golden/sched_traces.json holds small workloads that tests/golden/make_golden.py ran
through tkran2/bitwise's unmodified Engine (src/engine.cpp:304-488) with few blocks, small
token budgets, staggered arrivals and cancellations: after every step the state of every
running and waiting request (tokens, computed tokens, blocks held), the step's events and the
engine's counters.  The same workloads run here through this package's Engine (kernels replaced
by the CPU stand-in of the tests; eos is ignored, so the schedule does not depend on the
tokens) and must pass through exactly the same states: which request runs how many rows, who
is preempted when, in which order the preempted return, what a failed admission gives back.
The first trace is the reference's own scarce configuration, nine blocks
(tests/test_main.cpp:274-279).
"""
import json
import os
import struct

import pytest

from cpu_ops import CpuOps

from bitwise_b200 import Engine, EngineConfig, Model, SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))
TRACES = json.load(open(os.path.join(HERE, "golden", "sched_traces.json")))


def _state(eng):
    rows = []
    for tag, seqs in (("running", eng.scheduler.running), ("waiting", eng.scheduler.waiting)):
        for s in seqs:
            blocks = eng.manager.get(s.id).table_len(0) if eng.manager.has(s.id) else 0
            rows.append([tag, s.id, len(s.tokens), s.computed, blocks])
    return rows


@pytest.mark.parametrize("index", range(len(TRACES)))
def test_engine_passes_through_the_reference_engines_states(index, tiny_folders):
    t = TRACES[index]
    model = Model.load(tiny_folders["tiny_a"], "float32", device="cpu", ops=CpuOps("float32"))
    vocab = model.decoder.head.vocab
    eng = Engine(model, EngineConfig(num_blocks=t["num_blocks"], block_size=16,
                                     max_batched_tokens=t["max_batched_tokens"], max_num_seqs=t["max_num_seqs"]))
    reqs = t["requests"]
    ids = {}
    for want in t["steps"]:
        step = want["step"]
        for i, (arrival, prompt_len, max_new, cancel) in enumerate(reqs):
            if i not in ids and arrival <= step:
                prompt = [(i * 7 + j * 3 + 1) % vocab for j in range(prompt_len)]
                ids[i] = eng.add_request(prompt, SamplingParams(0.0, 0, max_new, True))
            if i in ids and cancel >= 0 and arrival + cancel == step:
                eng.cancel(ids[i])
        events = eng.step()
        where = f"trace {index} step {step}"
        assert [[e.id, len(e.tokens), int(e.finished)] for e in events] == want["events"], where
        s = eng.stats
        assert (s.prefill_tokens, s.decode_rows, s.preemptions, s.generated_tokens) == (
            want["prefill_tokens"], want["decode_rows"], want["preemptions"], want["generated"]), where
        assert (eng.num_running, eng.num_waiting, eng.free_blocks) == (
            want["running"], want["waiting"], want["free_blocks"]), where
        assert _state(eng) == want["seqs"], where
    assert eng.idle() and len(ids) == len(reqs)
    assert eng.manager.all_free()
    eng.manager.check_consistency()


def test_traces_hold_what_they_are_meant_to():
    """The stored workloads do exercise preemption, recompute and cancellation."""
    assert TRACES[0]["num_blocks"] == 9 and TRACES[0]["steps"][-1]["preemptions"] > 0
    assert sum(t["steps"][-1]["preemptions"] for t in TRACES) > 50
    assert any(r[3] >= 0 for t in TRACES for r in t["requests"])


def test_counter_uniform_equals_the_references_values():
    """counter_uniform(seed, position, stream) as printed by the reference's own function
    (src/engine.cpp:35-38), bit for bit, for the package's generator and the plain one."""
    import plain_llama as P
    from bitwise_b200.sampling import counter_uniform
    table = json.load(open(os.path.join(HERE, "golden", "counter_uniform.json")))
    assert len(table) >= 100
    for row in table:
        want = struct.unpack("<d", struct.pack("<Q", int(row["bits"], 16)))[0]
        assert 0.0 <= want < 1.0
        assert counter_uniform(row["seed"], row["position"], row["stream"]) == want, row
        assert P.counter_uniform(row["seed"], row["position"], row["stream"]) == want, row
