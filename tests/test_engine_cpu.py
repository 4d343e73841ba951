"""The engine's host logic without a GPU: the kernels are replaced by the CPU stand-in of
tests/cpu_ops.py (the package itself has no CPU path), everything else is the product:
batch building, block tables, page reuse, the run order of layers, scheduler, sampler keys.
Comparisons with the plain implementation use a tolerance here, because the stand-in's
arithmetic is ordinary torch; the bit-exact comparisons are the GPU tests."""
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as P
import replay_patterns as R
import toy_arch
from cpu_ops import CpuOps
from tiny_configs import TINY, tiny_tokens

from bitwise_b200 import Engine, EngineConfig, Model, SamplingParams
from bitwise_b200.engine.step import OutOfPages, StepEntry, StepError

TOL = 2e-5


def cpu_model(folder):
    return Model.load(folder, "float32", device="cpu", ops=CpuOps("float32"))


@pytest.mark.parametrize("name", list(TINY))
def test_replay_patterns_on_the_stand_in(name, tiny_folders):
    lens = {"tiny_a": [70, 45, 33, 5, 64], "tiny_b": [100, 40, 9, 1, 65]}[name]
    reqs = {f"{name}-{i}": tiny_tokens(name, n, salt=i) for i, n in enumerate(lens)}
    plain = P.PlainLlama(tiny_folders[name], exp="libm")
    want = {rid: plain.logits(t) for rid, t in reqs.items()}
    model = cpu_model(tiny_folders[name])
    vocab = TINY[name]["config"].vocab_size
    for steps, max_tokens in ((R.whole(reqs), 128), (R.tail_one_by_one(reqs, 8), 128), (R.portions(reqs), 128),
                              (R.mixed(reqs, 256, seed=2), 256)):
        got = R.collect(steps, R.run_in_process(model, steps, max_tokens), vocab)
        for rid in reqs:
            assert np.abs(got[rid] - want[rid]).max() < TOL


def test_model_logits_entry_point(tiny_folders):
    toks = tiny_tokens("tiny_a", 21)
    got = cpu_model(tiny_folders["tiny_a"]).logits(toks)
    assert got.shape == (21, 256)
    assert np.abs(got - P.PlainLlama(tiny_folders["tiny_a"]).logits(toks)).max() < TOL


def test_step_function_refuses_what_it_cannot_run(tiny_folders):
    from bitwise_b200.engine.replay import make_replay_stepper
    st = make_replay_stepper(cpu_model(tiny_folders["tiny_a"]), 64)
    with pytest.raises(StepError):
        st.run([])
    with pytest.raises(StepError):
        st.run([StepEntry("a", [1, 2], [2])])        # wanted place outside the tokens
    with pytest.raises(StepError):
        st.run([StepEntry("a", [1, 999], [])])       # token outside the vocabulary
    with pytest.raises(StepError):
        st.run([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    st.run([StepEntry("a", list(range(40)), [])])
    with pytest.raises(StepError):
        st.run([StepEntry("a", list(range(30)), [])])  # 70 tokens: beyond the 64 the table covers
    with pytest.raises(OutOfPages):
        st.run([StepEntry("b", list(range(40)), [])])  # the pool of 4 pages is spent
    assert st.run([StepEntry("a", [5], [])]) is None   # nothing wanted: no logits


@pytest.mark.parametrize("name,blocks,budget,seqs", [("tiny_a", 64, 24, 4), ("tiny_a", 5, 16, 4), ("tiny_b", 9, 7, 3)])
def test_generation_equals_the_plain_sampler(name, blocks, budget, seqs, tiny_folders):
    """Tokens through scheduler, portions, preemption and recompute equal the tokens of each
    request run alone by the plain implementation (the reference's oracle,
    sim/simulate.cpp:102-118)."""
    plain = P.PlainLlama(tiny_folders[name], exp="libm")
    prompts = [tiny_tokens(name, n, salt=i) for i, n in enumerate([5, 17, 31, 9])]
    params = [SamplingParams(0.0, 0, 8, True), SamplingParams(0.8, 7, 8, True), SamplingParams(0.0, 0, 6, True),
              SamplingParams(1.1, 3, 8, True)]
    want = [P.generate(plain, p, q.max_new_tokens, q.temperature, q.seed, ignore_eos=True)[0]
            for p, q in zip(prompts, params)]
    eng = Engine(cpu_model(tiny_folders[name]), EngineConfig(num_blocks=blocks, max_batched_tokens=budget,
                                                             max_num_seqs=seqs))
    got = eng.generate(prompts, params)
    assert got == want
    eng.manager.check_consistency()
    assert eng.manager.all_free() and eng.free_blocks == blocks
    if blocks == 5:
        assert eng.stats.preemptions > 0


def test_engine_surface(tiny_folders):
    eng = Engine(cpu_model(tiny_folders["tiny_a"]), EngineConfig(num_blocks=8, max_batched_tokens=16, max_num_seqs=2))
    with pytest.raises(ValueError):
        eng.add_request([])
    with pytest.raises(ValueError):
        eng.add_request([1, 2, 300])
    with pytest.raises(ValueError) as e:
        eng.add_request(list(range(100)), SamplingParams(max_new_tokens=40))
    assert "never fit" in str(e.value)
    a = eng.add_request([1, 2, 3], SamplingParams(max_new_tokens=3, ignore_eos=True))
    b = eng.add_request([4, 5], SamplingParams(max_new_tokens=50, ignore_eos=True))
    assert eng.num_waiting == 2 and not eng.idle()
    ev = eng.step()
    assert {x.id for x in ev} == {a, b} and eng.num_running == 2
    eng.cancel(b)
    assert eng.result(b).cancelled and eng.result(b).finished
    while not eng.idle():
        eng.step()
    r = eng.result(a)
    assert r.finished and not r.cancelled and len(r.tokens) == 3 and len(r.token_times) == 3
    assert eng.free_blocks == 8 and eng.stats.generated_tokens >= 4


def test_eos_stops_a_request(tiny_folders):
    model = cpu_model(tiny_folders["tiny_a"])
    prompt = tiny_tokens("tiny_a", 6)
    free = Engine(model, EngineConfig(num_blocks=16)).generate([prompt], SamplingParams(max_new_tokens=12, ignore_eos=True))[0]
    eos = free[4]
    model.decoder.config = type(model.config).from_json(dict(model.config.to_json(), eos_token_id=eos))
    stopped = Engine(model, EngineConfig(num_blocks=16)).generate([prompt], SamplingParams(max_new_tokens=12))[0]
    assert stopped == free[:free.index(eos) + 1]


@pytest.mark.parametrize("seed", range(3))
def test_random_traces_against_requests_run_alone(seed, tiny_folders):
    """Random arrivals, budgets and pool sizes: every request gives the tokens it gives
    alone on an idle engine; the engine goes idle and returns every page (the reference's
    simulator, sim/simulate.cpp:120-211).  The logits fingerprints are compared in the GPU
    tests only: the stand-in's torch arithmetic is not bit-invariant to the batch."""
    rng = np.random.default_rng(seed)
    model = cpu_model(tiny_folders["tiny_a"])
    reqs = []
    for i in range(int(rng.integers(3, 8))):
        prompt = rng.integers(0, 256, int(rng.integers(1, 40))).tolist()
        sp = SamplingParams(float(rng.choice([0.0, 0.7, 1.0])), int(rng.integers(0, 100)), int(rng.integers(1, 12)), True)
        reqs.append((prompt, sp, int(rng.integers(0, 6))))
    solo = []
    for prompt, sp, _ in reqs:
        e = Engine(model, EngineConfig(num_blocks=32, max_batched_tokens=64, max_num_seqs=1))
        rid = e.add_request(prompt, sp)
        while not e.idle():
            e.step()
        solo.append((e.result(rid).tokens, e.result(rid).logits_fingerprint))
    need = max((len(p) + sp.max_new_tokens + 1 + 15) // 16 for p, sp, _ in reqs)
    eng = Engine(model, EngineConfig(num_blocks=need + int(rng.integers(0, 6)), max_batched_tokens=int(rng.integers(4, 40)),
                                     max_num_seqs=int(rng.integers(1, 5))))
    ids, step = {}, 0
    while len(ids) < len(reqs) or not eng.idle():
        for i, (prompt, sp, arrive) in enumerate(reqs):
            if arrive == step or (arrive < step and i not in ids):
                if i not in ids:
                    ids[i] = eng.add_request(prompt, sp)
        eng.step()
        step += 1
        assert step < 5000, "the engine does not go idle"
    for i, rid in ids.items():
        assert eng.result(rid).tokens == solo[i][0]
    assert eng.free_blocks == eng.config.num_blocks and eng.manager.all_free()


def test_toy_architecture_with_parts_of_its_own(tmp_path):
    """A mixer with a state slot, a routed feed-forward, a learned position table, a windowed
    layer, a layer run twice and a run that reads another run's cache: registered, built,
    loaded and stepped through the unchanged framework."""
    toy_arch.register()
    cfg = toy_arch.ToyConfig()
    folder = Model.write_random_folder(str(tmp_path / "toy"), cfg, seed=4)
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyMixForCausalLM"]
    model = cpu_model(folder)
    assert [type(g).__name__ for g in model.decoder.cache_needs()] == ["PagedKVNeed", "SlotStateNeed", "PagedKVNeed",
                                                                       "SlotStateNeed"]
    reqs = {"x": np.random.default_rng(0).integers(0, 97, 90).tolist(),
            "y": np.random.default_rng(1).integers(0, 97, 41).tolist()}
    want = {rid: toy_arch.plain_forward(folder, t, exp="libm") for rid, t in reqs.items()}
    for steps in (R.whole(reqs), R.portions(reqs), R.mixed(reqs, 192, seed=5)):
        got = R.collect(steps, R.run_in_process(model, steps, 192), 97)
        for rid in reqs:
            assert np.abs(got[rid] - want[rid]).max() < 1e-4, rid
    # the windowed group gives pages back while a long request is still running
    from bitwise_b200.engine.replay import make_replay_stepper
    st = make_replay_stepper(model, 128)
    st.run([StepEntry("z", reqs["x"][:80], [])])
    full, windowed = [g.window for g in st.manager.groups].index(None), [g.window for g in st.manager.groups].index(24)
    assert st.manager.available(full) == 8 - 5 and st.manager.available(windowed) > 8 - 5
    st.finish("z")
    assert st.manager.all_free()
