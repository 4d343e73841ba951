"""Generation through the Python entry point, the parts alone, and a toy architecture, on the GPU."""
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as P
import replay_patterns as R
import toy_arch
from tiny_configs import TINY, tiny_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _model(folder, dtype):
    from bitwise_b200 import Model
    return Model.load(folder, dtype=dtype, device=DEV)


@pytest.mark.parametrize("name", list(TINY))
def test_generation_float32_equals_plain_tokens_and_fingerprints(name, tiny_folders):
    """The workloads of the two tiny configurations: greedy and temperature sampling through
    scheduler, portions and preemption give the tokens AND the logits fingerprint of the plain
    implementation run on each request alone."""
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    g = TINY[name]["generate"]
    lens = [5, 17, 31] if name == "tiny_a" else [1, 9, 40, 100]
    prompts = [tiny_tokens(name, n, salt=50 + i) for i, n in enumerate(lens)]
    sp = SamplingParams(g["temperature"], g["seed"], g["new"], True)
    plain = P.PlainLlama(tiny_folders[name], exp="det")
    want = [P.generate(plain, p, sp.max_new_tokens, sp.temperature, sp.seed, ignore_eos=True) for p in prompts]
    model = _model(tiny_folders[name], "float32")
    # the second pool is too small for the requests together: they preempt each other
    scarce = 6 if name == "tiny_a" else 10
    for cfg in (EngineConfig(num_blocks=64, max_batched_tokens=256, max_num_seqs=8),
                EngineConfig(num_blocks=scarce, max_batched_tokens=24, max_num_seqs=len(prompts))):
        eng = Engine(model, cfg)
        ids = [eng.add_request(p, sp) for p in prompts]
        steps = 0
        while not eng.idle():
            eng.step()
            steps += 1
            assert steps < 5000
        for rid, (toks, fp) in zip(ids, want):
            assert eng.result(rid).tokens == toks
            assert eng.result(rid).logits_fingerprint == fp
        assert eng.free_blocks == cfg.num_blocks and eng.manager.all_free()
        assert (eng.stats.preemptions > 0) == (cfg.num_blocks == scarce), eng.stats


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(3))
def test_random_traces_equal_requests_run_alone(dtype, seed, tiny_folders):
    """The reference's main oracle (sim/simulate.cpp:102-211): under random arrivals, budgets,
    pool sizes and preemption every request yields the tokens and the logits fingerprint it
    yields alone on an idle engine, in both precisions; nothing leaks, nothing hangs."""
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    rng = np.random.default_rng(100 + seed)
    name = "tiny_a" if seed % 2 == 0 else "tiny_b"
    vocab = TINY[name]["config"].vocab_size
    model = _model(tiny_folders[name], dtype)
    reqs = []
    for i in range(int(rng.integers(4, 9))):
        prompt = rng.integers(0, vocab, int(rng.integers(1, 60))).tolist()
        sp = SamplingParams(float(rng.choice([0.0, 0.8])), int(rng.integers(0, 100)), int(rng.integers(1, 20)), True)
        reqs.append((prompt, sp, int(rng.integers(0, 8))))
    solo = []
    for prompt, sp, _ in reqs:
        e = Engine(model, EngineConfig(num_blocks=32, max_batched_tokens=128, max_num_seqs=1))
        rid = e.add_request(prompt, sp)
        while not e.idle():
            e.step()
        solo.append((e.result(rid).tokens, e.result(rid).logits_fingerprint))
    need = max((len(p) + sp.max_new_tokens + 1 + 15) // 16 for p, sp, _ in reqs)
    eng = Engine(model, EngineConfig(num_blocks=need + int(rng.integers(0, 5)),
                                     max_batched_tokens=int(rng.integers(4, 48)), max_num_seqs=int(rng.integers(1, 5))))
    ids, step = {}, 0
    while len(ids) < len(reqs) or not eng.idle():
        for i, (prompt, sp, arrive) in enumerate(reqs):
            if arrive <= step and i not in ids:
                ids[i] = eng.add_request(prompt, sp)
        eng.step()
        step += 1
        assert step < 5000, "the engine does not go idle"
    for i, rid in ids.items():
        assert eng.result(rid).tokens == solo[i][0], f"request {i}"
        assert eng.result(rid).logits_fingerprint == solo[i][1], f"request {i}: logits differ in bits"
    assert eng.free_blocks == eng.config.num_blocks and eng.manager.all_free()


def test_generation_bfloat16_greedy_agrees_with_plain_where_the_choice_is_clear(tiny_folders):
    """Greedy bfloat16 generation against the plain implementation with the same rounding
    places: every generated token is the plain argmax, or the plain logits of the two differ
    by less than the bfloat16 tolerance of the replay tests (a near tie)."""
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    name = "tiny_a"
    plain = P.PlainLlama(tiny_folders[name], exp="det", round_bf16=True)
    model = _model(tiny_folders[name], "bfloat16")
    prompt = tiny_tokens(name, 17, salt=60)
    got = Engine(model, EngineConfig(num_blocks=16)).generate([prompt], SamplingParams(0.0, 0, 16, True))[0]
    toks = list(prompt)
    for t in got:
        row = plain.logits(toks)[-1]
        assert row.max() - row[t] <= 0.02 * np.abs(row).max(), f"token {t} is no near-maximum at length {len(toks)}"
        toks.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_on_the_gpu(dtype, tmp_path):
    toy_arch.register()
    from bitwise_b200 import Model
    folder = Model.write_random_folder(str(tmp_path / "toy"), toy_arch.ToyConfig(), seed=4)
    model = _model(folder, dtype)
    reqs = {"x": np.random.default_rng(0).integers(0, 97, 90).tolist(),
            "y": np.random.default_rng(1).integers(0, 97, 41).tolist()}
    want = {rid: toy_arch.plain_forward(folder, t, exp="det") for rid, t in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 0.03 * max(np.abs(w).max() for w in want.values())
    for steps in (R.whole(reqs), R.portions(reqs), R.mixed(reqs, 192, seed=5)):
        got = R.collect(steps, R.run_in_process(model, steps, 192), 97)
        for rid in reqs:
            assert np.abs(got[rid] - want[rid]).max() < tol, rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone(dtype, tiny_folders):
    """Each part of a layer run alone through its own forward: norm, attention mixer, SwiGLU
    feed-forward, block, embedding and head, against the plain functions."""
    from bitwise_b200.engine.replay import make_replay_stepper
    from bitwise_b200.engine.step import StepEntry
    name = "tiny_b"
    model = _model(tiny_folders[name], dtype)
    plain = P.PlainLlama(tiny_folders[name], exp="det", round_bf16=(dtype == "bfloat16"))
    c = TINY[name]["config"]
    toks = tiny_tokens(name, 37, salt=70)
    st = make_replay_stepper(model, 64)
    ctx, after = st.prepare([StepEntry("p", toks, [36])])
    views = st.storage.views(ctx.block_tables, ctx.seq_slot)
    dec = model.decoder
    w = plain.w
    act = ctx.act_dtype
    rb = (lambda a: P.bf16_round(a)) if dtype == "bfloat16" else (lambda a: a)
    tol = (lambda want: 1e-30) if dtype == "float32" else (lambda want: 0.02 * np.abs(want).max())

    def close(got, want, what):
        got = got.float().cpu().numpy()
        if dtype == "float32":
            assert np.array_equal(got.view(np.uint32), np.asarray(want, np.float32).view(np.uint32)), what
        else:
            assert np.abs(got - want).max() <= tol(want), what

    # embedding
    x = torch.empty(37, c.hidden_size, device=DEV)
    dec.embedding.forward(ctx, x)
    x0 = w["model.embed_tokens.weight"][np.asarray(toks)]
    if dtype == "bfloat16":
        x0 = P.bf16_round(x0)
    close(x, x0, "embedding")
    # norm
    blk = dec.blocks[0]
    xn = torch.empty(37, c.hidden_size, device=DEV, dtype=act)
    blk.mixer_norm.forward(ctx, x, xn)
    xn0 = rb(P.rmsnorm(x0, w["model.layers.0.input_layernorm.weight"], c.rms_norm_eps))
    close(xn, xn0, "norm")
    # mixer (adds into a copy of the stream)
    xa = x.clone()
    blk.mixer.forward(ctx, xn, xa, views[0])
    pos = np.arange(37)
    p = "model.layers.0."
    q = rb(P.rope(rb(P.linear(xn0, rb(w[p + "self_attn.q_proj.weight"]))).reshape(37, 3, 32), pos, plain.inv_freq))
    k = rb(P.rope(rb(P.linear(xn0, rb(w[p + "self_attn.k_proj.weight"]))).reshape(37, 1, 32), pos, plain.inv_freq))
    v = rb(P.linear(xn0, rb(w[p + "self_attn.v_proj.weight"]))).reshape(37, 1, 32)
    a = rb(P.attention(q, k, v, "det", 0, dtype == "bfloat16")).reshape(37, -1)
    xa0 = (x0 + P.linear(a, rb(w[p + "self_attn.o_proj.weight"]))).astype(np.float32)
    close(xa, xa0, "attention mixer")
    # feed-forward
    xn2 = torch.empty_like(xn)
    blk.ffn_norm.forward(ctx, xa, xn2)
    xf = xa.clone()
    blk.feed_forward.forward(ctx, xn2, xf)
    xn20 = rb(P.rmsnorm(xa0, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps))
    gu = np.concatenate([P.linear(xn20, rb(w[p + "mlp.gate_proj.weight"])), P.linear(xn20, rb(w[p + "mlp.up_proj.weight"]))], 1)
    xf0 = (xa0 + P.linear(rb(P.swiglu(rb(gu), c.intermediate_size, "det")), rb(w[p + "mlp.down_proj.weight"]))).astype(np.float32)
    close(xf, xf0, "feed-forward")
    # the whole block on a fresh stream equals the two halves
    xb = x.clone()
    blk.forward(ctx, xb, views[0])
    assert torch.equal(xb, xf), "block = mixer half + feed-forward half"
    # head on the wanted row
    logits = dec.head.forward(ctx, xf)
    hn = rb(P.rmsnorm(xf0[36:37], w["model.norm.weight"], c.rms_norm_eps))
    close(logits, P.linear(hn, rb(w["lm_head.weight"])), "head")


def test_engine_stops_on_a_raised_failure_word(tiny_folders):
    """The engine reads the kernels' failure word with every step's tokens: a step that follows
    a bounded wait that ran out raises instead of handing out tokens; after that the engine's
    device state is usable and generation gives the right tokens again."""
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    from bitwise_b200.kernels.ops import DeviceFailure
    model = _model(tiny_folders["tiny_a"], "bfloat16")
    sp = SamplingParams(0.0, 0, 6, True)
    prompt = tiny_tokens("tiny_a", 12, salt=91)
    want = Engine(model, EngineConfig(num_blocks=8)).generate([prompt], sp)
    eng = Engine(model, EngineConfig(num_blocks=8))
    eng.add_request(prompt, sp)
    assert model.ops.selftest_bounded_wait(polls=2000) == 2   # a wait ran out somewhere on the device
    with pytest.raises(DeviceFailure):
        for _ in range(3):   # an engine that runs a step ahead reads the word with the step's tokens, a call later
            eng.step()
    assert not model.ops.device_failure()                     # read and cleared by the engine
    assert Engine(model, EngineConfig(num_blocks=8)).generate([prompt], sp) == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_a_step_ahead_changes_no_token(dtype, tiny_folders):
    """The engine launches a step before it has read the tokens of the one before (they go from
    the sampler into the next batch on the device).  Tokens, fingerprints, preemptions and the
    end by an end-of-sequence token are those of the engine that reads every step at once."""
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    name = "tiny_b"
    model = _model(tiny_folders[name], dtype)
    prompts = [tiny_tokens(name, n, salt=70 + i) for i, n in enumerate((1, 9, 40, 100, 23, 64))]
    params = [SamplingParams(0.0 if i % 2 else 0.9, 5 + i, 10 + 3 * i, True) for i in range(len(prompts))]

    def run(lookahead, eos=None, blocks=10):
        if eos is not None:
            model.decoder.config = type(model.config).from_json(dict(model.config.to_json(), eos_token_id=eos))
        eng = Engine(model, EngineConfig(num_blocks=blocks, max_batched_tokens=24, max_num_seqs=4, lookahead=lookahead))
        assert eng._lookahead == lookahead
        ids = [eng.add_request(p, q) for p, q in zip(prompts, params)]
        steps = 0
        while not eng.idle():
            eng.step()
            steps += 1
            assert steps < 5000
        assert eng.free_blocks == blocks and eng.manager.all_free()
        return [(eng.result(i).tokens, eng.result(i).logits_fingerprint) for i in ids], eng.stats.preemptions

    plain, preempted = run(False)
    ahead, preempted_ahead = run(True)
    assert ahead == plain and preempted > 0 and preempted_ahead == preempted
    # a token that ends requests early: the most frequent one of the free runs
    flat = [t for toks, _ in plain for t in toks]
    eos = max(set(flat), key=flat.count)
    old = model.config.eos_token_id
    try:
        stop = [SamplingParams(q.temperature, q.seed, q.max_new_tokens, False) for q in params]
        params, keep = stop, params
        a, _ = run(False, eos)
        b, _ = run(True, eos)
        params = keep
    finally:
        model.decoder.config = type(model.config).from_json(dict(model.config.to_json(), eos_token_id=old))
    assert a == b
    assert any(toks and toks[-1] == eos and len(toks) < q.max_new_tokens for (toks, _), q in zip(a, keep))
