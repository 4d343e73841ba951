"""Contexts of several hundred keys through the step function, in both precisions.

The tiny models of the other tests hold at most 100 keys; everything that depends on a longer
context is met only here: key tiles of 64 beyond the second, the decode attention that gives
every tile a block of its own and merges the records, the streaming decode kernel (steps of 32
rows or more, head size 64), the tensor-core prefill attention, and CUDA graphs that are
captured at one context length and replayed at others.  A decode step that is replayed as a
graph must give what an eager step gives at every position, also right after a tile of 64 keys
or the graph's bound on the context (256 keys) has been passed; the reference's step function
has no such hazard because it recomputes everything from its arguments
(src/model.cpp:267-322), and its own test walks positions one by one against whole prompts
and against portions {3, 17, 1, 19} (tests/test_main.cpp:200-228).
"""
import numpy as np
import pytest

import plain_llama as P
import replay_patterns as R
from tiny_configs import tiny_tokens

pytestmark = pytest.mark.gpu

BF16_MAX, BF16_MEAN = 0.02, 0.005   # as in test_replay_gpu.py: of the largest logit of the request
LENGTH = 640


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _model(folder, dtype):
    from bitwise_b200 import Model
    return Model.load(folder, dtype=dtype, device="cuda:0")


def _same_bits(got, want, what):
    bad = _bits(got) != _bits(want)
    assert not bad.any(), (f"{what}: {int(bad.sum())} values differ in bits, first wrong position "
                           f"{int(np.argwhere(bad.any(axis=1))[0][0])} of {got.shape[0]}; "
                           f"max abs diff {np.abs(got - want).max():.3e}")


def _near(got, want, what):
    scale = np.abs(want).max()
    err = np.abs(got - want)
    assert err.max() <= BF16_MAX * scale and err.mean() <= BF16_MEAN * scale, (
        f"{what}: max error {err.max() / scale:.4f}, mean {err.mean() / scale:.5f} of the largest logit; "
        f"worst position {int(np.argmax(err.max(axis=1)))}")


def _one_by_one(rid, toks, head):
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []}]
    for i in range(head, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                      "end": [rid] if i == len(toks) - 1 else []})
    return steps


@pytest.mark.parametrize("name", ["tiny_long", "tiny_b", "tiny_a"])
def test_bfloat16_one_request_token_by_token_past_600_keys(name, tiny_folders):
    """Prompt of 100 tokens, then one token a step up to 640: replayed graphs = eager steps =
    the whole prompt = portions {3, 17, 1, 19}, bit for bit, and all of it near the plain
    implementation."""
    toks = tiny_tokens(name, LENGTH, salt=5)
    reqs = {"r": toks}
    model = _model(tiny_folders[name], "bfloat16")
    vocab = model.decoder.head.vocab
    pool = (LENGTH + 63) // 64 * 64
    whole = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), pool), vocab)["r"]
    want = P.PlainLlama(tiny_folders[name], exp="det", round_bf16=True).logits(toks)
    _near(whole, want, f"{name} whole")
    steps = _one_by_one("r", toks, 100)
    info = {}
    graphs = R.collect(steps, R.run_in_process(model, steps, pool, info=info), vocab)["r"]
    assert info["use_graphs"] and info["graph_replays"] > 400, info
    _same_bits(graphs, whole, f"{name} decode with graphs vs whole")
    eager = R.collect(steps, R.run_in_process(model, steps, pool, use_graphs=False, info=info), vocab)["r"]
    assert info["graph_replays"] == 0
    _same_bits(eager, whole, f"{name} decode without graphs vs whole")
    cut = R.portions(reqs, sizes=(3, 17, 1, 19))
    _same_bits(R.collect(cut, R.run_in_process(model, cut, pool), vocab)["r"], whole, f"{name} portions vs whole")


@pytest.mark.parametrize("name,length", [("tiny_long", 640), ("tiny_b", 330)])
def test_float32_token_by_token_past_300_keys(name, length, tiny_folders):
    """The exact path at the same kind of lengths: whole = one by one = portions = the plain
    implementation, bit for bit.  The whole prompt of 640 rows with 4 heads is more (row, head)
    pairs than 16 per SM: it takes the attention variant that reads the values straight from the
    cache, which every real prompt takes and no tiny one."""
    toks = tiny_tokens(name, length, salt=6)
    reqs = {"r": toks}
    model = _model(tiny_folders[name], "float32")
    vocab = model.decoder.head.vocab
    want = P.PlainLlama(tiny_folders[name], exp="det").logits(toks)
    for what, steps in (("whole", R.whole(reqs)), ("one by one", _one_by_one("r", toks, 70)),
                        ("portions", R.portions(reqs, sizes=(3, 17, 1, 19)))):
        got = R.collect(steps, R.run_in_process(model, steps, (length + 63) // 64 * 64), vocab)["r"]
        _same_bits(got, want, f"{name} float32 {what}")


def _together(reqs, heads):
    """Every request's prompt head in a step of its own, then all live requests decode one token
    each per step; requests end when their tokens are used up."""
    steps = []
    nxt = {}
    for rid, toks in reqs.items():
        h = heads[rid]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:h], "want": list(range(h))}], "end": []})
        nxt[rid] = h
    while nxt:
        entries, end = [], []
        for rid in list(nxt):
            i = nxt[rid]
            entries.append({"id": rid, "tokens": reqs[rid][i:i + 1], "want": [0]})
            nxt[rid] = i + 1
            if i + 1 == len(reqs[rid]):
                end.append(rid)
                del nxt[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


@pytest.mark.parametrize("name", ["tiny_long", "tiny_b"])
def test_bfloat16_batch_of_different_lengths_replays_graphs(name, tiny_folders):
    """Three requests of different lengths decoded together: the step's graph is captured while
    the longest context is short and replayed as the contexts grow past tile and bound edges;
    when a request ends the batch shape changes.  Each request = its whole run, bit for bit."""
    lengths = {"a": (100, 620), "b": (37, 300), "c": (230, 640)}
    reqs = {rid: tiny_tokens(name, n, salt=20 + i) for i, (rid, (_, n)) in enumerate(lengths.items())}
    heads = {rid: h for rid, (h, _) in lengths.items()}
    model = _model(tiny_folders[name], "bfloat16")
    vocab = model.decoder.head.vocab
    pool = sum((len(t) + 63) // 64 * 64 for t in reqs.values())
    whole = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), pool), vocab)
    steps = _together(reqs, heads)
    info = {}
    graphs = R.collect(steps, R.run_in_process(model, steps, pool, info=info), vocab)
    assert info["graph_replays"] > 300, info
    eager = R.collect(steps, R.run_in_process(model, steps, pool, use_graphs=False), vocab)
    for rid in reqs:
        _same_bits(graphs[rid], whole[rid], f"{name} {rid} together with graphs vs whole")
        _same_bits(eager[rid], whole[rid], f"{name} {rid} together without graphs vs whole")
    want = P.PlainLlama(tiny_folders[name], exp="det", round_bf16=True).logits(reqs["b"])
    _near(whole["b"], want, f"{name} b whole")


def test_bfloat16_many_requests_through_the_streaming_kernel(tiny_folders):
    """34 live requests (the streaming decode kernel takes steps of 32 rows or more at head size
    64) whose contexts pass 128, 192 and 256 keys while they decode together."""
    name = "tiny_long"
    model = _model(tiny_folders[name], "bfloat16")
    c = model.decoder.config
    lib = model.ops._attention_lib(c.head_dim)
    assert lib.bw_bf16_attention_stream_usable(34, c.num_attention_heads, c.num_key_value_heads, c.head_dim, 16,
                                               (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim)
    reqs, heads = {}, {}
    for i in range(34):
        heads[f"s{i}"] = 110 + 3 * i                      # 110 .. 209 keys when decoding starts
        reqs[f"s{i}"] = tiny_tokens(name, heads[f"s{i}"] + 90 - (i % 5), salt=40 + i)
    vocab = model.decoder.head.vocab
    pool = sum((len(t) + 63) // 64 * 64 for t in reqs.values())
    steps = _together(reqs, heads)
    info = {}
    graphs = R.collect(steps, R.run_in_process(model, steps, pool, max_live=34, info=info), vocab)
    assert info["graph_replays"] > 40, info
    eager = R.collect(steps, R.run_in_process(model, steps, pool, max_live=34, use_graphs=False), vocab)
    whole_steps = R.whole(reqs)
    whole = R.collect(whole_steps, R.run_in_process(model, whole_steps, 320), vocab)
    for rid in reqs:
        _same_bits(graphs[rid], whole[rid], f"{rid} with graphs vs whole")
        _same_bits(eager[rid], whole[rid], f"{rid} without graphs vs whole")
    plain = P.PlainLlama(tiny_folders[name], exp="det", round_bf16=True)
    for rid in ("s0", "s33"):
        _near(whole[rid], plain.logits(reqs[rid]), f"{rid} whole")
