"""The engine against the plain implementation, with the same requests cut in every way.

For each tiny configuration, in float32 and in bfloat16: each request alone and whole;
most of it in one step and the last 32 tokens one by one; portions of changing size; mixed
steps with up to four live requests over a pool so small that pages are used again.
float32 must reproduce the plain implementation (reproducible exp) bit for bit in every
pattern.  bfloat16 is compared with the plain implementation that rounds to bfloat16 where
the engine stores bfloat16; its patterns must agree with each other bit for bit.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as P
import replay_patterns as R
from tiny_configs import TINY, tiny_tokens

pytestmark = pytest.mark.gpu

# lengths up to 100 stay within two key tiles of 64; the longer ones cross tile edges and the
# 256-key bound under which a decode step's graph is kept
LENGTHS = {"tiny_a": [70, 45, 33, 5, 200, 64, 17, 131], "tiny_b": [100, 40, 9, 330, 1, 65, 33, 257]}
# bfloat16 against the plain implementation with the same rounding places: errors are a few
# bfloat16 steps (2^-8 relative) carried through the layers; bound the worst logit error by
# 2 % and the mean error by 0.5 % of the largest logit of the request.
BF16_MAX, BF16_MEAN = 0.02, 0.005


def _requests(name):
    return {f"{name}-{i}": tiny_tokens(name, n, salt=i) for i, n in enumerate(LENGTHS[name])}


_expected = {}


def expected(name, folder, mode):
    key = (name, mode)
    if key not in _expected:
        m = P.PlainLlama(folder, exp="det", round_bf16=(mode == "bfloat16"))
        _expected[key] = {rid: m.logits(toks) for rid, toks in _requests(name).items()}
    return _expected[key]


def _model(folder, dtype):
    from bitwise_b200 import Model
    return Model.load(folder, dtype=dtype, device="cuda:0")


def _patterns(reqs):
    return {
        "whole": (R.whole(reqs), 384),
        "tail": (R.tail_one_by_one(reqs), 384),
        "portions": (R.portions(reqs), 384),
        "mixed": (R.mixed(reqs, 704, seed=3), 704),
        "mixed-tight": (R.mixed(reqs, 448, seed=4), 448),
    }


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("name", list(TINY))
def test_float32_is_bit_exact_in_every_pattern(name, tiny_folders):
    reqs = _requests(name)
    want = expected(name, tiny_folders[name], "float32")
    model = _model(tiny_folders[name], "float32")
    vocab = TINY[name]["config"].vocab_size
    for pname, (steps, max_tokens) in _patterns(reqs).items():
        got = R.collect(steps, R.run_in_process(model, steps, max_tokens), vocab)
        for rid in reqs:
            bad = _bits(got[rid]) != _bits(want[rid])
            if bad.any():
                first = int(np.argwhere(bad.any(axis=1))[0][0])
                raise AssertionError(
                    f"{name} {pname} {rid}: {int(bad.sum())} values differ in bits, first wrong position "
                    f"{first} of {len(reqs[rid])}; max abs diff {np.abs(got[rid] - want[rid]).max():.3e}")


@pytest.mark.parametrize("name", list(TINY))
def test_bfloat16_matches_plain_and_itself(name, tiny_folders):
    reqs = _requests(name)
    want = expected(name, tiny_folders[name], "bfloat16")
    model = _model(tiny_folders[name], "bfloat16")
    vocab = TINY[name]["config"].vocab_size
    results = {}
    for pname, (steps, max_tokens) in _patterns(reqs).items():
        got = R.collect(steps, R.run_in_process(model, steps, max_tokens), vocab)
        results[pname] = got
        for rid in reqs:
            scale = np.abs(want[rid]).max()
            err = np.abs(got[rid] - want[rid])
            assert err.max() <= BF16_MAX * scale and err.mean() <= BF16_MEAN * scale, (
                f"{name} {pname} {rid}: max error {err.max() / scale:.4f}, mean {err.mean() / scale:.5f} of the "
                f"largest logit; worst position {int(np.argmax(err.max(axis=1)))}")
    for pname, got in results.items():
        for rid in reqs:
            bad = _bits(got[rid]) != _bits(results["whole"][rid])
            assert not bad.any(), (f"{name} {rid}: pattern {pname} differs from 'whole' in {int(bad.sum())} values, "
                                   f"first wrong position {int(np.argwhere(bad.any(axis=1))[0][0])}")


def test_long_decoding_and_first_tokens(tiny_folders):
    """A prompt of one token, then 120 tokens decoded one by one (float32, bit exact)."""
    name = "tiny_b"
    toks = tiny_tokens(name, 121, salt=77)
    want = P.PlainLlama(tiny_folders[name], exp="det").logits(toks)
    model = _model(tiny_folders[name], "float32")
    steps = [{"step": i, "entries": [{"id": "d", "tokens": [toks[i]], "want": [0]}], "end": []} for i in range(121)]
    steps[-1]["end"] = ["d"]
    got = R.collect(steps, R.run_in_process(model, steps, 128), want.shape[1])["d"]
    bad = _bits(got) != _bits(want)
    assert not bad.any(), f"first wrong position {int(np.argwhere(bad.any(axis=1))[0][0])}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tiny_folders, tmp_path):
    """bin/trace_run as a user calls it: steps on standard input, <step>.f32 files out."""
    name = "tiny_a"
    reqs = {k: v for k, v in list(_requests(name).items())[:3]}
    steps = R.mixed(reqs, 256, seed=9)
    out = tmp_path / "out"
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    proc = subprocess.run([sys.executable, exe, "--model", tiny_folders[name], "--dtype", dtype, "--out", str(out),
                           "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["config"].vocab_size
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    got = R.collect(steps, outs, vocab)
    want = expected(name, tiny_folders[name], dtype)
    for rid in reqs:
        if dtype == "float32":
            assert not (_bits(got[rid]) != _bits(want[rid])).any()
        else:
            scale = np.abs(want[rid]).max()
            assert np.abs(got[rid] - want[rid]).max() <= BF16_MAX * scale
