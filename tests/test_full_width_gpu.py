"""The 32-bit path and the serving path at real widths, and at head size 128.

The tiny models never reach the code that full-size models run: inner sizes of 2,048 and
8,192 in the products (many k-chunks, the streaming tile of steps of few rows next to the big
tile of prompts), 32 heads of 64, and the attention variant that the 32-bit path takes when a
step has more (row, head) pairs than a few waves of thread blocks.  One layer of the
SmolLM2-1.7B shape (hidden 2,048, feed-forward 8,192, 32 heads of 64; the vocabulary cut to
512 rows so that the plain implementation, whose products are loops over k, finishes in
half a minute) is run whole, in portions and token by token and compared with the plain
implementation: bit for bit in float32, as the reference checks its own kernels over hundreds
of shapes against one fixed-order loop (tests/test_main.cpp:71-120) and its model token by
token against whole prompts (tests/test_main.cpp:200-228).
"""
import numpy as np
import pytest

import plain_llama as P
import replay_patterns as R
from bitwise_b200 import LlamaConfig, Model, RopeScaling

pytestmark = pytest.mark.gpu

BF16_MAX, BF16_MEAN = 0.02, 0.005

WIDE = LlamaConfig(vocab_size=512, hidden_size=2048, num_hidden_layers=1, num_attention_heads=32,
                   num_key_value_heads=32, head_dim=64, intermediate_size=8192, rope_theta=130000.0,
                   rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=4096)
# grouped heads of 128 as in Llama-3-8B, in small
HEAD128 = LlamaConfig(vocab_size=300, hidden_size=192, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, intermediate_size=320, rope_theta=500000.0,
                      rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024,
                      rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 128))


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _tokens(cfg, n, salt):
    return np.random.default_rng(900 + salt).integers(0, cfg.vocab_size, n).tolist()


def _one_by_one(rid, toks, head):
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []}]
    for i in range(head, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                      "end": [rid] if i == len(toks) - 1 else []})
    return steps


def _patterns(toks, sizes):
    reqs = {"r": toks}
    return {"whole": R.whole(reqs), "one by one": _one_by_one("r", toks, 1), "portions": R.portions(reqs, sizes=sizes)}


def _check(folder, cfg, toks, sizes, pool):
    vocab = cfg.vocab_size
    m32 = Model.load(folder, dtype="float32", device="cuda:0")
    want = P.PlainLlama(folder, exp="det").logits(toks)
    for what, steps in _patterns(toks, sizes).items():
        got = R.collect(steps, R.run_in_process(m32, steps, pool), vocab)["r"]
        bad = _bits(got) != _bits(want)
        assert not bad.any(), (f"float32 {what}: {int(bad.sum())} values differ in bits, first wrong position "
                               f"{int(np.argwhere(bad.any(axis=1))[0][0])}; max abs diff {np.abs(got - want).max():.3e}")
    del m32
    m16 = Model.load(folder, dtype="bfloat16", device="cuda:0")
    want = P.PlainLlama(folder, exp="det", round_bf16=True).logits(toks)
    first = None
    for what, steps in _patterns(toks, sizes).items():
        got = R.collect(steps, R.run_in_process(m16, steps, pool), vocab)["r"]
        scale = np.abs(want).max()
        err = np.abs(got - want)
        assert err.max() <= BF16_MAX * scale and err.mean() <= BF16_MEAN * scale, (
            f"bfloat16 {what}: max error {err.max() / scale:.4f}, mean {err.mean() / scale:.5f} of the largest logit")
        if first is None:
            first = got
        else:
            assert not (_bits(got) != _bits(first)).any(), f"bfloat16 {what} differs from the whole prompt in bits"


def test_one_layer_at_full_width(tmp_path):
    folder = Model.write_random_folder(str(tmp_path / "wide"), WIDE, seed=5, dtype="bfloat16")
    _check(folder, WIDE, _tokens(WIDE, 12, 1), (3, 5, 1, 2), 64)


def test_heads_of_128(tmp_path):
    folder = Model.write_random_folder(str(tmp_path / "hd128"), HEAD128, seed=8, dtype="float32", norm_jitter=0.1)
    _check(folder, HEAD128, _tokens(HEAD128, 150, 2), (3, 17, 1, 19, 40), 192)
