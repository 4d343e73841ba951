"""The tiny configurations of the tests.  They differ in every size and option: head
counts and groups (4/2 vs 3/1), head size (16 vs 32), a feed-forward width that is no
multiple of 16 (172) vs a power of two, widths 64 vs 96, layers 2 vs 3, vocabulary 256 vs
384, eps 1e-5 vs 1e-6, tied vs untied head, plain rotary vs llama3-rescaled rotary, norm
weights 1 vs 1 + U(-0.1, 0.1), float32 vs bfloat16 checkpoint.  A third one is wider
(heads 5/5, head size 48) for the kernels' other code paths."""
import numpy as np

from bitwise_b200 import LlamaConfig, Model, RopeScaling

TINY = {
    "tiny_a": dict(
        config=LlamaConfig(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=172, rope_theta=10000.0,
                           rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128,
                           eos_token_id=2),
        seed=11, norm_jitter=0.0, file_dtype="float32", tokens=45,
        generate=dict(prompt_len=17, new=16, temperature=0.0, seed=0)),
    "tiny_b": dict(
        config=LlamaConfig(vocab_size=384, hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
                           num_key_value_heads=1, head_dim=32, intermediate_size=256, rope_theta=500000.0,
                           rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256,
                           rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 64), eos_token_id=5),
        seed=23, norm_jitter=0.1, file_dtype="bfloat16", tokens=70,
        generate=dict(prompt_len=9, new=24, temperature=0.8, seed=7)),
}


# For contexts of several hundred keys (key tiles, graph buckets, the streaming decode kernel
# and the tensor-core prefill attention want head size 64); not part of TINY, whose members every
# parametrised test runs.
LONG = {
    "tiny_long": dict(
        config=LlamaConfig(vocab_size=320, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=64, intermediate_size=192, rope_theta=50000.0,
                           rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024),
        seed=31, norm_jitter=0.05, file_dtype="bfloat16", tokens=640),
}


def tiny_tokens(name, count=None, salt=0):
    spec = TINY.get(name) or LONG[name]
    rng = np.random.default_rng(1000 + spec["seed"] + salt)
    return rng.integers(0, spec["config"].vocab_size, count or spec["tokens"]).tolist()


def write_tiny_folder(folder, name):
    spec = TINY.get(name) or LONG[name]
    return Model.write_random_folder(folder, spec["config"], seed=spec["seed"], dtype=spec["file_dtype"],
                                     norm_jitter=spec["norm_jitter"])
