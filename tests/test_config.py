"""Configuration and registry (no GPU)."""
import json

import pytest

from bitwise_b200.config import (ConfigError, LlamaConfig, RopeScaling, architecture_of, config_from_folder,
                                 known_architectures, lookup_architecture)

BASE = dict(architectures=["LlamaForCausalLM"], vocab_size=100, hidden_size=48, num_hidden_layers=2,
            num_attention_heads=3, intermediate_size=80)


def test_defaults_follow_the_reference_converter():
    c = LlamaConfig.from_json(BASE)
    assert c.num_key_value_heads == 3 and c.head_dim == 16           # tools/convert.py:64-72
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6        # tools/convert.py:74-75
    assert c.tie_word_embeddings is False and c.eos_token_id == -1   # tools/convert.py:77-80
    assert c.q_dim == 48 and c.kv_dim == 48 and c.rope_scaling is None


def test_every_key_is_read():
    d = dict(BASE, num_key_value_heads=1, head_dim=32, rope_theta=5e5, rms_norm_eps=1e-5, tie_word_embeddings=True,
             max_position_embeddings=77, bos_token_id=1, eos_token_id=[9, 10],
             rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=64), some_other_key=5)
    c = LlamaConfig.from_json(d)
    assert (c.num_key_value_heads, c.head_dim, c.rope_theta, c.rms_norm_eps) == (1, 32, 5e5, 1e-5)
    assert c.tie_word_embeddings and c.max_position_embeddings == 77 and c.bos_token_id == 1
    assert c.eos_token_id == 9  # first of a list
    assert c.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    assert c.extra == {"some_other_key": 5}
    assert LlamaConfig.from_json(c.to_json()) == c


@pytest.mark.parametrize("patch,word", [
    (dict(num_key_value_heads=2), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(hidden_size=50), "head_dim is absent"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "not supported"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "lacks the key"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(mlp_bias=True), "mlp_bias"),
])
def test_bad_configurations_are_refused(patch, word):
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_json(dict(BASE, **patch))
    assert word in str(e.value)


def test_options_that_change_nothing_are_accepted():
    c = LlamaConfig.from_json(dict(BASE, hidden_act="silu", attention_bias=False, mlp_bias=False,
                                   rope_scaling=dict(rope_type="default")))
    assert c.rope_scaling is None
    assert LlamaConfig.from_json(dict(BASE, rope_scaling=None)).rope_scaling is None


def test_missing_keys_are_listed_together():
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_json(dict(architectures=["LlamaForCausalLM"], vocab_size=5))
    for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size"):
        assert k in str(e.value)


def test_registry():
    assert "LlamaForCausalLM" in known_architectures()
    arch = architecture_of(BASE)
    assert arch.name == "LlamaForCausalLM" and isinstance(arch.config_from_json(BASE), LlamaConfig)
    with pytest.raises(ConfigError) as e:
        lookup_architecture("Qwen2ForCausalLM")
    assert "unsupported architecture" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        architecture_of({})


def test_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    arch, cfg = config_from_folder(str(tmp_path))
    assert cfg.hidden_size == 48
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))


def test_model_sizes_come_from_the_configuration_only():
    from bitwise_b200.models.llama import build_llama
    c = LlamaConfig.from_json(dict(BASE, num_key_value_heads=1, head_dim=32, tie_word_embeddings=True))
    m = build_llama(c)
    shapes = {s.name: s.shape for s in m.param_specs()}
    assert shapes["model.layers.1.self_attn.q_proj.weight"] == (96, 48)
    assert shapes["model.layers.0.self_attn.k_proj.weight"] == (32, 48)
    assert shapes["model.layers.0.mlp.down_proj.weight"] == (48, 80)
    assert "lm_head.weight" not in shapes and len(shapes) == 1 + 2 * 9 + 1
