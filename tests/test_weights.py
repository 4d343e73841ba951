"""Safetensors reading and writing, weight errors, random-weights mode (no GPU)."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest
import torch

from bitwise_b200 import LlamaConfig, Model
from bitwise_b200.models.llama import build_llama
from bitwise_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_state, write_safetensors)

CFG = LlamaConfig(vocab_size=50, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=40,
                  head_dim=16)


def test_round_trip_and_dtypes(tmp_path):
    a = torch.randn(3, 5)
    b = torch.randn(4, 2).to(torch.bfloat16)
    c = torch.arange(6, dtype=torch.int64).reshape(2, 3)
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, [("a", a), ("b", b), ("c", c)], {"k": "v"})
    f = SafetensorsFile(path)
    assert f.names() == ["a", "b", "c"] and f.metadata == {"k": "v"}
    assert torch.equal(f.tensor("a"), a) and torch.equal(f.tensor("b"), b) and torch.equal(f.tensor("c"), c)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = Model.write_random_folder(str(tmp_path / "m"), CFG, seed=1)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(32, 31)
    write_safetensors(os.path.join(folder, "model.safetensors"), list(tensors.items()))
    specs = build_llama(CFG).param_specs()
    with pytest.raises(WeightError) as e:
        load_state(folder, specs, torch.float32, "cpu")
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (32, 31), (32, 32))]
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[32, 31]"):
        assert word in str(err)


def test_storage_dtypes_of_the_two_paths(tmp_path):
    folder = Model.write_random_folder(str(tmp_path / "m"), CFG, seed=1, dtype="bfloat16")
    specs = build_llama(CFG).param_specs()
    s16 = load_state(folder, specs, torch.bfloat16, "cpu")
    s32 = load_state(folder, specs, torch.float32, "cpu")
    assert s16["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert s16["model.norm.weight"].dtype == torch.float32  # a norm weight is read in 32-bit by the kernels
    assert s32["model.layers.0.mlp.gate_proj.weight"].dtype == torch.float32
    assert torch.equal(s32["lm_head.weight"], s16["lm_head.weight"].float())  # widening is exact


def test_float32_file_is_rounded_to_nearest_even_for_bfloat16(tmp_path):
    folder = Model.write_random_folder(str(tmp_path / "m"), CFG, seed=2, dtype="float32")
    specs = build_llama(CFG).param_specs()
    s16 = load_state(folder, specs, torch.bfloat16, "cpu")
    s32 = load_state(folder, specs, torch.float32, "cpu")
    w = s32["lm_head.weight"].numpy()
    b = w.view(np.uint32).astype(np.uint64)
    want = (((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)  # src/model.cpp:69-74
    assert np.array_equal(s16["lm_head.weight"].float().numpy(), want)


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)  # data cut short
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(str(p))
    assert "truncated" in str(e.value)
    hdr = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(str(p))
    assert "unsupported dtype" in str(e.value)
    os.makedirs(tmp_path / "empty")
    with pytest.raises(SafetensorsError) as e:
        load_state(str(tmp_path / "empty"), [], torch.float32, "cpu")
    assert "no .safetensors" in str(e.value)


def test_random_folder_is_a_function_of_config_and_seed(tmp_path):
    def digest(folder):
        return hashlib.sha256(open(os.path.join(folder, "model.safetensors"), "rb").read()).hexdigest()
    a = Model.write_random_folder(str(tmp_path / "a"), CFG, seed=5)
    b = Model.write_random_folder(str(tmp_path / "b"), CFG, seed=5)
    c = Model.write_random_folder(str(tmp_path / "c"), CFG, seed=6)
    assert digest(a) == digest(b) != digest(c)
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 32
    f = SafetensorsFile(os.path.join(a, "model.safetensors"))
    w = f.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert torch.equal(f.tensor("model.norm.weight"), torch.ones(32))
    d = Model.write_random_folder(str(tmp_path / "d"), CFG, seed=5, norm_jitter=0.1)
    n = SafetensorsFile(os.path.join(d, "model.safetensors")).tensor("model.norm.weight")
    assert float(n.min()) >= 0.9 and float(n.max()) <= 1.1 and float(n.std()) > 0.02


def test_model_load_passes_over_rotary_buffers_and_a_repeated_tied_head(tmp_path):
    """Older exports keep ``rotary_emb.inv_freq`` buffers, and some store ``lm_head.weight``
    although the head is tied: the first is of no use (the table is built from the
    configuration), the second is passed over when it repeats the embedding bit for bit and
    refused when it does not."""
    from cpu_ops import CpuOps
    tied = LlamaConfig(vocab_size=50, hidden_size=32, num_hidden_layers=1, num_attention_heads=2,
                       intermediate_size=40, head_dim=16, tie_word_embeddings=True)
    folder = Model.write_random_folder(str(tmp_path / "m"), tied, seed=2)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    assert "lm_head.weight" not in tensors
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(path, list(tensors.items()))
    m = Model.load(folder, "float32", device="cpu", ops=CpuOps("float32"))
    assert m.decoder.head.weight is m.decoder.embedding.table
    tensors["lm_head.weight"][3, 4] += 1.0
    write_safetensors(path, list(tensors.items()))
    with pytest.raises(SafetensorsError) as e:
        Model.load(folder, "float32", device="cpu", ops=CpuOps("float32"))
    assert "lm_head.weight" in str(e.value) and "differ" in str(e.value)
    # anything else that the model does not declare is still reported
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(32)
    write_safetensors(path, list(tensors.items()))
    with pytest.raises(WeightError) as e:
        Model.load(folder, "float32", device="cpu", ops=CpuOps("float32"))
    assert e.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
