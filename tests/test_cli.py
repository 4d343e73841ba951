"""The command line, run as a user runs it (a child process of ``bin/bitwise_b200``).

The reference's command line is a hand-parsed argv program with ``--help`` and exit code 2 on
an unknown option, and its simulator is what its CI runs (sim/simulate.cpp:231-301).  Here:
``random`` writes a model folder, ``generate`` must give the tokens and the logits fingerprint
of the plain implementation, ``sim`` must find no violation while preemptions do happen, an
unknown option ends with 2, and a machine without a CUDA device gets one line, not a traceback.
"""
import json
import os
import subprocess
import sys

import pytest

import plain_llama as P
from tiny_configs import TINY, tiny_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "bin", "bitwise_b200")


def run(*args, env=None, timeout=900):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, EXE, *args], capture_output=True, text=True, timeout=timeout, env=e)


def test_help_and_unknown_options():
    p = run("--help")
    assert p.returncode == 0 and "generate" in p.stdout and "sim" in p.stdout and "random" in p.stdout
    assert run("generate", "--help").returncode == 0
    for args in (["generate", "--no-such-option"], ["sim", "--traces"], []):
        p = run(*args)
        assert p.returncode == 2, (args, p.returncode, p.stderr)
        assert "Traceback" not in p.stderr


def test_random_writes_a_model_folder_and_bad_input_is_one_line(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY["tiny_a"]["config"].to_json()))
    out = tmp_path / "model"
    p = run("random", "--config", str(cfg), "--seed", "11", "--out", str(out), "--dtype", "float32")
    assert p.returncode == 0, p.stderr
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    cfg.write_text(json.dumps(dict(TINY["tiny_a"]["config"].to_json(), architectures=["NoSuchModel"])))
    p = run("random", "--config", str(cfg), "--out", str(tmp_path / "m2"))
    assert p.returncode == 1 and "unsupported architecture" in p.stderr and "Traceback" not in p.stderr


def test_without_a_cuda_device_there_is_one_line_and_no_traceback(tiny_folders):
    for cmd in (["generate", "--prompt-ids", "1,2,3"], ["sim", "--traces", "1"]):
        p = run(cmd[0], "--model", tiny_folders["tiny_a"], *cmd[1:], env={"CUDA_VISIBLE_DEVICES": ""})
        assert p.returncode == 3, (p.returncode, p.stderr)
        assert "no CUDA device" in p.stderr and "Traceback" not in p.stderr
        assert len(p.stderr.strip().split("\n")) == 1


@pytest.mark.gpu
def test_random_then_generate_equals_the_plain_implementation(tmp_path):
    """``random`` -> ``generate`` in float32: tokens and fingerprint of P.generate, greedy and sampled."""
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY["tiny_b"]["config"].to_json()))
    folder = tmp_path / "model"
    assert run("random", "--config", str(cfg), "--seed", "5", "--out", str(folder), "--dtype", "bfloat16",
               "--norm-jitter", "0.1").returncode == 0
    prompts = [tiny_tokens("tiny_b", n, salt=60 + i) for i, n in enumerate((9, 40, 3))]
    plain = P.PlainLlama(str(folder), exp="det")
    for temperature, seed in ((0.0, 0), (0.8, 7)):
        args = ["generate", "--model", str(folder), "--dtype", "float32", "--max-new-tokens", "12", "--ignore-eos",
                "--temperature", str(temperature), "--seed", str(seed), "--num-blocks", "8", "--max-batched-tokens", "16"]
        for p in prompts:
            args += ["--prompt-ids", ",".join(map(str, p))]
        proc = run(*args)
        assert proc.returncode == 0, proc.stderr[-2000:]
        rows = [json.loads(l) for l in proc.stdout.strip().split("\n")]
        assert len(rows) == len(prompts)
        for p, row in zip(prompts, rows):
            toks, fp = P.generate(plain, p, 12, temperature, seed, ignore_eos=True)
            assert row["tokens"] == toks and row["logits_fingerprint"] == fp


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sim_finds_no_violation_while_preemptions_happen(dtype, tiny_folders):
    p = run("sim", "--model", tiny_folders["tiny_a"], "--dtype", dtype, "--traces", "20", "--seed", "3")
    assert p.returncode == 0, p.stdout[-1000:] + p.stderr[-2000:]
    words = p.stdout.split()
    fields = {words[i]: words[i + 1] for i in range(0, len(words) - 1)}
    assert int(fields["traces"]) == 20 and int(fields["requests"]) > 40
    assert int(fields["preemptions"]) > 0
