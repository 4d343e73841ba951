"""Makes the golden outputs of this folder by running tkran2/bitwise's OWN model code.

    python tests/golden/make_golden.py --reference /path/to/tkran2-bitwise

For each tiny configuration of tests/tiny_configs.py it writes a model folder with this
package's random-weights mode, converts it with the reference's ``tools/convert.py``
(unmodified; for the configuration with ``rope_scaling``, which that converter refuses,
the key is left out of a copy of config.json and the rescaled frequencies are handed to
the harness instead), compiles ``ref_harness.cpp`` with the reference's ``src/*.cpp`` and
its flags (``-O2 -ffp-contract=off -fno-fast-math``, CMakeLists.txt:15), and stores

    <name>.logits.f32   logits at every position of one whole sequence (float32, [T, vocab])
    <name>.json         the token ids, the sha256 of the model file, generated tokens and
                        the logits fingerprint of the reference's Engine

    sched_traces.json   small workloads run through the reference's Engine under scarce blocks:
                        the state of every request after every step (length, computed tokens,
                        blocks held), events and counters; tests/test_scheduler_vs_reference.py
                        replays them through this package's scheduler and cache manager
    counter_uniform.json  values of the reference's counter_uniform for a list of arguments

tests/test_plain_vs_reference.py then checks that the plain implementation under tests/
reproduces these bits.  The model folder itself is not stored: it is rebuilt from the
seed, and the stored hash says whether the rebuilt file is the one the golden run saw.
"""
import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import plain_llama  # noqa: E402
from tiny_configs import TINY, tiny_tokens, write_tiny_folder  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of tkran2/bitwise (its src/ is compiled)")
    args = ap.parse_args()
    ref = args.reference
    work = tempfile.mkdtemp(prefix="golden-")
    exe = os.path.join(work, "ref_harness")
    srcs = [os.path.join(ref, "src", f) for f in ("kernels.cpp", "model.cpp", "engine.cpp", "block_manager.cpp")]
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fno-fast-math", "-pthread",
                    "-I", os.path.join(ref, "src"), os.path.join(HERE, "ref_harness.cpp"), *srcs, "-o", exe],
                   check=True)
    for name, spec in TINY.items():
        folder = os.path.join(work, name)
        write_tiny_folder(folder, name)
        conv = os.path.join(work, name + "-conv")
        shutil.copytree(folder, conv)
        cfg = json.load(open(os.path.join(conv, "config.json")))
        scaling = cfg.pop("rope_scaling", None)
        json.dump(cfg, open(os.path.join(conv, "config.json"), "w"))
        bw = os.path.join(work, name + ".bw")
        subprocess.run([sys.executable, os.path.join(ref, "tools", "convert.py"), conv, bw], check=True)
        inv_arg = "-"
        if scaling:
            hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
            inv = plain_llama.rope_inv_freq(hd, cfg.get("rope_theta", 10000.0), scaling)
            inv_arg = os.path.join(work, name + ".inv")
            inv.astype("<f4").tofile(inv_arg)
        toks = tiny_tokens(name)
        tok_file = os.path.join(work, name + ".tok")
        np.asarray(toks, dtype="<i4").tofile(tok_file)
        out = os.path.join(HERE, name + ".logits.f32")
        gen = os.path.join(work, name + ".gen")
        g = spec["generate"]
        subprocess.run([exe, bw, inv_arg, tok_file, out, gen, str(g["prompt_len"]), str(g["new"]),
                        repr(g["temperature"]), str(g["seed"])], check=True)
        fp, gen_toks = open(gen).read().split("\n")[:2]
        meta = {
            "tokens": toks,
            "model_sha256": hashlib.sha256(open(os.path.join(folder, "model.safetensors"), "rb").read()).hexdigest(),
            "generate": dict(g, tokens=[int(t) for t in gen_toks.split()], fingerprint=int(fp)),
            "reference_flags": "-O2 -ffp-contract=off -fno-fast-math (scalar build)",
        }
        json.dump(meta, open(os.path.join(HERE, name + ".json"), "w"), indent=1)
        print("wrote", out, os.path.getsize(out), "bytes")
        if name == "tiny_a":
            make_sched_traces(exe, bw, work)
    uni = os.path.join(work, "uniform.txt")
    subprocess.run([exe, "--uniform", uni], check=True)
    rows = [l.split() for l in open(uni).read().split("\n") if l]
    json.dump([{"seed": int(a), "position": int(b), "stream": int(c), "bits": d} for a, b, c, d in rows],
              open(os.path.join(HERE, "counter_uniform.json"), "w"), indent=0)
    shutil.rmtree(work, ignore_errors=True)


# (num_blocks, max_batched_tokens, max_num_seqs), [(arrival step, prompt length, new tokens, cancel step)]
SCHED_TRACES = [
    # the reference's own scarce configuration: nine blocks force preemption and recompute
    # (tests/test_main.cpp:274-279)
    ((9, 32, 4), [(0, 30, 20, -1), (0, 40, 24, -1), (1, 17, 30, -1), (3, 50, 10, -1), (5, 5, 40, -1)]),
    ((9, 16, 8), [(0, 60, 12, -1), (0, 9, 30, -1), (2, 33, 20, -1), (2, 20, 20, 9), (4, 1, 25, -1), (20, 70, 5, -1)]),
    ((6, 7, 3), [(0, 31, 16, -1), (0, 17, 16, -1), (0, 5, 16, -1), (1, 47, 10, -1)]),
    ((12, 64, 2), [(0, 100, 30, -1), (0, 64, 40, -1), (1, 16, 50, 30), (2, 15, 60, -1)]),
    ((5, 24, 5), [(0, 16, 40, -1), (0, 16, 40, -1), (0, 16, 40, -1), (7, 33, 8, -1), (8, 2, 60, 12)]),
    ((64, 8, 16), [(i // 2, 3 + 5 * i, 6 + i, -1) for i in range(10)]),
]


def make_sched_traces(exe, bw, work):
    traces = []
    for t, ((blocks, budget, seqs), reqs) in enumerate(SCHED_TRACES):
        spec = os.path.join(work, f"sched{t}.txt")
        out = os.path.join(work, f"sched{t}.out")
        with open(spec, "w") as f:
            f.write(f"{blocks} {budget} {seqs}\n" + "".join("%d %d %d %d\n" % r for r in reqs))
        subprocess.run([exe, "--sched", bw, spec, out], check=True)
        steps, cur = [], None
        for line in open(out).read().split("\n"):
            w = line.split()
            if not w or w[0] == "end":
                continue
            if w[0] == "step":
                cur = {"step": int(w[1]), "seqs": []}
                steps.append(cur)
            elif w[0] == "events":
                cur["events"] = [[int(x) for x in e.split(":")] for e in w[1:]]
            elif w[0] == "stats":
                cur["prefill_tokens"], cur["decode_rows"], cur["preemptions"], cur["generated"] = map(int, w[1:])
            elif w[0] == "counts":
                cur["running"], cur["waiting"], cur["free_blocks"] = map(int, w[1:])
            elif w[0] in ("running", "waiting"):
                kv = dict(x.split("=") for x in w[1:])
                cur["seqs"].append([w[0], int(kv["id"]), int(kv["len"]), int(kv["computed"]), int(kv["blocks"])])
        traces.append({"num_blocks": blocks, "max_batched_tokens": budget, "max_num_seqs": seqs,
                       "requests": [list(r) for r in reqs], "steps": steps})
        print(f"sched trace {t}: {len(steps)} steps, {steps[-1]['preemptions']} preemptions")
    with open(os.path.join(HERE, "sched_traces.json"), "w") as f:
        f.write("[\n" + ",\n".join(json.dumps(t, separators=(",", ":")) for t in traces) + "\n]\n")


if __name__ == "__main__":
    main()
