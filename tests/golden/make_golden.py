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
    shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    main()
