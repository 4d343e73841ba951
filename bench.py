#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the SmolLM2-1.7B shape (24 layers, hidden 2048, 32/32 heads, head size
64, SwiGLU 8192, vocabulary 49152, tied embeddings), random N(0, 0.02) bfloat16 weights,
synthetic prompt ids uniform over the vocabulary; batch of 8 requests decoding at a
2,048-token context.  A "step" is one decode step of the whole batch.  Prints ONE JSON line:

  value        decoded tokens per second, timed on the device with CUDA events
  e2e          the same through the Python entry point (Engine.step): host tokens in from
               pinned memory, sampled tokens read back to the host, every step
  prefill      one step of 2,048 prompt tokens; frac = flops / time / bf16 peak (float32 runs:
               / the float32 peak of the CUDA cores)
  roofline     decode step: bytes it must read (every weight once + the cache of the live
               requests) / time, against the copy bandwidth
  points       decode tokens per second at batch 1 and 64
  fp32         decode and prefill of the same shape on the true 32-bit path

Other workloads: --shape smollm2-360m|llama3-8b runs the same measurements on those layer
sizes; --workload serve pushes 64 mixed requests through the engine's scheduler under a
512-token budget and reports generated tokens per second by the host clock.

Peaks come from MEASURED_PEAKS.json beside this file when present ("of measured"), else
from the fallback figures of an earlier measurement on this kind of GPU ("of fallback").
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# The like-for-like baseline: tkran2/bitwise's Runner::forward on the SmolLM2-1.7B shape, 8 threads on
# this image's CPU, 2,048-token contexts, as BASELINE.md records it (decode tokens per second by batch).
# The reference publishes no figure for this batch and context (its README has 7.26 tok/s single stream).
BASELINE_DECODE_TOKS = {("smollm2-1.7b", 2048, 1): 10.7, ("smollm2-1.7b", 2048, 8): 29.9, ("smollm2-1.7b", 2048, 64): 35.4}
REFERENCE_SOURCE = "/root/reference"


def fp32_simt_tflops():
    """The float32 peak of the CUDA cores, from the device's own figures: SMs x 128 lanes x 2
    flops x the highest SM clock (what the true 32-bit path, which uses no tensor core, is
    measured against)."""
    import torch
    props = torch.cuda.get_device_properties(0)
    mhz = 0.0
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits", "-i", "0"],
                             capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
        mhz = float(out[0])
    except Exception:
        mhz = 0.0
    if mhz <= 0:
        mhz = 1965.0
    return props.multi_processor_count * 128 * 2 * mhz * 1e6 / 1e12


def peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            flat = {}

            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            hbm = flat.get("hbm_gbs")
            tf = flat.get("bf16_tflops")
            tfs = flat.get("bf16_tflops_sustained", tf)
            if hbm and tf:
                return dict(hbm_gbs=hbm, bf16_tflops=tf, bf16_tflops_sustained=tfs, source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_tflops_sustained=1400.0,
                source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            p = [x.strip() for x in line.split(",")]
            if len(p) >= 6 and p[0].isdigit():
                self.samples.append(p)

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


SHAPES = {
    # name: (title, layers, LlamaConfig keywords, default decode context)
    "smollm2-1.7b": ("SmolLM2-1.7B shape", 24, dict(
        vocab_size=49152, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32, head_dim=64,
        intermediate_size=8192, rope_theta=130000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
        max_position_embeddings=8192), 2048),
    "smollm2-360m": ("SmolLM2-360M shape", 32, dict(
        vocab_size=49152, hidden_size=960, num_attention_heads=15, num_key_value_heads=5, head_dim=64,
        intermediate_size=2560, rope_theta=100000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
        max_position_embeddings=8192), 2048),
    "llama3-8b": ("Llama-3-8B shape", 32, dict(
        vocab_size=128256, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
        max_position_embeddings=8192,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)), 4096),
}


def model_config(shape, layers):
    from bitwise_b200 import LlamaConfig
    from bitwise_b200.config.llama import RopeScaling
    kw = dict(SHAPES[shape][2])
    if "rope_scaling" in kw:
        kw["rope_scaling"] = RopeScaling(**kw["rope_scaling"])
    return LlamaConfig(num_hidden_layers=layers, **kw)


def matrix_params(c):
    per_layer = (c.q_dim + 2 * c.kv_dim) * c.hidden_size + c.hidden_size * c.q_dim + 3 * c.hidden_size * c.intermediate_size
    return per_layer * c.num_hidden_layers, c.vocab_size * c.hidden_size


def decode_bytes(c, batch, ctx, elt):
    body, head = matrix_params(c)
    kv = batch * ctx * c.num_hidden_layers * 2 * c.kv_dim * elt
    return (body + head) * elt + kv + batch * c.hidden_size * elt


def prefill_flops(c, tokens):
    body, head = matrix_params(c)
    attn = c.num_hidden_layers * 2 * 2 * c.q_dim * (tokens * (tokens + 1) // 2)
    return 2.0 * tokens * body + 2.0 * head + attn


def run_decode(model, batch, ctx, steps, warmup, page, seed=0):
    """Device-timed decode: `batch` requests, each with `ctx` tokens in the cache, one new
    token each per step, sampled greedily on the device."""
    import numpy as np
    import torch
    from bitwise_b200.cache.storage import build_cache
    from bitwise_b200.engine.step import StepEntry, Stepper
    c = model.config
    total = ctx + warmup + steps + 1
    pages_per = (total + page - 1) // page
    manager, storage = build_cache(model.decoder, pages_per * batch, page, batch, torch.bfloat16 if
                                   model.dtype == "bfloat16" else torch.float32, model.device)
    chunk = 2048
    st = Stepper(model.decoder, manager, storage, model.ops, max_rows=max(chunk, batch), max_seqs=batch,
                 max_tokens_per_request=pages_per * page)
    rng = np.random.default_rng(seed)
    for b in range(batch):  # fill the contexts by real prefill
        toks = rng.integers(0, c.vocab_size, ctx - 1).tolist()
        for i in range(0, len(toks), chunk):
            st.run([StepEntry(b, toks[i:i + chunk], [])])
    nxt = rng.integers(0, c.vocab_size, batch).tolist()
    temps = torch.zeros(batch, device=model.device)
    us = torch.zeros(batch, dtype=torch.float64, device=model.device)
    out = torch.zeros(batch, dtype=torch.int32, device=model.device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one_step():
        logits = st.run([StepEntry(b, [nxt[b]], [0]) for b in range(batch)])
        model.ops.sample_rows(logits, temps, us, out)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    l0 = model.ops.launches
    ev0.record()
    for _ in range(steps):
        one_step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    launches = model.ops.launches - l0
    del st, manager, storage
    torch.cuda.empty_cache()
    return ms, launches


def run_prefill(model, tokens, reps, warmup, page):
    import numpy as np
    import torch
    from bitwise_b200.cache.storage import build_cache
    from bitwise_b200.engine.step import StepEntry, Stepper
    c = model.config
    pages = (tokens + page - 1) // page
    manager, storage = build_cache(model.decoder, pages, page, 1, torch.bfloat16 if model.dtype == "bfloat16"
                                   else torch.float32, model.device)
    st = Stepper(model.decoder, manager, storage, model.ops, max_rows=tokens, max_seqs=1,
                 max_tokens_per_request=pages * page)
    toks = np.random.default_rng(1).integers(0, c.vocab_size, tokens).tolist()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(warmup + reps):
        torch.cuda.synchronize()
        ev0.record()
        st.run([StepEntry("p", toks, [tokens - 1])])
        ev1.record()
        torch.cuda.synchronize()
        st.finish("p")
        if i >= warmup:
            times.append(ev0.elapsed_time(ev1))
    del st, manager, storage
    torch.cuda.empty_cache()
    return sorted(times)[len(times) // 2]


def run_e2e(model, batch, ctx, steps, warmup, page, fingerprint=True):
    """Through Engine.step(): prompts of ctx-1 tokens are prefilled by the engine itself, then
    `steps` decode steps are timed by the host clock, each with its host-to-device copy of the
    step's inputs and the device-to-host read of the sampled tokens.  ``fingerprint``: the
    engine's default, a hash of every sampled row's logits chained on the device."""
    import numpy as np
    import torch
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    c = model.config
    total = ctx + warmup + steps + batch + 16
    pages_per = (total + page - 1) // page
    eng = Engine(model, EngineConfig(num_blocks=pages_per * batch, block_size=page, max_batched_tokens=2048,
                                     max_num_seqs=batch, fingerprint_logits=fingerprint,
                                     max_model_len=pages_per * page))
    rng = np.random.default_rng(2)
    sp = SamplingParams(temperature=0.0, max_new_tokens=warmup + steps + batch + 8, ignore_eos=True)
    for b in range(batch):
        eng.add_request(rng.integers(0, c.vocab_size, ctx - 1).tolist(), sp)
    guard = 0
    while eng.stats.prefill_tokens < batch * (ctx - 1):  # until every request has left its prompt behind
        eng.step()
        guard += 1
        assert guard < 10000
    for _ in range(max(warmup, 3)):  # decode steps only from here on; the first ones build the step's graph
        eng.step()
    torch.cuda.synchronize()
    g0 = eng.stats.generated_tokens
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = eng.stats.generated_tokens - g0
    h2d = eng.stepper.h2d_bytes + eng._samp_host.numel()
    d2h = eng.d2h_bytes
    del eng
    torch.cuda.empty_cache()
    return made / dt, h2d, d2h


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="layers to run (default: all of the shape's)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=0, help="tokens in each request's cache (default: the shape's)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"],
                    help="serve: 64 requests with prompts of 16..1024 and outputs of 16..256 tokens through the "
                         "engine's scheduler under a 512-token budget")
    ap.add_argument("--skip-fp32", action="store_true", help="leave out the float32 figures")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="only the headline decode (for profiling runs)")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        print(json.dumps(reference_arm(args)))
        return 0
    warmup = max(3, args.warmup)

    import torch
    from bitwise_b200 import Model
    pk = peaks()
    title, full_layers, _, shape_ctx = SHAPES[args.shape]
    args.layers = args.layers or full_layers
    args.ctx = args.ctx or shape_ctx
    cfg = model_config(args.shape, args.layers)
    model = Model.random(cfg, seed=0, dtype=args.dtype, device="cuda:0", fast=True)
    elt = 2 if args.dtype == "bfloat16" else 4
    if args.workload == "serve":
        print(json.dumps(run_serve(model, title, args, pk)))
        return 0

    with ClockSampler() as clocks:
        ms, launches = run_decode(model, args.batch, args.ctx, args.steps, warmup, args.page)
    value = args.batch / (ms / 1e3)
    bytes_step = decode_bytes(cfg, args.batch, args.ctx, elt)
    achieved = bytes_step / (ms / 1e3) / 1e9

    line = {
        "metric": f"decode tok/s at batch {args.batch}, {args.ctx:,}-token context ({title})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": baseline_ratio(args, value), "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary",
        "impl": "ours",
        "config": {"model": title, "layers": full_layers, "layers_run": args.layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied_embeddings": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.ctx,
                   "page_size": args.page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights + cache read per step exceed 126 MB)",
                   "peaks": "of " + pk["source"], "baseline": BASELINE_NOTE},
        "clocks": clocks.summary(),
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": bytes_step},
    }
    if not args.skip_prefill:
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        fl = prefill_flops(cfg, 2048)
        peak_tf = pk["bf16_tflops"] if args.dtype == "bfloat16" else fp32_simt_tflops()
        line["prefill"] = {"value": round(2048 / (pms / 1e3), 1), "tokens": 2048, "ms": round(pms, 3),
                           "frac": round(fl / (pms / 1e3) / 1e12 / peak_tf, 4), "flops": fl}
        if args.dtype != "bfloat16":
            line["prefill"]["peak"] = "float32 on the CUDA cores, %.1f TFLOP/s nominal" % peak_tf
    if not args.skip_points:
        pts = {}
        for b in (1, 64):
            pm, _ = run_decode(model, b, args.ctx, max(10, args.steps // 2), 3, args.page)
            pts[f"decode_b{b}"] = round(b / (pm / 1e3), 1)
            pts[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, args.ctx, elt) / (pm / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = pts
        e, h2d, d2h = run_e2e(model, args.batch, args.ctx, args.steps, warmup, args.page, fingerprint=True)
        e_plain, _, _ = run_e2e(model, args.batch, args.ctx, args.steps, warmup, args.page, fingerprint=False)
        line["e2e"] = {"value": round(e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "settings": "Engine defaults (fingerprint_logits on, a step ahead of the reads)",
                       "value_without_fingerprint": round(e_plain, 1)}
    if not args.skip_fp32 and args.dtype == "bfloat16" and not args.skip_points:
        # the true 32-bit path of the same shape (no reduced-precision matrix mode anywhere)
        del model
        torch.cuda.empty_cache()
        m32 = Model.random(cfg, seed=0, dtype="float32", device="cuda:0", fast=True)
        fm, _ = run_decode(m32, args.batch, args.ctx, max(5, args.steps // 5), 3, args.page)
        f32 = {"decode_b%d" % args.batch: round(args.batch / (fm / 1e3), 1), "ms_per_step": round(fm, 3),
               "decode_hbm_frac": round(decode_bytes(cfg, args.batch, args.ctx, 4) / (fm / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
        if not args.skip_prefill:
            fp = run_prefill(m32, 2048, reps=3, warmup=3, page=args.page)
            f32["prefill"] = round(2048 / (fp / 1e3), 1)
            f32["prefill_ms"] = round(fp, 2)
            # against the float32 peak of the CUDA cores (no tensor core on this path)
            f32["prefill_frac"] = round(prefill_flops(cfg, 2048) / (fp / 1e3) / 1e12 / fp32_simt_tflops(), 4)
        line["fp32"] = f32
    print(json.dumps(line))
    return 0


BASELINE_NOTE = ("vs_baseline divides by BASELINE.md's figure for the same shape, batch and context: the reference's "
                 "Runner::forward on this image's CPU, 8 threads")


def baseline_ratio(args, value):
    base = BASELINE_DECODE_TOKS.get((args.shape, args.ctx, args.batch))
    if base is None or args.layers != SHAPES[args.shape][1]:
        return None
    return round(value / base, 1)


def _cpu_flags():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def reference_arm(args):
    """tkran2/bitwise itself, unmodified, on the same shape, batch and context.  It is a CMake
    C++ project for the CPU without a Python package to install, so its sources are copied
    beside the harness baseline/ref_bench.cpp into baseline/_ref/ and compiled there with its own
    flags (CMakeLists.txt:5-18: Release, -ffp-contract=off -fno-fast-math, AVX-512 where the CPU
    has it); the harness drives Model::random, Runner::forward and argmax_row."""
    import shutil
    unavailable = lambda why: {"impl": "reference", "unavailable": why}
    ref = os.path.join(HERE, "baseline", "_ref")
    src = os.path.join(ref, "src")
    names = ("kernels.cpp", "model.cpp", "engine.cpp", "block_manager.cpp")
    if not all(os.path.isfile(os.path.join(src, f)) for f in names):
        origin = os.path.join(REFERENCE_SOURCE, "src")
        if not os.path.isdir(origin):
            return unavailable("the reference's sources are neither in baseline/_ref/src nor at " + REFERENCE_SOURCE)
        os.makedirs(ref, exist_ok=True)
        shutil.copytree(origin, src, dirs_exist_ok=True)
    cxx = shutil.which("g++") or shutil.which("c++")
    flags = _cpu_flags()
    avx = {"avx512f", "avx512bw", "avx512vl", "fma"} <= flags
    exe = os.path.join(ref, "ref_bench_avx512" if avx else "ref_bench_scalar")
    harness = os.path.join(HERE, "baseline", "ref_bench.cpp")
    newest = max(os.path.getmtime(os.path.join(src, f)) for f in os.listdir(src))
    if not os.path.isfile(exe) or os.path.getmtime(exe) < max(newest, os.path.getmtime(harness)):
        if not cxx:
            return unavailable("no C++ compiler on this machine (g++, c++) to build the reference with")
        cmd = [cxx, "-std=c++20", "-O3", "-DNDEBUG", "-ffp-contract=off", "-fno-fast-math", "-pthread"]
        cmd += ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mfma"] if avx else []
        cmd += ["-I", src, harness, *[os.path.join(src, f) for f in names], "-o", exe]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            return unavailable("the reference does not compile here: " + r.stderr.strip().split("\n")[-1][:200])
    title, full_layers, kw, shape_ctx = SHAPES[args.shape]
    layers = args.layers or full_layers
    ctx = args.ctx or shape_ctx
    warmup = max(3, args.warmup)
    threads = min(os.cpu_count() or 8, 64)
    points = [] if args.skip_points else [b for b in (1, 64) if b != args.batch]
    cmd = [exe, layers, kw["hidden_size"], kw["num_attention_heads"], kw["num_key_value_heads"], kw["head_dim"],
           kw["intermediate_size"], kw["vocab_size"], kw["rope_theta"], threads, ctx, args.batch, args.steps, warmup,
           0 if args.skip_prefill else 2048, *points]
    try:
        r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=3000)
    except subprocess.TimeoutExpired:
        return unavailable("the reference did not finish the workload within 50 minutes on this machine's CPU")
    if r.returncode != 0:
        return unavailable(f"the reference's harness ended with code {r.returncode}: {r.stderr.strip()[-200:]}")
    out = json.loads(r.stdout.strip().split("\n")[-1])
    ms = out["ms_per_step"]
    value = args.batch / (ms / 1e3)
    line = {
        "metric": f"decode tok/s at batch {args.batch}, {ctx:,}-token context ({title})",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights, fp32 compute (the reference's serving mode)",
        "data": "synthetic: the reference's Model::random weights, zero-filled cache, fixed token ids",
        "impl": "reference",
        "config": {"model": title, "layers": full_layers, "layers_run": layers, "hidden": kw["hidden_size"],
                   "heads": kw["num_attention_heads"], "kv_heads": kw["num_key_value_heads"], "head_dim": kw["head_dim"],
                   "intermediate": kw["intermediate_size"], "vocab": kw["vocab_size"], "global_batch": args.batch,
                   "seq_len": ctx, "page_size": 16, "parallelism": f"CPU, {threads} threads",
                   "build": "AVX-512" if avx else "portable scalar path (this CPU lacks AVX-512)",
                   "api": "bw::Model::random, bw::Runner::forward, bw::argmax_row", "timing": "host clock"},
        "clocks": {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["runs on the CPU"]},
        "gpu_launches": 0,
        "e2e": {"value": round(args.batch / (out["e2e_ms_per_step"] / 1e3), 2), "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "settings": "Runner::forward plus the reference's greedy sampler, host tokens in and out"},
    }
    if "prefill_ms" in out:
        line["prefill"] = {"value": round(2048 / (out["prefill_ms"] / 1e3), 2), "tokens": 2048, "ms": out["prefill_ms"]}
    pts = {f"decode_b{b}": round(b / (out[f"decode_b{b}_ms"] / 1e3), 2) for b in points if f"decode_b{b}_ms" in out}
    if pts:
        line["points"] = pts
    return line


def run_serve(model, title, args, pk):
    """Continuous batching through the engine: 64 requests, prompt lengths uniform in [16, 1024],
    output lengths uniform in [16, 256], prompts cut under a 512-token budget; host clock around
    the whole run, which is repeated after one untimed pass."""
    import numpy as np
    import torch
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    c = model.config
    rng = np.random.default_rng(3)
    n = 64
    plen = rng.integers(16, 1025, n)
    olen = rng.integers(16, 257, n)
    prompts = [rng.integers(0, c.vocab_size, int(l)).tolist() for l in plen]
    params = [SamplingParams(temperature=0.0, max_new_tokens=int(o), ignore_eos=True) for o in olen]
    page = args.page
    blocks = sum((int(p) + int(o) + page) // page for p, o in zip(plen, olen)) + 8
    out = {}
    with ClockSampler() as clocks:
        for rep in range(2):
            eng = Engine(model, EngineConfig(num_blocks=blocks, block_size=page, max_batched_tokens=512,
                                             max_num_seqs=n, fingerprint_logits=False, max_model_len=2048))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = eng.generate(prompts, params)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            made = sum(len(r) for r in res)
            out = {"value": made / dt, "seconds": dt, "steps": eng.stats.steps, "generated": made,
                   "prompt_tokens": int(plen.sum()), "launches": model.ops.launches,
                   "graph_replays": eng.stepper.graph_replays, "preemptions": eng.stats.preemptions}
            del eng
            torch.cuda.empty_cache()
    # what the crowd generated must be what each request generates alone (the reference's oracle,
    # sim/simulate.cpp:102-118): five of the requests are run again, each on an idle engine
    checked, wrong = 0, 0
    for i in (0, 13, 27, 41, 63):
        solo = Engine(model, EngineConfig(num_blocks=(int(plen[i]) + int(olen[i]) + page) // page + 1, block_size=page,
                                          max_batched_tokens=512, max_num_seqs=1, fingerprint_logits=False))
        checked += 1
        wrong += int(solo.generate([prompts[i]], [params[i]])[0] != res[i])
        del solo
    return {
        "metric": f"generated tok/s, 64 mixed requests under a 512-token budget ({title})",
        "value": round(out["value"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": out["steps"], "warmup": 1,
        "ms_per_step": round(out["seconds"] * 1e3 / max(1, out["steps"]), 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "impl": "ours",
        "config": {"model": title, "layers": c.num_hidden_layers, "hidden": c.hidden_size,
                   "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size, "requests": n,
                   "prompt_tokens": out["prompt_tokens"], "generated_tokens": out["generated"],
                   "token_budget": 512, "page_size": page, "parallelism": "single GPU",
                   "timing": "host clock around Engine.generate, second of two passes",
                   "steps_replayed_as_graphs": out["graph_replays"], "preemptions": out["preemptions"],
                   "requests_checked_against_solo_runs": checked, "requests_that_differ": wrong},
        "clocks": clocks.summary(), "gpu_launches": out["launches"],
        "total_tokens_per_s": round((out["prompt_tokens"] + out["generated"]) / out["seconds"], 1),
    }


if __name__ == "__main__":
    sys.exit(main())
