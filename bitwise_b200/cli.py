"""Command line of the engine.

The reference ships no generate program; its command line is the simulator ``bitwise_sim``
with hand-parsed options ``--traces N --seed S --trace N --verbose --model PATH --help`` and
exit code 2 on an unknown option (sim/simulate.cpp:231-263).  ``sim`` below keeps those
names and meanings (``--kernels``, ``--fault``, ``--sweep-faults`` and ``--draft`` belong to
parts this engine does not have).  ``generate`` exposes SamplingParams and EngineConfig
under the reference's field names (src/engine.h:26-50); ``random`` writes a model folder
from a config.json and a seed.

    bitwise_b200 generate --model DIR --prompt-ids 5,17,3 --max-new-tokens 16
    bitwise_b200 sim --model DIR --traces 100
    bitwise_b200 random --config config.json --seed 1 --out DIR

Exit codes: 0 done, 1 a violation found by ``sim`` or an error in the model folder or the
request (one line on standard error), 2 an unknown or malformed option, 3 no CUDA device.
"""
from __future__ import annotations

import argparse
import json
import sys


def _add_model_args(p):
    p.add_argument("--model", help="folder with config.json and model.safetensors")
    p.add_argument("--random", metavar="CONFIG_JSON", help="use random weights for this config.json instead")
    p.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    p.add_argument("--device", default="cuda:0")


class _NoDevice(Exception):
    pass


def _load_model(args):
    import torch
    if not torch.cuda.is_available():
        raise _NoDevice("no CUDA device is visible; this engine has no CPU path")
    from .config.registry import architecture_of
    from .model import Model
    if args.model:
        return Model.load(args.model, dtype=args.dtype, device=args.device)
    if args.random:
        raw = json.load(open(args.random))
        cfg = architecture_of(raw).config_from_json(raw)
        return Model.random(cfg, seed=args.weights_seed, dtype=args.dtype, device=args.device)
    raise SystemExit("give --model DIR or --random CONFIG_JSON")


def cmd_generate(args) -> int:
    from .engine.engine import Engine, EngineConfig
    from .sampling.sampler import SamplingParams
    model = _load_model(args)
    prompts = []
    for spec in args.prompt_ids or []:
        prompts.append([int(t) for t in spec.replace(",", " ").split()])
    if args.prompt_file:
        for line in open(args.prompt_file):
            if line.strip():
                prompts.append([int(t) for t in line.replace(",", " ").split()])
    if not prompts:
        raise SystemExit("no prompt: give --prompt-ids or --prompt-file")
    eng = Engine(model, EngineConfig(num_blocks=args.num_blocks, block_size=args.block_size,
                                     max_batched_tokens=args.max_batched_tokens, max_num_seqs=args.max_num_seqs,
                                     fingerprint_logits=not args.no_fingerprint))
    sp = SamplingParams(args.temperature, args.seed, args.max_new_tokens, args.ignore_eos)
    ids = [eng.add_request(p, sp) for p in prompts]
    while not eng.idle():
        eng.step()
    for rid in ids:
        r = eng.result(rid)
        print(json.dumps({"id": rid, "tokens": r.tokens, "logits_fingerprint": r.logits_fingerprint,
                          "preemptions": r.preemptions}))
    s = eng.stats
    print(f"steps {s.steps}  prefill tokens {s.prefill_tokens}  decode rows {s.decode_rows}  generated "
          f"{s.generated_tokens}  preemptions {s.preemptions}  forward {s.forward_seconds:.3f} s", file=sys.stderr)
    return 0


def cmd_sim(args) -> int:
    from .engine.simulate import run_traces
    model = _load_model(args)
    out = run_traces(model, args.traces, args.seed, args.trace, args.verbose)
    print(f"traces {out.traces}  requests {out.requests_checked}  token mismatches {out.token_mismatch}  "
          f"fingerprint mismatches {out.fingerprint_mismatch}  hangs {out.hangs}  leaks {out.leaks}  "
          f"preemptions {out.preemptions}")
    if out.violations:
        print(f"first bad trace: {out.first_bad_trace} (rerun with --trace {out.first_bad_trace} --verbose)")
        return 1
    return 0


def cmd_random(args) -> int:
    from .config.registry import architecture_of
    from .model import Model
    raw = json.load(open(args.config))
    cfg = architecture_of(raw).config_from_json(raw)
    Model.write_random_folder(args.out, cfg, seed=args.seed, dtype=args.dtype, std=args.std,
                              norm_jitter=args.norm_jitter)
    print(f"wrote {args.out}/config.json and model.safetensors")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bitwise_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    _add_model_args(g)
    g.add_argument("--prompt-ids", action="append", help="token ids of one prompt, comma separated (repeatable)")
    g.add_argument("--prompt-file", help="file with one prompt (token ids) a line")
    g.add_argument("--temperature", type=float, default=0.0, help="0 means greedy")
    g.add_argument("--seed", type=int, default=0, help="sampling seed")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--num-blocks", type=int, default=512)
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--max-batched-tokens", type=int, default=256)
    g.add_argument("--max-num-seqs", type=int, default=32)
    g.add_argument("--no-fingerprint", action="store_true", help="do not hash the logits behind each token")
    g.set_defaults(fn=cmd_generate)

    s = sub.add_parser("sim", help="randomised traces against requests run alone")
    _add_model_args(s)
    s.add_argument("--traces", type=int, default=500)
    s.add_argument("--seed", type=int, default=1)
    s.add_argument("--trace", type=int, default=-1, help="run only this trace")
    s.add_argument("--verbose", action="store_true")
    s.set_defaults(fn=cmd_sim)

    r = sub.add_parser("random", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-jitter", type=float, default=0.0)
    r.set_defaults(fn=cmd_random)

    args = ap.parse_args(argv)
    try:
        return args.fn(args)
    except _NoDevice as e:
        print(f"bitwise_b200: {e}", file=sys.stderr)
        return 3
    except (OSError, ValueError, RuntimeError) as e:
        # configuration, weight, kernel and request errors carry their own one-line messages
        print(f"bitwise_b200: {type(e).__name__}: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
