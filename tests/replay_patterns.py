"""Step traces for the replay tests: the same requests cut in different ways.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``
as bin/trace_run reads them.  ``collect`` turns the logits that a replay returned into
one array per request, indexed by position, so that every pattern can be compared with
the plain implementation position by position.
"""
import numpy as np


def whole(requests):
    """Each request alone and whole, one after the other."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_one_by_one(requests, tail=32):
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(3, 17, 2, 19, 1, 5, 2, 31, 7)):
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + c], "want": list(range(c))}],
                          "end": [rid] if i + c == len(toks) else []})
            i += c
    return steps


def mixed(requests, max_tokens, seed=0, max_live=4):
    """Up to ``max_live`` live requests; portions of some beside single tokens of others;
    a request may sit out a step; a new one starts only when the pool (each request's
    length rounded up to 64) has room, so pages of finished requests are used again."""
    rng = np.random.default_rng(seed)
    pending = list(requests.items())
    live = {}  # rid -> next index
    steps = []

    def held(extra=0):
        return sum((len(requests[r]) + 63) // 64 * 64 for r in live) + extra

    while pending or live:
        while pending and len(live) < max_live and held((len(pending[0][1]) + 63) // 64 * 64) <= max_tokens:
            rid, _ = pending.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks = requests[rid]
            i = live[rid]
            mode = rng.integers(0, 6)
            if mode == 0 and len(live) > 1:
                continue  # sits out this step
            left = len(toks) - i
            c = 1 if mode in (1, 2) else int(rng.choice([2, 3, 5, 8, 13, 21]))
            c = min(c, left)
            entries.append({"id": rid, "tokens": toks[i:i + c], "want": list(range(c))})
            live[rid] = i + c
            if i + c == len(toks):
                end.append(rid)
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            del live[rid]
    return steps


def collect(steps, logits_by_step, vocab):
    """{request id: [len, vocab] array} from the per-step outputs (None where nothing was wanted)."""
    pos = {}
    rows = {}
    for st in steps:
        out = logits_by_step.get(st["step"])
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], {})[base + w] = out[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert out is None or r == out.shape[0]
    return {rid: np.stack([d[i] for i in sorted(d)]) for rid, d in rows.items()}


def run_in_process(model, steps, max_tokens, page_size=16, use_graphs=None, max_live=4, info=None):
    """Replay through the package's stepper (what bin/trace_run drives), in this process.
    ``use_graphs``: None leaves the stepper's default, False runs every step eagerly.  ``info``:
    a dict that receives the stepper's counters."""
    import torch
    from bitwise_b200.engine.replay import make_replay_stepper
    from bitwise_b200.engine.step import StepEntry
    stepper = make_replay_stepper(model, max_tokens, page_size, max_live=max_live, use_graphs=use_graphs)
    outs = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        lg = stepper.run(entries)
        if lg is not None:
            outs[st["step"]] = lg.detach().float().cpu().numpy().copy()
        for rid in st["end"]:
            stepper.finish(rid)
    stepper.manager.check_consistency()
    assert stepper.manager.all_free(), "pages or slots were not given back"
    if info is not None:
        info.update(graph_replays=stepper.graph_replays, steps=stepper.steps, use_graphs=stepper.use_graphs)
    return outs
