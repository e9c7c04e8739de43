"""Builds replay traces in the four ways the tests cut requests, runs them through an
engine's own cache manager and step function, and compares with the plain model."""
import random

import torch

from tiny_transformer_inference_engine_b200.engine.batch import StepEntry


def whole(requests):
    """Each request alone and whole: one step per request, every position wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def prefill_then_decode(requests, tail=32):
    """Most of it in one step and the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        cut = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:cut], "want": list(range(cut))}],
                      "end": [rid] if cut == len(toks) else []})
        for i in range(cut, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
    return steps


def portions(requests, seed=0, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 9)):
    """In portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": [rid] if i + n == len(toks) else []})
            i += n
    return steps


def mixed(requests, max_live=4, seed=0, decode_tail=12):
    """Up to ``max_live`` live requests; portions of some beside single tokens of others in the
    same step; a request joins when another has ended, so pages are used again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live = {}                      # rid -> (tokens, fed)
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = [toks, 0]
        entries, end = [], []
        for rid in list(live):
            toks, fed = live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            left = len(toks) - fed
            if left <= decode_tail:
                n = 1
            else:
                n = min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 16, 17, 31, 40]))
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            live[rid][1] = fed + n
            if fed + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def max_live_tokens(steps, rounding=64):
    """The most tokens live requests hold at any time, each rounded up to ``rounding``."""
    held, peak = {}, 0
    for st in steps:
        for en in st["entries"]:
            held[en["id"]] = held.get(en["id"], 0) + len(en["tokens"])
        peak = max(peak, sum(-(-n // rounding) * rounding for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_steps(engine, steps):
    """Drives the engine's cache manager and step function; returns {(rid, position): logits}."""
    mgr, lengths, got = engine.manager, {}, {}
    for st in steps:
        entries = []
        for en in st["entries"]:
            rid = en["id"]
            if rid not in lengths:
                mgr.admit(rid)
                lengths[rid] = 0
            start = lengths[rid]
            mgr.extend(rid, start, start + len(en["tokens"]))
            entries.append(StepEntry(rid, start, en["tokens"], en["want"]))
        logits = engine.stepper.step(entries).float().cpu()
        k = 0
        for e in entries:
            for w in e.want:
                got[(e.rid, e.start + w)] = logits[k].clone()
                k += 1
            lengths[e.rid] += len(e.tokens)
        assert k == logits.shape[0]
        mgr.check()
        for rid in st["end"]:
            mgr.release(rid)
            del lengths[rid]
    mgr.check()
    assert mgr.num_free_pages == mgr.num_usable_pages, "pages leaked"
    return got


def worst_relative(got, expected):
    """Largest |difference| / max|expected row| over all wanted places; also the place."""
    worst, where = 0.0, None
    for (rid, pos), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        ref = expected[rid][pos]
        err = ((row.double() - ref.double()).abs().max() / ref.double().abs().max()).item()
        if not (err <= worst):
            worst, where = err, (rid, pos)
    return worst, where


def first_wrong(got, expected, tol):
    for (rid, pos), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        ref = expected[rid][pos]
        err = ((row.double() - ref.double()).abs().max() / ref.double().abs().max()).item()
        if not err <= tol:
            return rid, pos, err
    return None
