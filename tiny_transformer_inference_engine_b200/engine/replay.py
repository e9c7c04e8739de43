"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and owns no forward pass, cache or loader: it builds the same
``Engine`` that generation uses and drives its cache manager and its step function.

Input: one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` are one batch: for each request its next tokens (a request seen for the
first time starts at position 0) and ``want``, the places among these tokens whose logits
are asked for.  ``end`` lists requests that are finished after this step; their pages and
state slot are given back.  For a step that wants something, ``<out>/<step>.f32`` holds the
logits ``[wanted, vocab]`` as little-endian float32 in the order of the entries and of
``want``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np

PAGE_ROUNDING = 64          # a request's token count is rounded up to this when sizing the pool


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page (must divide 64)")
    ap.add_argument("--max-live", type=int, default=8, help="state slots (requests live at a time)")
    ap.add_argument("--device", default="cuda:0")
    return ap


def make_engine(args):
    from .engine import Engine
    from ..config import EngineConfig, CacheConfig, SchedulerConfig
    if args.block_size <= 0 or PAGE_ROUNDING % args.block_size:
        raise SystemExit(f"--block-size must divide {PAGE_ROUNDING}")
    pages = -(-args.max_tokens // args.block_size) + 1            # + the scratch page
    ec = EngineConfig(dtype=args.dtype, device=args.device, use_cuda_graphs=False,
                      cache=CacheConfig(block_size=args.block_size, num_gpu_blocks=max(pages, 2)),
                      sched=SchedulerConfig(max_num_seqs=args.max_live,
                                            max_num_batched_tokens=max(args.max_live, 512)))
    return Engine.from_folder(args.model, ec)


def run(engine, lines, out_dir: str, log=sys.stdout) -> None:
    from .batch import StepEntry
    os.makedirs(out_dir, exist_ok=True)
    lengths: Dict[str, int] = {}
    mgr = engine.manager
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for en in rec.get("entries", []):
            rid, tokens = en["id"], list(en["tokens"])
            if not tokens:                                     # nothing to run for this request in this step
                continue
            if rid not in lengths:
                mgr.admit(rid)
                lengths[rid] = 0
            start = lengths[rid]
            mgr.extend(rid, start, start + len(tokens))
            entries.append(StepEntry(rid, start, tokens, list(en.get("want", []))))
        if entries:
            logits = engine.stepper.step(entries)
            for e in entries:
                lengths[e.rid] += len(e.tokens)
            if logits.shape[0]:
                arr = logits.float().cpu().numpy().astype("<f4", copy=False)
                if hasattr(engine.ops, "check_tc"):
                    engine.ops.check_tc()
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            if rid in lengths:
                mgr.release(rid)
                del lengths[rid]
        print(f"done {step}", file=log, flush=True)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    engine = make_engine(args)
    run(engine, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
