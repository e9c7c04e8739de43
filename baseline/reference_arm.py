#!/usr/bin/env python3
"""The reference arm of ``bench.py``: the unmodified reference, through its own serving path, on the
same workload as this repository's arm.

    python baseline/reference_arm.py --steps K --warmup W [--batch 8] [--ctx 4096] [--layers 32]

It imports nothing of this repository's package.  The copy under ``baseline/_ref`` (made and built by
``baseline/build_reference.py``) is put on ``sys.path``; ``tiktoken`` is replaced by an empty stand-in
before ``serving/generation.py`` is imported, because that module fetches the ``gpt2`` vocabulary at
import time (serving/generation.py:8) and there is no network - token ids go in and out here, no text.

Model: ``PagedTransformer`` (serving/paged_model.py:34-67) at the Llama-2-7B layer sizes with one kv
head, built from a ``ModelConfig`` subclass whose ``hidden_size`` is the feed-forward width (the
reference's own property returns ``d_model``, models/model_config.py:32-34), default-initialised
weights cast to float16 (the dtype its attention kernel takes, serving/fake_paged_attn.py:44), a
``KVPool`` and ``BlockAllocator`` of its own (serving/kv_pool.py, serving/allocator.py).

Timed: the loop body of its ``generate_batched`` (serving/generation.py:135-143: ``append_token``,
``ensure_blocks``, ``build_batch_step``, ``forward_batch``, argmax per row on the host), W warm-up
iterations and exactly K timed ones between CUDA events with a synchronize on both sides.  ``e2e`` is
the same quantity through ``generate_batched`` itself, host token lists in and out: the time of a call
that generates 1 + W + K tokens minus the time of a call that generates 1 + W, divided by K.

A tiny configuration runs first; if that raises, or gives logits that are not finite, the full size is
not attempted and the line printed says why.
"""
import argparse
import json
import os
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def import_reference():
    if not os.path.isdir(os.path.join(REF, "serving")):
        raise RuntimeError("no copy of the reference under baseline/_ref (run baseline/build_reference.py)")
    for sub in ("", "kernels/pagedattn"):
        p = os.path.join(REF, sub) if sub else REF
        if p not in sys.path:
            sys.path.insert(0, p)
    if "tiktoken" not in sys.modules or not hasattr(sys.modules["tiktoken"], "_stand_in"):
        fake = types.ModuleType("tiktoken")
        fake._stand_in = True
        fake.get_encoding = lambda name: None
        sys.modules["tiktoken"] = fake
    from models.model_config import ModelConfig
    from serving.paged_model import PagedTransformer
    from serving.kv_pool import KVPool
    from serving.allocator import BlockAllocator
    from serving.sequence import Sequence
    from serving.batch import build_batch_step
    from serving.generation import generate_batched
    return ModelConfig, PagedTransformer, KVPool, BlockAllocator, Sequence, build_batch_step, generate_batched


def build(ref, sizes, block_size, num_blocks, device):
    import torch
    ModelConfig, PagedTransformer, KVPool, BlockAllocator = ref[:4]
    hidden = sizes["hidden_size"]

    class Config(ModelConfig):
        @property
        def hidden_size(self):
            return hidden

    cfg = Config(vocab_size=sizes["vocab_size"], d_model=sizes["d_model"], num_layers=sizes["num_layers"],
                 num_heads=sizes["num_heads"], num_kv_heads=sizes["num_kv_heads"], max_seq_len=sizes["max_seq_len"], bias=False)
    with torch.device(device):
        model = PagedTransformer(cfg, backend="pytorch")
    model = model.half().eval()
    pool = KVPool(cfg.num_layers, block_size, num_blocks, cfg.num_kv_heads, cfg.head_dim, torch.float16, device)
    return cfg, model, pool, BlockAllocator(num_blocks)


def decode_loop(ref, model, pool, alloc, prompts, block_size, warmup, steps, device):
    """serving/generation.py:121-143 with events around the last ``steps`` iterations."""
    import torch
    Sequence, build_batch_step = ref[4], ref[5]
    seqs = [Sequence(i, list(p), block_size) for i, p in enumerate(prompts)]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        with torch.no_grad():
            for s in seqs:
                s.ensure_blocks(alloc)
            batch = build_batch_step([(s, s.token_ids) for s in seqs], device)
            logits = model.forward_batch(batch, pool)
            next_tokens = [int(logits[i].argmax()) for i in range(len(seqs))]
            finite = bool(torch.isfinite(logits).all())
            for it in range(warmup + steps):
                if it == warmup:
                    torch.cuda.synchronize()
                    a.record()
                for s, t in zip(seqs, next_tokens):
                    s.append_token(t)
                    s.ensure_blocks(alloc)
                batch = build_batch_step([(s, [t]) for s, t in zip(seqs, next_tokens)], device)
                logits = model.forward_batch(batch, pool)
                next_tokens = [int(logits[i].argmax()) for i in range(len(seqs))]
            b.record()
            torch.cuda.synchronize()
            finite = finite and bool(torch.isfinite(logits).all())
    finally:
        for s in seqs:
            s.release(alloc)
    return a.elapsed_time(b), finite


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--tiny-only", action="store_true")
    args = ap.parse_args()
    W, K, B, ctx = max(args.warmup, 3), args.steps, args.batch, args.ctx
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        ref = import_reference()
    except Exception as e:                                   # noqa: BLE001 - whatever stops the import is the reason
        return unavailable(f"the reference does not import here: {type(e).__name__}: {e}")
    device = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    block = 64

    # ---- a tiny model first
    tiny = dict(vocab_size=256, d_model=64, num_layers=2, num_heads=4, num_kv_heads=1, hidden_size=176, max_seq_len=128)
    try:
        _, model, pool, alloc = build(ref, tiny, 16, 64, device)
        prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (5, 17, 33)]
        _, finite = decode_loop(ref, model, pool, alloc, prompts, 16, 2, 4, device)
        outs = ref[6](model, prompts, 6, pool, alloc, 16)
        if not finite or [len(o) for o in outs] != [6, 6, 6]:
            return unavailable("the reference's paged path gives logits that are not finite on a tiny model on this GPU")
        del model, pool
    except Exception as e:                                   # noqa: BLE001
        return unavailable(f"the reference's paged path fails on a tiny model here: {type(e).__name__}: {e}")
    if args.tiny_only:
        print(json.dumps({"impl": "reference", "tiny": "ok"}))
        return 0

    # ---- the benchmark's sizes
    sizes = dict(vocab_size=32000, d_model=4096, num_layers=args.layers, num_heads=32, num_kv_heads=1, hidden_size=11008,
                 max_seq_len=ctx)
    try:
        num_blocks = B * (-(-ctx // block)) + 2
        _, model, pool, alloc = build(ref, sizes, block, num_blocks, device)
        start_len = ctx - (W + K) - 1
        prompts = [torch.randint(0, sizes["vocab_size"], (start_len,), generator=g).tolist() for _ in range(B)]
        ms, finite = decode_loop(ref, model, pool, alloc, prompts, block, W, K, device)
        if not finite:
            return unavailable("the reference's paged path gives logits that are not finite at the benchmark's sizes")
        generate_batched = ref[6]

        def whole(n):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = generate_batched(model, prompts, n, pool, alloc, block)
            torch.cuda.synchronize()
            assert all(len(o) == n for o in out)
            return time.perf_counter() - t0

        whole(1)
        t_short, t_long = whole(1 + W), whole(1 + W + K)
        e2e_s = max(t_long - t_short, 1e-9)
    except Exception as e:                                   # noqa: BLE001
        return unavailable(f"the reference's paged path fails at the benchmark's sizes: {type(e).__name__}: {e}")
    out = {
        "impl": "reference", "metric": "decode tokens/s (batch 8, context 4096)", "value": B * K / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic token ids, default-initialised weights",
        "config": {"model": "llama2-7b-sizes-mqa", "global_batch": B, "seq_len": ctx, "parallelism": "single-gpu",
                   "layers": args.layers, "layers_in_config": 32, "d_model": 4096, "heads": 32, "kv_heads": 1, "head_dim": 128,
                   "ffn_hidden": 11008, "vocab": 32000, "page_size": block, "prompt_len": start_len,
                   "l2": "inputs larger than L2 (weights 11 GB per step)", "path": "serving.generation.generate_batched loop"},
        "e2e": {"value": B * K / e2e_s, "unit": "tokens/s", "steps": K, "method": "generate_batched(1+W+K) minus generate_batched(1+W)",
                "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
        "gpu_launches": None,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
