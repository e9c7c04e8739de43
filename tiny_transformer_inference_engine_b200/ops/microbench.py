"""Per-kernel timings against their rooflines, at the sizes of a model configuration.

    python -m tiny_transformer_inference_engine_b200.ops.microbench [--what decode|prefill|gemm_tc|attention|prefill_attention|mixed|tune|all]
                                                                    [--batch 8] [--ctx 4096] [--tokens 2048]

Every kernel is timed alone inside a captured CUDA graph of ``--iters`` launches (so the host's launch
cost is not in the number), over inputs that rotate through more than the L2's 126 MB where the
kernel streams weights.  Printed: microseconds per launch, the bytes or flops the kernel has to move,
and the fraction of the peak (``MEASURED_PEAKS.json`` beside the repository root if present, else
6.65 TB/s and 1.59 PFLOP/s).  The defaults are the Llama-2-7B layer sizes with one kv head.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import get_ops

DEV = "cuda:0"


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)

        def find(d, key):
            if isinstance(d, dict):
                if isinstance(d.get(key), (int, float)):
                    return float(d[key])
                for v in d.values():
                    r = find(v, key)
                    if r:
                        return r
            return None
        hbm, tf, src = find(m, "hbm_gbs") or hbm, find(m, "bf16_tflops") or tf, "measured"
    except (OSError, ValueError):
        pass
    return hbm, tf, src


EAGER = False        # --eager: plain launches between two events (what a profiler sees as single kernels), few of them


def timeit(fn, iters=24, warm=3):
    """Microseconds per call of ``fn(i)``, measured as one replay of a graph of ``iters`` calls."""
    if EAGER:
        fn(0)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(2):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 2 * 1e3
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e3


def line(name, us, bytes_=None, flops=None):
    hbm, tf, src = peaks()
    parts = [f"{name:42s} {us:9.1f} us"]
    if bytes_ is not None:
        gbs = bytes_ / us / 1e3
        parts.append(f"{bytes_ / 1e6:9.1f} MB {gbs:8.0f} GB/s = {gbs / hbm:5.2f} of {src} HBM peak")
    if flops is not None:
        t = flops / us / 1e6
        parts.append(f"{flops / 1e9:9.1f} GF {t:7.0f} TF/s = {t / tf:5.2f} of {src} bf16 peak")
    print("  ".join(parts), flush=True)


def decode(ops, a):
    d, F, V, Hq, Hkv, D = a.d_model, a.hidden, a.vocab, a.heads, a.kv_heads, a.d_model // a.heads
    B, ctx, page = a.batch, a.ctx, 64
    print(f"== decode step kernels, batch {B}, context {ctx}")

    def weights(N, K):
        n = max(2, int(400e6 // (N * K * 2)))
        return [torch.randn(N, K, device=DEV).bfloat16() * 0.02 for _ in range(n)]

    x = torch.randn(B, d, device=DEV).bfloat16()
    for name, N, K in (("qkv projection", (Hq + 2 * Hkv) * D, d), ("output projection", d, Hq * D), ("down projection", d, F),
                       ("lm_head", V, d)):
        ws = weights(N, K)
        ops.tune_products(ws)                                        # as when a model is loaded: the product and its form by measurement
        xin = torch.randn(B, K, device=DEV).bfloat16()
        f32 = torch.float32 if name == "lm_head" else None
        line(f"{name}", timeit(lambda i: ops.linear(xin, ws[i % len(ws)], None, out_dtype=f32, partial_ok=f32 is None)),
             bytes_=N * K * 2)
    ws = weights(2 * F, d)
    line("gate/up projection + SwiGLU", timeit(lambda i: ops.linear_swiglu(x, ws[i % len(ws)], None, F)), bytes_=2 * F * d * 2)
    resid, part, w = torch.randn(B, d, device=DEV), torch.randn(4, B, d, device=DEV), torch.ones(d, device=DEV)
    out = torch.empty(B, d, device=DEV, dtype=torch.bfloat16)
    line("residual add (4 partial sums) + RMSNorm", timeit(lambda i: ops.add_rmsnorm(resid, part, w, 1e-5, out)), bytes_=B * d * (4 * 5 + 4 + 2))
    nb = B * -(-ctx // page) + 1                                     # pages of whole requests, and the scratch page
    kp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    vp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    table = (torch.arange(B * -(-ctx // page), device=DEV, dtype=torch.int32) + 1).view(B, -1)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    tseq = torch.arange(B, dtype=torch.int32, device=DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))).to(DEV)
    qkvp = torch.randn(4, B, (Hq + 2 * Hkv) * D, device=DEV)
    q = torch.empty(B, Hq * D, device=DEV, dtype=torch.bfloat16)
    cs = ops.rope_table(pos, inv)
    line("rotate + store k/v (from 4 partial sums)", timeit(lambda i: ops.rope_store(qkvp, Hq, Hkv, D, pos, tseq, inv, 0, kp, vp, table, page, True, q_out=q, cs_table=cs)),
         bytes_=B * (Hq + 2 * Hkv) * D * (4 * 4 + 2))
    qsl = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    sl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    o = torch.empty(B, Hq * D, device=DEV, dtype=torch.bfloat16)
    plan = ops.attention_plan(torch.bfloat16, B, Hq, Hkv, D, 1, ctx, page)
    line(f"paged attention {plan} + merge", timeit(lambda i: ops.paged_attention(q, Hq, Hkv, D, kp, vp, table, page, qsl, sl, B, 1, ctx, 1 / math.sqrt(D), 0, o)),
         bytes_=B * ctx * Hkv * D * 2 * 2)
    logits = torch.randn(B, V, device=DEV)
    st = torch.zeros(max(B, 1), 8, dtype=torch.int32, device=DEV)
    st[:, 4] = 0x3f800000
    st[:, 5] = 0x3f800000
    tok = torch.empty(B, dtype=torch.int32, device=DEV)
    line("sampling (temperature)", timeit(lambda i: ops.sample(logits, tseq, st, tok)), bytes_=B * V * 4)
    st[:, 3] = 32
    st[:, 5] = 0x3f666666                                     # top-k 32, top-p 0.9
    line("sampling (temperature, top-k 32, top-p 0.9)", timeit(lambda i: ops.sample(logits, tseq, st, tok)), bytes_=B * V * 4)


def prefill(ops, a):
    d, F, Hq, Hkv, D = a.d_model, a.hidden, a.heads, a.kv_heads, a.d_model // a.heads
    T, page = a.tokens, 64
    print(f"== prefill kernels, one prompt of {T} tokens")
    resid, delta, w = torch.randn(T, d, device=DEV), torch.randn(T, d, device=DEV).bfloat16(), torch.ones(d, device=DEV)
    out = torch.empty(T, d, device=DEV, dtype=torch.bfloat16)
    line("residual add + RMSNorm", timeit(lambda i: ops.add_rmsnorm(resid, delta, w, 1e-5, out), iters=8), bytes_=T * d * (4 + 4 + 2 + 2))
    gu = torch.randn(T, 2 * F, device=DEV).bfloat16()
    act = torch.empty(T, F, device=DEV, dtype=torch.bfloat16)
    line("SwiGLU activation", timeit(lambda i: ops.swiglu(gu, act), iters=8), bytes_=T * F * 2 * 3)
    nb = T // page + 2
    kp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    vp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    table = (torch.arange(nb - 1, device=DEV, dtype=torch.int32) + 1).view(1, -1)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    tseq = torch.zeros(T, dtype=torch.int32, device=DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))).to(DEV)
    cs = ops.rope_table(pos, inv)
    line("rotate + store k/v", timeit(lambda i: ops.rope_store(qkv, Hq, Hkv, D, pos, tseq, inv, 0, kp, vp, table, page, True, cs_table=cs), iters=8),
         bytes_=T * (Hq + 2 * Hkv) * D * 2 * 2)
    qsl = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    sl = torch.tensor([T], dtype=torch.int32, device=DEV)
    o = torch.empty(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    planned = ops.attention_plan(torch.bfloat16, 1, Hq, Hkv, D, T, T, page)
    for plan in dict.fromkeys([planned, ("tcpp", 1, 0), ("tc", 1, 0), ("mma", 1, 0)]):
        if plan[0].startswith("tc") and not ops.lib.ttie_attn_tc_supported(D, page):
            continue
        if (plan[0] == "tc" and D > 128) or (plan[0] == "mma" and not ops.lib.ttie_attn_mma_supported(D)):
            continue
        line(f"causal paged attention {plan}", timeit(lambda i: ops.paged_attention(qkv, Hq, Hkv, D, kp, vp, table, page, qsl, sl, 1, T, T, 1 / math.sqrt(D), 0, o, plan=plan), iters=4),
             flops=4 * Hq * D * T * (T + 1) // 2)
    err = ops.tc_error()
    if err:
        raise RuntimeError(f"a tensor-core kernel reported wait failure code {err}")


def prefill_attention(ops, a):
    """Causal attention over prompt lengths and three head layouts (32 heads of 128, 71 heads of 64, 8 heads of 256,
    one kv head each; pages of 64 and of 16 keys): the two-tile tcgen05 kernel (one tile at head size 256) beside the
    one-tile one, and a 512-token portion behind a long context with the planned split of the key range."""
    print("== causal attention of one prompt: two-tile tcgen05 kernel | one-tile tcgen05 kernel")
    for Hq, D, page in ((32, 128, 64), (71, 64, 64), (32, 128, 16), (8, 256, 64), (8, 256, 16)):
        for T in (512, 2048, 8192):
            nb = T // page + 2
            kp = torch.randn(nb, 1, page, D, device=DEV).bfloat16()
            vp = torch.randn(nb, 1, page, D, device=DEV).bfloat16()
            table = (torch.arange(nb - 1, device=DEV, dtype=torch.int32) + 1).view(1, -1)
            qkv = torch.randn(T, (Hq + 2) * D, device=DEV).bfloat16()
            qsl = torch.tensor([0, T], dtype=torch.int32, device=DEV)
            sl = torch.tensor([T], dtype=torch.int32, device=DEV)
            o = torch.empty(T, Hq * D, device=DEV, dtype=torch.bfloat16)
            for plan in dict.fromkeys([ops.attention_plan(torch.bfloat16, 1, Hq, 1, D, T, T, page), ("tcpp", 1, 0), ("tc", 1, 0)]):
                if plan[0] == "tc" and D > 128:
                    continue                                     # head size 256 has the one form
                us = timeit(lambda i: ops.paged_attention(qkv, Hq, 1, D, kp, vp, table, page, qsl, sl, 1, T, T, 1 / math.sqrt(D), 0, o, plan=plan), iters=4)
                line(f"{Hq} heads of {D}, pages of {page}, {T:5d} tokens {plan}", us, flops=4 * Hq * D * T * (T + 1) // 2)
    Hq, D, page, T, ctx = 32, 128, 64, 512, 8192
    nb = ctx // page + 2
    kp = torch.randn(nb, 1, page, D, device=DEV).bfloat16()
    vp = torch.randn(nb, 1, page, D, device=DEV).bfloat16()
    table = (torch.arange(nb - 1, device=DEV, dtype=torch.int32) + 1).view(1, -1)
    qkv = torch.randn(T, (Hq + 2) * D, device=DEV).bfloat16()
    qsl = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    sl = torch.tensor([ctx], dtype=torch.int32, device=DEV)
    o = torch.empty(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    flops = 4 * Hq * D * (T * (ctx - T) + T * (T + 1) // 2)
    for plan in dict.fromkeys([ops.attention_plan(torch.bfloat16, 1, Hq, 1, D, T, ctx, page), ("tcpp", 1, 0), ("tc", 1, 0)]):
        us = timeit(lambda i: ops.paged_attention(qkv, Hq, 1, D, kp, vp, table, page, qsl, sl, 1, T, ctx, 1 / math.sqrt(D), 0, o, plan=plan), iters=4)
        line(f"last {T} tokens of {ctx} {plan}", us, flops=flops)
    err = ops.tc_error()
    if err:
        raise RuntimeError(f"a tensor-core kernel reported wait failure code {err}")


def attention(ops, a):
    """Decode attention over batch sizes and context lengths: the planned kernel beside the mma.sync tile loop
    with split keys (the plan before the decode form and the tcgen05 splits existed)."""
    Hq, Hkv, D, page = a.heads, a.kv_heads, a.d_model // a.heads, 64
    print("== decode attention: planned kernel | mma.sync tile loop with split keys and merge")
    batches = [int(v) for v in a.attn_batches.split(",")]
    contexts = [int(v) for v in a.attn_contexts.split(",")] if a.attn_contexts else [512, 2048, a.ctx, 4 * a.ctx]
    for B in batches:
        for ctx in contexts:
            nb = B * -(-ctx // page) + 1
            kp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
            vp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
            table = (torch.arange(B * -(-ctx // page), device=DEV, dtype=torch.int32) + 1).view(B, -1)
            q = torch.randn(B, Hq * D, device=DEV).bfloat16()
            qsl = torch.arange(B + 1, dtype=torch.int32, device=DEV)
            sl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
            o = torch.empty(B, Hq * D, device=DEV, dtype=torch.bfloat16)
            planned = ops.attention_plan(torch.bfloat16, B, Hq, Hkv, D, 1, ctx, page)
            keep = ops._cluster_plan, ops._tc_split_plan
            ops._cluster_plan = ops._tc_split_plan = lambda *x: None
            loop = ops._attention_plan(torch.bfloat16, B, Hq, Hkv, D, 1, ctx, page)        # (not the kept answer)
            ops._cluster_plan, ops._tc_split_plan = keep
            for plan in (planned, loop):
                us = timeit(lambda i: ops.paged_attention(q, Hq, Hkv, D, kp, vp, table, page, qsl, sl, B, 1, ctx, 1 / math.sqrt(D), 0, o, plan=plan))
                line(f"batch {B:3d} context {ctx:6d} {plan}", us, bytes_=B * ctx * Hkv * D * 2 * 2)
    err = ops.tc_error()
    if err:
        raise RuntimeError(f"a tensor-core kernel reported wait failure code {err}")


def gemm_tc(ops, a):
    d, F, Hq, Hkv, D = a.d_model, a.hidden, a.heads, a.kv_heads, a.d_model // a.heads
    M = a.tokens
    print(f"== matrix products of a {M}-token portion: library product and the tcgen05 kernel of this package")
    for name, N, K in (("qkv", (Hq + 2 * Hkv) * D, d), ("out", d, Hq * D), ("gate_up", 2 * F, d), ("down", d, F)):
        x = torch.randn(M, K, device=DEV).bfloat16()
        w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
        flops = 2 * M * N * K
        line(f"{name} [{M}x{K}]x[{K}x{N}] library (cuBLAS)", timeit(lambda i: torch.mm(x, w.t()), iters=8), flops=flops)
        line(f"{name} [{M}x{K}]x[{K}x{N}] tcgen05 128x256", timeit(lambda i: ops.linear_tc(x, w, None, None, 256), iters=8), flops=flops)
        line(f"{name} [{M}x{K}]x[{K}x{N}] tcgen05 CTA pairs 256x256", timeit(lambda i: ops.linear_tc_pair(x, w, None), iters=8), flops=flops)
        if name == "gate_up":
            act = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
            line(f"{name} library + SwiGLU kernel", timeit(lambda i: ops.swiglu(torch.mm(x, w.t()), act), iters=8), flops=flops)
            line(f"{name} tcgen05 CTA pairs with SwiGLU epilogue", timeit(lambda i: ops.linear_swiglu_tc_pair(x, w, None, F), iters=8), flops=flops)
    err = ops.tc_error()
    if err:
        raise RuntimeError(f"a tensor-core kernel reported wait failure code {err}")


def mixed(ops, a):
    """The attention of a mixed step - ``--batch`` one-token requests with contexts of ``--ctx`` keys beside one 512-token
    portion behind 2,048 cached tokens - as one launch planned for the whole step, as the two launches the engine makes
    (one per class), and each class alone."""
    Hq, Hkv, D, page = a.heads, a.kv_heads, a.d_model // a.heads, 64
    B, ctx, Tp, behind = a.batch, a.ctx, 512, 2048
    print(f"== attention of a mixed step: {B} one-token requests at {ctx} keys beside a {Tp}-token portion behind {behind}")
    lens = [ctx] * B + [behind + Tp]
    q_lens = [1] * B + [Tp]
    pages_of = [-(-n // page) for n in lens]
    nb = sum(pages_of) + 1
    kp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    vp = torch.randn(nb, Hkv, page, D, device=DEV).bfloat16()
    table = torch.zeros(B + 1, max(pages_of), dtype=torch.int32)
    nxt = 1
    for i, n in enumerate(pages_of):
        table[i, :n] = torch.arange(nxt, nxt + n)
        nxt += n
    table = table.to(DEV)
    T = B + Tp
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    qsl_tail = torch.tensor([0, Tp], dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    o = torch.empty(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    sc = 1 / math.sqrt(D)
    nbytes = sum(lens) * Hkv * D * 2 * 2
    whole = lambda i: ops.paged_attention(qkv, Hq, Hkv, D, kp, vp, table, page, qsl, sl, B + 1, Tp, max(lens), sc, 0, o)
    first = lambda i: ops.paged_attention(qkv[:B], Hq, Hkv, D, kp, vp, table[:B], page, qsl[:B + 1], sl[:B], B, 1, ctx, sc, 0, o[:B])
    second = lambda i: ops.paged_attention(qkv[B:], Hq, Hkv, D, kp, vp, table[B:], page, qsl_tail, sl[B:], 1, Tp, behind + Tp, sc, 0, o[B:])
    line(f"one launch for the step {ops.attention_plan(torch.bfloat16, B + 1, Hq, Hkv, D, Tp, max(lens), page)}", timeit(whole, iters=8), bytes_=nbytes)
    line("two launches, one per class", timeit(lambda i: (first(i), second(i)), iters=8), bytes_=nbytes)
    line(f"the one-token requests alone {ops.attention_plan(torch.bfloat16, B, Hq, Hkv, D, 1, ctx, page)}", timeit(first, iters=8))
    line(f"the portion alone {ops.attention_plan(torch.bfloat16, 1, Hq, Hkv, D, Tp, behind + Tp, page)}", timeit(second, iters=8))


def tune(ops, a):
    """What ``CudaOps.tune_products`` measures at 8, 16, 32 and 64 rows for the model's matrix shapes: the library's
    product against this package's weight-streaming kernel in its best form (both rotate over several matrices of a shape)."""
    d, F, V, Hq, Hkv, D = a.d_model, a.hidden, a.vocab, a.heads, a.kv_heads, a.d_model // a.heads
    print("== products of 8 / 16 / 32 / 64 rows, us per launch: library | weight-streaming kernel -> choice for callers that take partial sums; for the others")
    weights = []
    for N, K in (((Hq + 2 * Hkv) * D, d), (d, Hq * D), (d, F), (V, d)):
        n = max(2, min(8, int(400e6 // (N * K * 2))))
        weights += [torch.randn(N, K, device=DEV).bfloat16() * 0.02 for _ in range(n)]
    ops._product_choice.clear()
    ops.tune_products(weights)
    for (N, K, M), took in sorted(ops.product_timings.items(), key=lambda kv: str(kv[0])):
        if N == "swiglu":
            continue
        form = took.get("skinny_form")
        print(f"[{N}, {K}] {M:3d} rows   {took['library'] * 1000 / 8:7.1f} | {took['skinny'] * 1000 / 8:7.1f}   -> {ops._product_choice[(N, K, M, 'split')]}"
              + (f"   (K in {form['k_ranges']} ranges, {form['row_sets']} row set(s) per CTA)" if form else "")
              + f"; K uncut {took['skinny_uncut'] * 1000 / 8:7.1f} -> {ops._product_choice[(N, K, M)]}", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--what", default="all", choices=("decode", "prefill", "gemm_tc", "attention", "prefill_attention", "mixed", "tune", "all"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--attn-batches", default="1,8,64", help="batch sizes of --what attention")
    ap.add_argument("--attn-contexts", default="", help="context lengths of --what attention (default 512, 2048, ctx, 4 ctx)")
    ap.add_argument("--eager", action="store_true", help="three plain launches per line instead of a replayed graph (for a profiler)")
    ap.add_argument("--skinny-max-rows", type=int, default=None, help="rows up to which the weight-streaming product is used (default: the engine's)")
    a = ap.parse_args(argv)
    global EAGER
    EAGER = a.eager
    ops = get_ops(DEV)
    if a.skinny_max_rows is not None:
        ops.skinny_max_rows = a.skinny_max_rows
    if a.what in ("decode", "all"):
        decode(ops, a)
    if a.what in ("prefill", "all"):
        prefill(ops, a)
    if a.what in ("gemm_tc", "all"):
        gemm_tc(ops, a)
    if a.what in ("attention", "all"):
        attention(ops, a)
    if a.what in ("prefill_attention", "all"):
        prefill_attention(ops, a)
    if a.what == "mixed":
        mixed(ops, a)
    if a.what == "tune":
        tune(ops, a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
