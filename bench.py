#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the layer sizes of BASELINE.json's configs[2] (Llama-2-7B sizes with one kv
head: 32 layers, width 4096, 32 heads of 128, SwiGLU 11008, vocabulary 32000), random bfloat16
weights, batch 8, context 4096.  A step is one decode step of the whole batch.  One JSON line
is printed: ``value`` = decoded tokens per second timed on the device over exactly K steps;
``e2e`` = the same through ``Engine.step()`` with host tokens in and out; ``prefill`` = one
2,048-token prompt; ``roofline`` = bytes a decode step must read / time / measured HBM peak;
``points`` = decode at batch 1 and 64.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_json(name):
    try:
        with open(os.path.join(ROOT, name)) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def peaks():
    m = load_json("MEASURED_PEAKS.json") or {}
    out, src = dict(FALLBACK_PEAKS), "fallback"
    def find(d, key):
        if isinstance(d, dict):
            if key in d and isinstance(d[key], (int, float)):
                return float(d[key])
            for v in d.values():
                r = find(v, key)
                if r is not None:
                    return r
        return None
    for k in ("hbm_gbs", "bf16_tflops"):
        v = find(m, k)
        if v:
            out[k], src = v, "measured"
    out["source"] = src
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg, layers):
    """Bytes a decode step must read and flops of a prefill, from the shapes (2 bytes per value)."""
    d, F, V, Hq, Hkv = cfg["d_model"], cfg["hidden_size"], cfg["vocab_size"], cfg["num_heads"], cfg["num_kv_heads"]
    D = d // Hq
    per_layer = (Hq + 2 * Hkv) * D * d + d * Hq * D + 3 * F * d + 2 * d
    weights = layers * per_layer + V * d + d                     # lm_head + final norm; embedding rows are counted per token
    kv_per_token = layers * 2 * Hkv * D * 2
    return {"matmul_params": layers * ((Hq + 2 * Hkv) * D * d + d * Hq * D + 3 * F * d), "weights_bytes": 2 * weights,
            "kv_bytes_per_token": kv_per_token, "head_dim": D, "lm_head_params": V * d}


def build_engine(cfg, layers, batch, ctx, graphs, seed=0):
    import torch
    from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
    from tiny_transformer_inference_engine_b200.weights import random_tensors
    mc = ModelConfig.from_dict({**cfg, "num_layers": layers})
    w = random_tensors(mc, seed, store_dtype="bfloat16", device="cuda:0")
    page = 64
    pages = batch * (-(-ctx // page)) + 2 * batch + 2        # admission keeps a growth page per running request
    ec = EngineConfig(dtype="bfloat16", device="cuda:0", use_cuda_graphs=True,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=max(2048, batch),
                                            cudagraph_batch_sizes=graphs))
    eng = Engine(mc, w, ec)
    del w
    torch.cuda.empty_cache()
    return eng


def timed(fn, steps):
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


def decode_kernel_path(eng, batch, start_len, steps, warmup, vocab, synthetic_fill, prefix="b"):
    """Device-timed decode: K steps of (metadata copy, captured model step, sampling kernel)."""
    import torch
    from tiny_transformer_inference_engine_b200 import StepEntry, SamplingParams
    mgr, g = eng.manager, torch.Generator().manual_seed(1)
    rids = [f"{prefix}{i}" for i in range(batch)]
    for rid in rids:
        mgr.admit(rid)
        eng.sampler.set_request(mgr.slot_of[rid], SamplingParams(temperature=0.8, seed=mgr.slot_of[rid]))
    if synthetic_fill:
        for rid in rids:
            mgr.extend(rid, 0, start_len)
        for grp in mgr.groups:
            grp.kv.normal_(0, 0.5)
    else:
        chunk = 2048
        for rid in rids:
            for s in range(0, start_len, chunk):
                n = min(chunk, start_len - s)
                mgr.extend(rid, s, s + n)
                eng.stepper.step([StepEntry(rid, s, torch.randint(0, vocab, (n,), generator=g).tolist(), [])])
    tokens = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()
    slot_ids = torch.tensor([mgr.slot_of[r] for r in rids], dtype=torch.int32, device="cuda:0")
    pos = [start_len]

    def one(i, base=0):
        for rid in rids:
            mgr.extend(rid, pos[0], pos[0] + 1)
        entries = [StepEntry(rid, pos[0], [tokens[base + i][j]], [0]) for j, rid in enumerate(rids)]
        logits = eng.stepper.step(entries, eng.sampler)         # a captured step samples inside its graph
        if eng.stepper.last_tokens is None:
            eng.sampler.sample(logits, slot_ids)
        pos[0] += 1

    for i in range(warmup):
        one(i)
    l0 = eng.ops.launches
    ms = timed(lambda i: one(i, warmup), steps)
    for rid in rids:
        mgr.release(rid)
    return ms, pos[0], eng.ops.launches - l0


WORKLOADS = {
    # BASELINE.json configs[3]: Falcon-7B widths in Llama style, a mixed batch of 32 requests
    "falcon_mixed": dict(
        cfg=dict(architecture="mqa_gpt", vocab_size=65024, d_model=4544, num_layers=32, num_heads=71, num_kv_heads=1,
                 hidden_size=18176, max_seq_len=2048, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="bfloat16"),
        requests=32, prompt_lo=64, prompt_hi=1024, new_tokens=128, token_budget=2048, page=64),
    # BASELINE.json configs[4]: Gemma-2B layer sizes, 6,144-token prompts in 512-token portions beside decode
    "gemma_chunked": dict(
        cfg=dict(architecture="mqa_gpt", vocab_size=256000, d_model=2048, num_layers=18, num_heads=8, num_kv_heads=1,
                 hidden_size=16384, max_seq_len=8192, rope_theta=10000.0, rms_norm_eps=1e-6, bias=False, dtype="bfloat16"),
        requests=16, prompt_lo=6144, prompt_hi=6144, new_tokens=256, token_budget=512, page=64),
}


def run_workload(name, pk, layers=None, split_classes=True):
    """One of BASELINE.json's serving workloads through ``Engine.generate`` (host token lists in and out): requests are
    admitted, their prompts cut into portions under the token budget and run beside the decoded tokens of the others.
    Timed by the host's clock around the whole call, after one untimed run of the same workload; the faster of two timed
    runs counts.  ``frac`` is the sum
    over the steps of the time each would need at the roofline (the larger of bytes / HBM peak and flops / bf16 peak)
    divided by the time taken."""
    import torch
    from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams
    from tiny_transformer_inference_engine_b200.weights import random_tensors
    w = WORKLOADS[name]
    cfg, n_req, page = w["cfg"], w["requests"], w["page"]
    full_layers = cfg["num_layers"]
    layers = layers or full_layers
    mc = ModelConfig.from_dict({**cfg, "num_layers": layers})
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(w["prompt_lo"], w["prompt_hi"] + 1, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + w["new_tokens"]) // page) for n in lens) + 2 * n_req + 2
    ec = EngineConfig(dtype="bfloat16", device="cuda:0", use_cuda_graphs=True, split_step_classes=split_classes,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=n_req, max_num_batched_tokens=w["token_budget"],
                                            cudagraph_batch_sizes=[1, 2, 4, 8, 16, 32]))
    eng = Engine(mc, random_tensors(mc, 0, store_dtype="bfloat16", device="cuda:0"), ec)
    torch.cuda.empty_cache()
    nums = model_numbers(cfg, layers)
    params = SamplingParams(max_new_tokens=w["new_tokens"], temperature=0.8, ignore_eos=True)
    log = []
    inner = eng.stepper.step

    def logged(entries, *a, **k):                                  # what each step ran, for the roofline sum
        log.append([(e.start, len(e.tokens)) for e in entries])
        return inner(entries, *a, **k)

    eng.stepper.step = logged
    eng.generate(prompts, params)                                   # untimed: graphs captured, kernels loaded
    # timed twice, the faster run counts: the host's clock around a whole workload also sees whatever else the host does
    # (the same workload on an idle and on a busy host of this pool: 1.22 and 1.3-2.3 s with the GPU's clocks unchanged)
    secs = []
    for _ in range(2):
        log.clear()
        l0 = eng.ops.launches
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = eng.generate(prompts, params)
        torch.cuda.synchronize()
        secs.append(time.perf_counter() - t0)
        assert all(len(o) == w["new_tokens"] for o in out)
    sec = min(secs)
    ideal, mixed_steps = 0.0, 0
    Hq, D = cfg["num_heads"], nums["head_dim"]
    for step in log:
        T = sum(n for _, n in step)
        keys = sum(s + n for s, n in step)
        flops = 2 * T * nums["matmul_params"] + 2 * len(step) * nums["lm_head_params"] \
            + layers * 4 * Hq * D * sum(n * s + n * (n + 1) // 2 for s, n in step)
        bytes_ = nums["weights_bytes"] + keys * nums["kv_bytes_per_token"]
        ideal += max(bytes_ / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
        mixed_steps += any(n == 1 for _, n in step) and any(n > 1 for _, n in step)
    gen = n_req * w["new_tokens"]
    res = {"value": gen / sec, "unit": "generated tokens/s", "seconds": sec, "seconds_of_both_runs": [round(t, 4) for t in secs], "prompt_tokens": sum(lens), "generated_tokens": gen,
           "all_tokens_per_s": (sum(lens) + gen) / sec, "steps": len(log), "mixed_steps": int(mixed_steps),
           "roofline_frac": ideal / sec, "layers": layers, "layers_in_config": full_layers,
           "requests": n_req, "token_budget": w["token_budget"], "page_size": page, "gpu_launches": eng.ops.launches - l0,
           "preemptions": eng.stats()["preemptions"]}
    del eng
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the Falcon-width and Gemma-size serving workloads")
    ap.add_argument("--only-workload", default=None, choices=sorted(WORKLOADS), help="run one serving workload and print its record")
    ap.add_argument("--no-class-split", action="store_true", help="with --only-workload: mixed steps as one attention launch (the comparison)")
    args = ap.parse_args()

    if args.impl == "reference":
        # The unmodified reference from baseline/_ref, in a process of its own (none of this package is imported there):
        # baseline/reference_arm.py builds its PagedTransformer at the same sizes and times its generate_batched loop.
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU"}))
            return 0
        cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(args.steps),
               "--warmup", str(max(args.warmup, 3)), "--batch", str(args.batch)]
        if args.layers:
            cmd += ["--layers", str(args.layers)]
        try:
            run = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
            lines = [l for l in run.stdout.strip().split("\n") if l.startswith("{")]
            if run.returncode == 0 and lines:
                print(lines[-1])
            else:
                tail = " ".join((run.stderr or run.stdout).split())[-300:]
                print(json.dumps({"impl": "reference", "unavailable": f"the reference's process ended with code {run.returncode}: {tail}"}))
        except subprocess.TimeoutExpired:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's process did not finish in 1500 s"}))
        return 0
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    if args.only_workload:
        print(json.dumps({args.only_workload: run_workload(args.only_workload, peaks(), args.layers, not args.no_class_split)}))
        return 0
    cfg = dict(architecture="mqa_gpt", vocab_size=32000, d_model=4096, num_layers=32, num_heads=32, num_kv_heads=1,
               hidden_size=11008, max_seq_len=4096, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="bfloat16")
    full_layers = cfg["num_layers"]
    layers = args.layers or full_layers
    ctx, batch, K, W = cfg["max_seq_len"], args.batch, args.steps, args.warmup
    pk = peaks()
    nums = model_numbers(cfg, layers)

    eng = build_engine(cfg, layers, max(batch, 1), ctx, sorted({1, batch}))
    vocab = cfg["vocab_size"]

    # ---- prefill of 2,048 tokens (one request, empty cache)
    from tiny_transformer_inference_engine_b200 import StepEntry, SamplingParams
    g = torch.Generator().manual_seed(0)
    Tp = 2048
    ptoks = torch.randint(0, vocab, (Tp,), generator=g).tolist()

    def prefill_once(_):
        eng.manager.admit("p")
        eng.manager.extend("p", 0, Tp)
        eng.stepper.step([StepEntry("p", 0, ptoks, [Tp - 1])])
        eng.manager.release("p")

    for i in range(3):
        prefill_once(i)
    p_ms = timed(prefill_once, 3) / 3
    p_flops = 2 * Tp * nums["matmul_params"] + 4 * cfg["num_heads"] * nums["head_dim"] * (Tp * (Tp + 1) // 2) * layers \
        + 2 * nums["lm_head_params"]
    prefill = {"value": Tp / (p_ms / 1e3), "tokens": Tp, "ms": p_ms,
               "frac": p_flops / (p_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode, device-timed
    start_len = ctx - (W + K)
    clocks = ClockSampler(); clocks.start()
    ms, end_len, launches = decode_kernel_path(eng, batch, start_len, K, W, vocab, synthetic_fill=False)
    clock_rec = clocks.stop()
    ms_per_step = ms / K
    value = batch * K / (ms / 1e3)
    mean_ctx = (start_len + W + end_len) / 2
    step_bytes = nums["weights_bytes"] + batch * cfg["d_model"] * 2 + batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "of": pk["source"]}

    # ---- decode end to end through Engine.step(): host tokens in, host tokens out
    # requests that finish their prompt early decode while the others still prefill, so each gets
    # room for those extra tokens and none finishes inside the timed region
    prefill_steps = -(-batch * start_len // 2048) + batch
    room = W + K + prefill_steps + 2
    e2e_prompt = ctx - room
    prompts = torch.randint(0, vocab, (batch, e2e_prompt), generator=g).tolist()
    for p in prompts:
        eng.add_request(p, SamplingParams(max_new_tokens=room, temperature=0.8, ignore_eos=True))
    while any(r.remaining > 1 for r in list(eng.scheduler.running) + list(eng.scheduler.waiting)) or eng.scheduler.waiting:
        eng.step()
    for _ in range(W):
        eng.step()
    n_e2e = K
    got = [0]

    def e2e_step(_):
        got[0] += len(eng.step())

    e_ms = timed(e2e_step, n_e2e)
    assert got[0] == batch * n_e2e, (got[0], batch, n_e2e)
    for r in list(eng.scheduler.running):
        eng.manager.release(r.rid)
    eng.scheduler.running.clear()
    h2d = 4 * (8 * (batch + 4) + batch * (-(-ctx // 64)) + 64)          # the step's packed int32 metadata
    e2e = {"value": got[0] / (e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
           "steps": n_e2e}

    # ---- other batch sizes
    points = {}
    eng = None
    torch.cuda.empty_cache()
    if not args.no_points:
        for b in (1, 64):
            e2 = build_engine(cfg, layers, b, ctx, [b])
            k2 = min(K, 32)
            # twice on the same engine, the better one kept: these are side figures of a few dozen steps, and one slow
            # stretch of the GPU (seen once: 9 x) would otherwise stand as the figure
            m2 = min(decode_kernel_path(e2, b, ctx - (W + k2), k2, W, vocab, synthetic_fill=True, prefix=tag)[0] for tag in ("p", "q"))
            points[f"decode_b{b}"] = b * k2 / (m2 / 1e3)
            del e2
            torch.cuda.empty_cache()

    workloads = {}
    if not args.no_workloads:
        for name in WORKLOADS:
            workloads[name] = run_workload(name, pk)

    out = {
        "metric": "decode tokens/s (batch 8, context 4096)", "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K,
        "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "config": {"model": "llama2-7b-sizes-mqa", "global_batch": batch, "seq_len": ctx, "parallelism": "single-gpu",
                   "layers": layers, "layers_in_config": full_layers, "d_model": cfg["d_model"], "heads": cfg["num_heads"],
                   "kv_heads": cfg["num_kv_heads"], "head_dim": nums["head_dim"], "ffn_hidden": cfg["hidden_size"],
                   "vocab": vocab, "page_size": 64, "prompt_len": start_len, "l2": "inputs larger than L2 (weights 11 GB per step)",
                   "cuda_graph": True, "sampling": "temperature 0.8 on device"},
        "e2e": e2e, "gpu_launches": launches, "e2e_prompt_len": e2e_prompt, "prefill": prefill, "roofline": roofline, "points": points, "workloads": workloads, "clocks": clock_rec,
        "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
