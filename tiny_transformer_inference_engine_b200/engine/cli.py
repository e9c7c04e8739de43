"""Command line in the manner of the reference's ``inference.py`` (inference.py:220-270).

Option names and meanings follow it where it has them: ``--tokens/--token`` (100),
``--temperature`` (1.0), ``--top-k/--top_k`` (0 = off), ``--top-p/--top_p`` (1.0 = off),
``--device`` (auto), ``--num-gpu-blocks`` (256), ``--block-size`` (16), ``--prompts`` for several
requests at once (its ``--serving`` path; here every run goes through the scheduler).  Where the
reference takes a checkpoint file (``--ckpt``), this takes a model folder (``--model``, or ``--ckpt``
as an alias) or such a file, which is converted on the way in (``weights/convert.py``).  Prompts are token ids (``--prompt-ids 1,2,3``, repeatable) or, as in the reference,
text (``--prompt "Once upon a time"``, repeatable), which is encoded and decoded with tiktoken's
``gpt2`` vocabulary (inference.py:256-269) if that package and its vocabulary file are there; without
them ``--prompt`` is refused with a message and token ids remain.  ``--random-config`` makes a random-weights
model from a config.json and ``--seed``.  Its backend, attention-type and quantization options have
no counterpart (one kernel path, one architecture, no quantized weights).
"""
from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tiny_transformer_inference_engine_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", "--ckpt", dest="model", help="folder with config.json and *.safetensors, or a checkpoint file of the reference")
    ap.add_argument("--random-config", help="config.json for a model with random weights (see --seed)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    ap.add_argument("--prompt-ids", "--prompts", dest="prompt_ids", action="append", default=[],
                    help="comma-separated token ids; give it several times for several requests")
    ap.add_argument("--prompt-ids-file", help="JSON file with a list of token-id lists")
    ap.add_argument("--prompt", dest="prompt_text", action="append", default=[],
                    help="a text prompt (tiktoken's gpt2 vocabulary, as the reference); may be given several times")
    ap.add_argument("--tokens", "--token", dest="tokens", type=int, default=100)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", "--top_k", dest="top_k", type=int, default=0)
    ap.add_argument("--top-p", "--top_p", dest="top_p", type=float, default=1.0)
    ap.add_argument("--greedy", action="store_true", help="argmax instead of sampling")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--serving", action="store_true", help="accepted for the reference's sake; every run is scheduled")
    ap.add_argument("--num-gpu-blocks", type=int, default=256)
    ap.add_argument("--kv-budget-bytes", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-num-seqs", type=int, default=32)
    ap.add_argument("--max-num-batched-tokens", type=int, default=512)
    ap.add_argument("--ignore-eos", action="store_true")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    # inference.py:241-242
    if args.tokens < 0 or args.temperature <= 0 or args.top_k < 0 or not 0 < args.top_p <= 1:
        ap.error("tokens/top-k must be nonnegative, temperature positive, and top-p in (0, 1]")
    if bool(args.model) == bool(args.random_config):
        ap.error("give exactly one of --model and --random-config")
    if args.block_size <= 0:
        ap.error("block_size must be positive")                                   # inference.py:203-204
    if args.num_gpu_blocks <= 0:
        ap.error("num_gpu_blocks must be positive")                               # inference.py:205-206
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            prompts.extend([int(t) for t in p] for p in json.load(f))
    texts = [None] * len(prompts)
    tokenizer = None
    if args.prompt_text:
        try:
            import tiktoken
            tokenizer = tiktoken.get_encoding("gpt2")                              # inference.py:256
        except Exception as e:                                                     # noqa: BLE001 - not installed, or no vocabulary file offline
            ap.error(f"--prompt needs tiktoken's gpt2 vocabulary ({type(e).__name__}: {e}); give --prompt-ids instead")
        for t in args.prompt_text:
            prompts.append(list(tokenizer.encode_ordinary(t)))                     # inference.py:262
            texts.append(t)
    if not prompts:
        ap.error("give at least one --prompt-ids or --prompt")

    import torch
    device = args.device
    if device == "auto":
        device = "cuda:0"                                                          # there is no CPU path to fall back to
    if not torch.cuda.is_available():
        ap.error("CUDA is unavailable and this engine has no CPU path")           # inference.py:253-254
    from .engine import Engine
    from ..config import EngineConfig, CacheConfig, SchedulerConfig
    from ..sampling import SamplingParams
    ec = EngineConfig(dtype=args.dtype, device=device,
                      cache=CacheConfig(block_size=args.block_size,
                                        num_gpu_blocks=None if args.kv_budget_bytes else args.num_gpu_blocks,
                                        kv_budget_bytes=args.kv_budget_bytes or 2 * 1024 ** 3),
                      sched=SchedulerConfig(max_num_seqs=args.max_num_seqs,
                                            max_num_batched_tokens=args.max_num_batched_tokens))
    if args.model:
        import os
        engine = Engine.from_checkpoint(args.model, ec) if os.path.isfile(args.model) else Engine.from_folder(args.model, ec)
    else:
        engine = Engine.from_random(args.random_config, args.seed, ec)
    params = [SamplingParams(max_new_tokens=args.tokens, temperature=args.temperature, top_k=args.top_k,
                             top_p=args.top_p, greedy=args.greedy, seed=args.seed + i, ignore_eos=args.ignore_eos)
              for i in range(len(prompts))]
    for prompt, text, out in zip(prompts, texts, engine.generate(prompts, params)):
        if text is None:
            print(json.dumps({"prompt_ids": prompt, "generated_ids": out}))
        else:
            print(text + tokenizer.decode(out))                                    # inference.py:269
    return 0


if __name__ == "__main__":
    sys.exit(main())
