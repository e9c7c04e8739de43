"""Makes tests/golden/reference_logits.pt: logits of the REFERENCE's own model classes
(models/transformer_block.py ``Transformer``, pytorch backend, float32, CPU) on tiny random
models, for the plain implementation to be compared with once.

Run from the repository root:  python tests/golden/make_golden.py /path/to/reference/checkout

The reference's CUDA extension modules cannot be imported here (they are built for
another Python and GPU), so six empty stand-in modules are put into ``sys.modules``;
on the CPU with ``backend="pytorch"`` none of their functions is called.  The reference's
``ModelConfig.hidden_size`` is a property equal to ``d_model``, its norms fix eps and its
rotary table fixes the base in code; to express the tiny configurations the script
subclasses the config (hidden_size), sets ``eps`` on every RMSNorm and swaps in a
``RoPE`` built with the wanted base.  Nothing of the reference is copied.
"""
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.dont_write_bytecode = True


def reference_logits(ref_path, cfg, weights, prompts, chunked=None):
    for name in ("rmsnorm_cuda", "softmax_cuda", "rope_cuda", "flash_acc_reg_ext", "topk_cuda", "pagedattn"):
        sys.modules.setdefault(name, types.ModuleType(name))
    if ref_path not in sys.path:
        sys.path.insert(0, ref_path)
    from models.model_config import ModelConfig as RefConfig
    from models.transformer_block import Transformer
    from models.rope import RoPE
    from models.rmsnorm import RMSNorm
    from kv_cache import KVCache_kv

    hidden = cfg["hidden_size"]

    class Cfg(RefConfig):
        @property
        def hidden_size(self):
            return hidden

    rc = Cfg(vocab_size=cfg["vocab_size"], d_model=cfg["d_model"], num_layers=cfg["num_layers"],
             num_heads=cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"], max_seq_len=cfg["max_seq_len"],
             bias=cfg["bias"])
    model = Transformer(rc, attn_type="mqa", backend="pytorch").eval()
    for m in model.modules():
        if isinstance(m, RMSNorm):
            m.eps = cfg["rms_norm_eps"]
    for layer in model.layers:
        layer.attn.rope = RoPE(rc.head_dim, rc.max_seq_len, base=cfg["rope_theta"])
    model.load_state_dict({k: v.float() for k, v in weights.items()}, strict=True)
    out = []
    with torch.no_grad():
        for p in prompts:
            cache = KVCache_kv(rc.num_layers, 1, rc.num_kv_heads, rc.max_seq_len, rc.head_dim,
                               dtype=torch.float32, device="cpu")
            ids = torch.tensor([p], dtype=torch.long)
            out.append(model(ids, kv_cache=cache)[0].clone())
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference/checkout")
    ref_path = sys.argv[1]
    from tiny_configs import TINY_A, TINY_B, SEEDS
    from tiny_transformer_inference_engine_b200.config import ModelConfig
    from tiny_transformer_inference_engine_b200.weights import random_tensors
    from plain_model import plain_forward
    record = {}
    for name, cfg in (("A", TINY_A), ("B", TINY_B)):
        weights = random_tensors(ModelConfig.from_dict(cfg), SEEDS[name], perturb_norms=True)
        g = torch.Generator().manual_seed(100 + SEEDS[name])
        prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (1, 9, 33)]
        ref = reference_logits(ref_path, cfg, weights, prompts)
        worst = 0.0
        for p, r in zip(prompts, ref):
            mine = plain_forward(cfg, weights, p)
            worst = max(worst, ((mine - r).abs().max() / r.abs().max()).item())
        print(f"tiny {name}: plain vs reference, worst relative difference {worst:.3e}")
        record[name] = {"config": cfg, "seed": SEEDS[name], "prompts": prompts,
                        "logits": [r.to(torch.float32) for r in ref], "plain_vs_reference": worst}
    torch.save(record, os.path.join(HERE, "reference_logits.pt"))
    print("wrote", os.path.join(HERE, "reference_logits.pt"))


if __name__ == "__main__":
    main()
