"""The reference's architecture as data: Llama-style multi-query GPT.

models/transformer_block.py:140-182 - token embedding, ``num_layers`` pre-norm blocks
(RMSNorm, rotary multi-query attention, RMSNorm, SwiGLU), final RMSNorm, untied
``lm_head``.  Tensor names are the reference's state-dict keys
(``embedding.embedding.weight``, ``layers.{i}.attn_norm.weight``,
``layers.{i}.attn.{q_proj,k_proj,v_proj,out}.weight``, ``layers.{i}.mlp_norm.weight``,
``layers.{i}.mlp.{gate_proj,up_proj,down_proj}.weight``, ``final_norm.weight``,
``lm_head.weight``; ``.bias`` on the seven linears iff ``bias``).  Every size and
constant comes from the configuration.
"""
from __future__ import annotations

from ..config import ModelConfig
from ..parts.base import PartSpec, LayerSpec, RunEntry, ModelSpec
from ..registry import register_model


@register_model("mqa_gpt")
def mqa_gpt(config: ModelConfig) -> ModelSpec:
    d, D = config.d_model, config.head_dim
    position = PartSpec("rope", "", {"dim": D, "base": config.rope_theta, "style": "interleaved"})
    layers = []
    for i in range(config.num_layers):
        p = f"layers.{i}"
        block = PartSpec("pre_norm", p, {
            "mixer_norm": PartSpec("rmsnorm", f"{p}.attn_norm", {"dim": d, "eps": config.rms_norm_eps}),
            "mixer": PartSpec("attention", f"{p}.attn", {
                "d_model": d, "num_heads": config.num_heads, "num_kv_heads": config.num_kv_heads,
                "head_dim": D, "position": position, "bias": config.bias}),
            "ffn_norm": PartSpec("rmsnorm", f"{p}.mlp_norm", {"dim": d, "eps": config.rms_norm_eps}),
            "ffn": PartSpec("swiglu", f"{p}.mlp", {"d_model": d, "hidden": config.hidden_size, "bias": config.bias}),
        })
        layers.append(LayerSpec(block))
    return ModelSpec(
        d_model=d, vocab_size=config.vocab_size, max_seq_len=config.max_seq_len,
        embedding=PartSpec("token", "embedding.embedding", {"vocab_size": config.vocab_size, "dim": d}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(config.num_layers)),
        final_norm=PartSpec("rmsnorm", "final_norm", {"dim": d, "eps": config.rms_norm_eps}),
        head=PartSpec("linear", "lm_head", {"dim": d, "vocab_size": config.vocab_size}),
        eos_token_id=config.eos_token_id,
    )
