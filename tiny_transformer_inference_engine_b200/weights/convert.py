"""Turns a checkpoint file of the reference into a model folder of this package.

    python -m tiny_transformer_inference_engine_b200.weights.convert CKPT.pt FOLDER

The reference saves ``{"model_config": ..., "model": state_dict, ...}`` with ``torch.save`` and reads
it back in ``inference.py:16-29,68-87``: the config keeps the fields of its ``ModelConfig``, the state
dict may carry the ``_orig_mod.`` prefix of a compiled model (inference.py:87).  The tensor names are
the ones this package loads by (models/mqa_gpt.py), so the tensors go into ``model.safetensors`` as
they are.  ``config.json`` gets the checkpoint's config fields and three values the reference does
not store but fixes in code, so that the folder describes the model that was trained:

* ``hidden_size``: the width of ``layers.0.mlp.gate_proj.weight`` (the reference's config property
  returns ``d_model``, models/model_config.py:32-34, while its SwiGLU takes any width, models/mlp.py:18);
* ``rope_theta = 10000.0``: its rotary table is built with the default base whatever the config says
  (models/mqa.py:52,135; models/rope.py:6);
* ``rms_norm_eps = 1e-5``: likewise its norms (models/transformer_block.py:144-146,169; models/rmsnorm.py:7).

A quantized checkpoint (``quant_metadata``, inference.py:89-98) is refused: there are no quantized
weights here.  The file is read with ``weights_only=True``; a checkpoint whose config was pickled as
an object rather than saved as a dict cannot be read that way and is refused with that reason.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict

import torch

from ..config import ModelConfig

_CONFIG_FIELDS = ("vocab_size", "d_model", "num_layers", "num_heads", "num_kv_heads", "max_seq_len", "causal", "dropout",
                  "bias", "eos_token_id")
_PREFIX = "_orig_mod."


class CheckpointError(ValueError):
    pass


def convert_checkpoint(ckpt_path: str, folder: str) -> ModelConfig:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` from the reference's checkpoint file; returns
    the configuration written."""
    from safetensors.torch import save_file
    try:
        ckpt = torch.load(ckpt_path, map_location="cpu", weights_only=True)
    except Exception as e:                                               # noqa: BLE001 - unpickling errors come in many classes
        raise CheckpointError(f"{ckpt_path} cannot be read as plain tensors and containers ({type(e).__name__}: {e}); "
                              "save its model_config as a dict") from e
    if not isinstance(ckpt, dict) or "model" not in ckpt:
        raise CheckpointError(f"{ckpt_path} holds no 'model' state dict (inference.py:87)")
    raw = ckpt.get("model_config")
    if raw is None:
        raise CheckpointError("checkpoint is missing model_config (inference.py:24-26)")
    if "quant_metadata" in ckpt:
        raise CheckpointError("a quantized checkpoint cannot be converted: this engine has no quantized weights")
    raw = dict(raw) if isinstance(raw, dict) else vars(raw)
    state: Dict[str, torch.Tensor] = {}
    for key, value in ckpt["model"].items():
        if not isinstance(value, torch.Tensor):
            raise CheckpointError(f"state dict entry {key!r} is not a tensor")
        name = key[len(_PREFIX):] if key.startswith(_PREFIX) else key
        if name in state:
            raise CheckpointError(f"tensor {name!r} appears twice once the {_PREFIX!r} prefix is dropped")
        state[name] = value.detach().contiguous()
    gate = state.get("layers.0.mlp.gate_proj.weight")
    if gate is None or gate.dim() != 2:
        raise CheckpointError("the state dict has no layers.0.mlp.gate_proj.weight to take the feed-forward width from")
    cfg: Dict[str, Any] = {k: raw[k] for k in _CONFIG_FIELDS if k in raw and raw[k] is not None}
    dtypes = {str(t.dtype).replace("torch.", "") for t in state.values() if t.is_floating_point()}
    cfg.update(architecture="mqa_gpt", hidden_size=int(gate.shape[0]), rope_theta=10000.0, rms_norm_eps=1e-5,
               dtype=dtypes.pop() if len(dtypes) == 1 else "float32")
    config = ModelConfig.from_dict(cfg)                                  # refuses what cannot describe a model
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    save_file(state, os.path.join(folder, "model.safetensors"), metadata={"source": os.path.basename(ckpt_path)})
    return config


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tiny_transformer_inference_engine_b200.weights.convert", description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoint", help="the reference's checkpoint file (torch.save of model_config and model)")
    ap.add_argument("folder", help="where config.json and model.safetensors go")
    args = ap.parse_args(argv)
    try:
        config = convert_checkpoint(args.checkpoint, args.folder)
    except (CheckpointError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(json.dumps({"folder": args.folder, "layers": config.num_layers, "d_model": config.d_model, "hidden_size": config.hidden_size,
                      "vocab_size": config.vocab_size, "dtype": config.dtype}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
