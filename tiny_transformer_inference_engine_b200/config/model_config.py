"""Typed model configuration read from a model folder's ``config.json``.

The keys are the field names of the reference's ``ModelConfig``
(models/model_config.py:10-22): ``vocab_size, d_model, num_layers, num_heads,
num_kv_heads, max_seq_len, causal, dropout, bias, dtype, eos_token_id,
rope_theta, rms_norm_eps``.  Two keys are added:

* ``hidden_size`` - the feed-forward width.  In the reference it is a read-only
  property equal to ``d_model`` (models/model_config.py:32-34) although the
  SwiGLU class takes any width (models/mlp.py:18); here it is a real key whose
  default is ``d_model``.
* ``architecture`` - the registry name of the model.  A config without it is
  the reference's own (and only) architecture.

``rope_theta`` and ``rms_norm_eps`` are declared by the reference but never
passed to its layers (models/mqa.py:135, models/transformer_block.py:144); here
they reach the rotary position encoding and the norms.

The sizes have no defaults: a config.json that lacks one is an error, so that
no model size ever lives in code.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, fields, asdict
from typing import Any, Dict, Optional

DEFAULT_ARCHITECTURE = "mqa_gpt"

_DTYPE_NAMES = {
    "float32": "float32", "fp32": "float32", "torch.float32": "float32",
    "bfloat16": "bfloat16", "bf16": "bfloat16", "torch.bfloat16": "bfloat16",
    "float16": "float16", "fp16": "float16", "torch.float16": "float16",
}

_REQUIRED = ("vocab_size", "d_model", "num_layers", "num_heads", "max_seq_len")


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the named architecture."""


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int
    d_model: int
    num_layers: int
    num_heads: int
    max_seq_len: int
    num_kv_heads: int = 1
    hidden_size: Optional[int] = None      # feed-forward width; None -> d_model
    causal: bool = True
    dropout: float = 0.0
    bias: bool = False
    dtype: str = "float32"                 # dtype the weights were trained in (informative)
    eos_token_id: Optional[int] = None
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    architecture: str = DEFAULT_ARCHITECTURE
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self):
        for name in _REQUIRED + ("num_kv_heads",):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config key {name!r} must be a positive integer, got {v!r}")
        if self.hidden_size is None:
            object.__setattr__(self, "hidden_size", self.d_model)
        if not isinstance(self.hidden_size, int) or self.hidden_size <= 0:
            raise ConfigError(f"config key 'hidden_size' must be a positive integer, got {self.hidden_size!r}")
        # same checks as models/model_config.py:24-26
        if self.d_model % self.num_heads != 0:
            raise ConfigError(f"d_model={self.d_model} is not a multiple of num_heads={self.num_heads}")
        if self.num_heads % self.num_kv_heads != 0:
            raise ConfigError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head size {self.head_dim} must be even for rotary pairs (models/rope.py:8)")
        if not self.causal:
            raise ConfigError("causal=false is not supported: the reference model always attends causally "
                              "(models/transformer_block.py:152)")
        if self.dtype not in _DTYPE_NAMES:
            raise ConfigError(f"unknown dtype {self.dtype!r}; known: {sorted(set(_DTYPE_NAMES.values()))}")
        object.__setattr__(self, "dtype", _DTYPE_NAMES[self.dtype])
        if not (isinstance(self.rope_theta, (int, float)) and math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be a positive number, got {self.rope_theta!r}")
        if not (isinstance(self.rms_norm_eps, (int, float)) and math.isfinite(self.rms_norm_eps) and self.rms_norm_eps >= 0):
            raise ConfigError(f"rms_norm_eps must be a non-negative number, got {self.rms_norm_eps!r}")
        if self.eos_token_id is not None and not (0 <= int(self.eos_token_id)):
            raise ConfigError(f"eos_token_id must be >= 0 or null, got {self.eos_token_id!r}")

    # -- derived, as models/model_config.py:28-30 -------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.d_model // self.num_heads

    # -- I/O --------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raw = dict(raw)
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json lacks required key(s) {missing}; required: {list(_REQUIRED)}")
        arch = raw.pop("architecture", None)
        if arch is None:
            arch = raw.pop("model_type", None)
        if arch is None and isinstance(raw.get("architectures"), (list, tuple)) and raw["architectures"]:
            arch = raw.pop("architectures")[0]
        known = {f.name for f in fields(cls)} - {"extra", "architecture"}
        kwargs = {k: raw.pop(k) for k in list(raw) if k in known}
        if "dtype" in kwargs:
            kwargs["dtype"] = str(kwargs["dtype"])
        # unknown keys are kept aside, like the reference's filter (inference.py:28-29) drops them
        return cls(architecture=arch or DEFAULT_ARCHITECTURE, extra=raw, **kwargs)

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.isfile(path):
            raise ConfigError(f"no config.json at {path}")
        with open(path, "r", encoding="utf-8") as f:
            try:
                raw = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path} is not valid JSON: {e}") from e
        if not isinstance(raw, dict):
            raise ConfigError(f"{path} must hold a JSON object")
        return cls.from_dict(raw)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra")
        d.update({k: v for k, v in extra.items() if k not in d})
        return d

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
        return path
