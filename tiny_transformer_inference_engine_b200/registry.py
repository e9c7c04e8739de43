"""One registry from names to builders: architectures, and the parts they are made of.

``register_model(name)`` decorates a function ``ModelConfig -> ModelSpec``.
``register_part(category, kind)`` decorates a part class whose constructor takes
``prefix`` and the ``args`` of its ``PartSpec`` as keywords.  The reference picks
classes by ``attn_type``/``backend`` strings (models/transformer_block.py:32-46);
here the architecture name in config.json picks the builder.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .parts.base import PartSpec, Part

_MODELS: Dict[str, Callable] = {}
_PARTS: Dict[Tuple[str, str], type] = {}

CATEGORIES = ("norm", "position", "mixer", "ffn", "embedding", "head", "block")


class RegistryError(KeyError):
    def __str__(self):
        return self.args[0] if self.args else ""


def register_model(name: str):
    def deco(fn):
        if name in _MODELS and _MODELS[name] is not fn:
            raise RegistryError(f"architecture {name!r} is already registered")
        _MODELS[name] = fn
        return fn
    return deco


def unregister_model(name: str) -> None:
    _MODELS.pop(name, None)


def known_models():
    return sorted(_MODELS)


def model_spec(config):
    """The ModelSpec of ``config.architecture``."""
    try:
        builder = _MODELS[config.architecture]
    except KeyError:
        raise RegistryError(f"unknown architecture {config.architecture!r}; known: {known_models()}") from None
    return builder(config)


def register_part(category: str, kind: str):
    if category not in CATEGORIES:
        raise RegistryError(f"unknown part category {category!r}; known: {CATEGORIES}")

    def deco(cls):
        key = (category, kind)
        if key in _PARTS and _PARTS[key] is not cls:
            raise RegistryError(f"{category} {kind!r} is already registered")
        _PARTS[key] = cls
        return cls
    return deco


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def known_parts(category: str):
    return sorted(k for c, k in _PARTS if c == category)


def build_part(category: str, spec: PartSpec) -> Part:
    try:
        cls = _PARTS[(category, spec.kind)]
    except KeyError:
        raise RegistryError(f"unknown {category} {spec.kind!r}; known: {known_parts(category)}") from None
    return cls(prefix=spec.prefix, **spec.args)
