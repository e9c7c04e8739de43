"""Parts a model is assembled from.  Importing this package registers the built-in kinds."""
from .base import (PartSpec, ParamSpec, LayerSpec, RunEntry, ModelSpec, PagedKVNeed, FixedStateNeed,
                   PagedKVView, FixedStateView, StepContext, ResidualStream, Part, Norm, PositionEncoding,
                   Mixer, FeedForward, Embedding, Head, Block)
from . import norm, rope, attention, ffn, embedding, block  # noqa: F401  (registration)
