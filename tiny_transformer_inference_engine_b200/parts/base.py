"""Interfaces of the parts a model is put together from.

A model is data: a ``ModelSpec`` lists layers, each layer names a mixer, a
feed-forward and two norms by ``PartSpec`` (registry kind + constants), and
``run_order`` lists which layer runs when and whose cache it uses.  No part
knows which model it sits in; a part sees only its own constants, its own
weights (by names relative to its prefix), the step's metadata and the cache
view the cache manager made for it.

Categories and the methods each must have:

``norm``      ``add_norm(resid, delta) -> x``; ``norm_rows(resid, delta, rows) -> x``
``position``  ``rotary_table() -> (inv_freq, style) | None``; ``apply(q, k, positions)``
``mixer``     ``cache_need()`` (or ``cache_needs()`` for several); ``forward(x, ctx, cache) -> y``
``ffn``       ``forward(x, ctx) -> y``
``embedding`` ``forward(ctx) -> resid``
``head``      ``forward(x) -> logits``
``block``     ``cache_needs()``; ``forward(stream, ctx, caches)`` (arrangement of the four above)

Every part may also say ``capturable = False`` (its step reads device values on the host, so it
cannot run inside a captured CUDA graph: a model with such a part steps without graphs) or
``capturable = "decode"`` (only its steps of single tokens can be captured) and
override ``validate(ops, dtype, page_size)`` to refuse, when the engine is built, sizes that
its kernels do not take.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- specs
@dataclass(frozen=True)
class PartSpec:
    """Registry kind of a part, the prefix of its tensor names, and its sizes and constants."""
    kind: str
    prefix: str = ""
    args: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ParamSpec:
    """Shape and storage class of one tensor of a part.

    ``matrix`` tensors are cast to the compute dtype.  ``vector`` tensors that the
    file stores in 32-bit stay 32-bit (their kernels read either width); stored in
    16-bit they are widened only for a float32 run.  ``table`` tensors are integer
    tables and are kept as int32.
    """
    shape: Tuple[int, ...]
    storage: str = "matrix"            # "matrix" | "vector" | "table"
    init: str = "normal"               # random-weights mode: "normal" | "ones" | "zeros"; tables: "randint" | "arange" | "zeros"
    high: Optional[int] = None         # "randint": values are uniform in [0, high)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                    # arrangement; its args hold the four part specs


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.  ``cache_from`` names an earlier run entry whose cache this
    run reads instead of owning one (it then writes nothing into it)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    d_model: int
    vocab_size: int
    max_seq_len: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: Optional[int] = None


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every past token (or of the last ``window`` tokens) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None       # None: all keys
    page_size: Optional[int] = None    # None: the engine's page size


@dataclass(frozen=True)
class FixedStateNeed:
    """Per-request state of fixed size, one row per state slot."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class PagedKVView:
    k_pages: torch.Tensor              # [pages, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor          # int32 [num_seqs, max_pages_per_seq] for this step
    page_size: int
    writable: bool = True


@dataclass
class FixedStateView:
    state: torch.Tensor                # [state_slots + 1, *shape]; row = ctx.slot_ids[seq]; the last row is scratch (slot id -1)
    writable: bool = True


# --------------------------------------------------------------------------- step metadata
@dataclass
class SeqClass:
    """A contiguous range of a step's requests (and of their tokens) that bring alike numbers of tokens.

    A step that mixes decoded tokens with prompt portions is packed with the one-token requests first, and
    carries two classes; a mixer may run each class with the kernel that suits it (a decode step's form for
    the first, a prompt portion's for the second) instead of sizing one launch for the longest portion.
    ``query_start_loc`` counts from the class's first token, so the class reads like a step of its own:
    tokens ``tok_lo:tok_hi``, requests ``seq_lo:seq_hi`` of the step's per-request arrays."""
    seq_lo: int
    seq_hi: int
    tok_lo: int
    tok_hi: int
    max_q_len: int
    max_kv_len: int
    query_start_loc: torch.Tensor      # int32 [seq_hi - seq_lo + 1]


@dataclass
class StepContext:
    """What one step brings: the packed tokens and where each sits.

    All device tensors are int32 and live in one buffer that one host-to-device
    copy filled.  ``T`` tokens of ``N`` requests; request ``i`` owns tokens
    ``query_start_loc[i]:query_start_loc[i+1]`` at positions
    ``seq_lens[i]-q_len_i .. seq_lens[i]-1``.
    """
    ops: Any
    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    max_q_len: int
    max_kv_len: int
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T]
    token_seq: torch.Tensor            # [T] index of the token's request in this step
    query_start_loc: torch.Tensor      # [N+1]
    seq_lens: torch.Tensor             # [N] keys visible to the request's last token (cache length after the step)
    slot_ids: torch.Tensor             # [N] state slot of each request; -1 for the padding rows of a fixed-size (captured) batch
    logit_rows: torch.Tensor           # [R] flat token indices whose logits are wanted
    num_logit_rows: int
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # cache group -> [N, max_pages]
    host: Dict[str, Any] = field(default_factory=dict)                    # the same numbers as Python lists
    step_cache: Dict[Any, Any] = field(default_factory=dict)              # device values parts compute once per step
    seq_classes: Optional[List[SeqClass]] = None                          # None: one class, the whole step

    def classes(self) -> List[SeqClass]:
        """The step's request classes; a step without a division is one class."""
        if self.seq_classes:
            return self.seq_classes
        return [SeqClass(0, self.num_seqs, 0, self.num_tokens, self.max_q_len, self.max_kv_len, self.query_start_loc)]


class ResidualStream:
    """The residual sum in 32-bit plus the last sub-layer's output not yet added to it.

    Norm parts add ``delta`` into ``resid`` in the same kernel that normalises, so the
    sum is formed and kept in 32-bit whatever the compute dtype is.
    """
    __slots__ = ("resid", "delta")

    def __init__(self, resid: torch.Tensor, delta: Optional[torch.Tensor] = None):
        self.resid = resid
        self.delta = delta


# --------------------------------------------------------------------------- base classes
class Part:
    """Base of every part: constants in, tensor specs out, tensors loaded by relative name."""
    category = "part"
    capturable = True                  # True: any step; "decode": only steps of single tokens; False: none can be captured in a CUDA graph

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.ops = None
        self.dtype = None
        self.device = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def children(self) -> List["Part"]:
        return []

    def load(self, params: Dict[str, torch.Tensor]) -> None:
        """Receives this part's tensors (relative names), already on the device and in
        the storage class its ParamSpec asked for."""

    def bind(self, ops, dtype: torch.dtype, device: torch.device) -> None:
        self.ops, self.dtype, self.device = ops, dtype, device
        for c in self.children():
            c.bind(ops, dtype, device)

    def product_weights(self) -> List[torch.Tensor]:
        """The matrices this part multiplies activations by (after ``load``), for kernel libraries that choose an
        implementation per matrix shape by measuring."""
        return []

    def validate(self, ops, dtype: torch.dtype, page_size: int) -> None:
        """Raises if the part's sizes, the compute dtype or the page size are something its kernels do not take.
        Called when the engine is built, before weights are read or a pool is allocated."""


class Norm(Part):
    category = "norm"

    def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def norm_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                  num_rows: int) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def rotary_table(self):
        """(inv_freq float32 [rotary_dim/2], style) if the encoding is a rotation of pairs
        by ``pos * inv_freq`` that the fused rotate-and-store kernel can do, else None."""
        return None

    def step_table(self, ctx):
        """Optional: sines and cosines of the step's positions (float32 [T, D/2, 2]), computed once
        per step, for encodings whose rotary_table() is not None."""
        return None

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        """General path, in place: q [T, heads, D], k [T, kv_heads, D] (views)."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_need(self):
        """The one thing this mixer keeps between steps (``PagedKVNeed``, ``FixedStateNeed``) or None; ``forward``
        then receives the one view made for it (or None)."""
        return None

    def cache_needs(self) -> List[object]:
        """For a mixer that keeps several things (say pages and a state of fixed size): the list of its needs;
        ``forward`` then receives the list of views in the same order.  The default wraps ``cache_need()``."""
        need = self.cache_need()
        return [] if need is None else [need]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    category = "ffn"

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    category = "block"

    def cache_needs(self) -> List[object]:
        """Everything the block's sub-parts keep between steps, as one list; ``forward`` receives as many views, in
        this order, and hands each sub-part its own."""
        return []

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: List[object]) -> None:
        raise NotImplementedError


def mixer_cache_argument(mixer: Mixer, views: List[object]):
    """What a mixer's ``forward`` gets as ``cache`` out of the views made for its needs: the list itself if the
    mixer declares ``cache_needs()`` of its own, else the single view (None if it keeps nothing)."""
    if type(mixer).cache_needs is not Mixer.cache_needs:
        return list(views)
    return views[0] if views else None
