"""Causal attention over a paged key/value cache (multi-query, grouped or multi-head).

Order of the reference's serving path (serving/paged_mqa.py:64-113): project q, k, v;
rotate q and k at the tokens' positions; store rotated k and raw v into the pages
at ``table[pos // page] * page + pos % page``; attend over every key of the request
read back from the pages (new ones included) with scale ``1/sqrt(head_dim)`` and a
bottom-right aligned causal mask (kernels/pagedattn/pagedattn.cu:196-207,256);
project the concatenated heads with ``out``.  Query head ``h`` uses kv head
``h // (heads / kv_heads)`` (kernels/flashattn/flashattn.cu, same rule).

The three projections are fused at load into one matrix ``[(Hq+2*Hkv)*D, d]`` so one
product feeds the rotate-and-store kernel.  ``window`` (keys ``pos-window+1..pos``)
and ``page_size`` (a page size of this layer's own cache group) are parameters of the part; the reference's
model has neither.  A run entry that reads
another entry's cache (``shares_kv``) has no k/v projection and stores nothing.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, PartSpec, PagedKVNeed, PagedKVView, StepContext
from ..registry import register_part, build_part


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    def __init__(self, prefix: str, d_model: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, bias: bool = False, window: Optional[int] = None,
                 scale: Optional[float] = None, shares_kv: bool = False,
                 names: Optional[Dict[str, str]] = None, page_size: Optional[int] = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        self.d_model, self.num_heads, self.num_kv_heads, self.head_dim = d_model, num_heads, num_kv_heads, head_dim
        self.bias, self.window, self.shares_kv = bool(bias), window, bool(shares_kv)
        self.page_size = None if page_size is None else int(page_size)     # None: the engine's page size
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = build_part("position", position)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "out"}
        if names:
            self.names.update(names)
        self.w_in = self.b_in = self.w_out = self.b_out = None

    def children(self):
        return [self.position]

    # ---------------------------------------------------------------- tensors
    def param_specs(self):
        n, d, D = self.names, self.d_model, self.head_dim
        specs = {f"{n['q']}.weight": ParamSpec((self.num_heads * D, d)),
                 f"{n['o']}.weight": ParamSpec((d, self.num_heads * D))}
        if not self.shares_kv:
            specs[f"{n['k']}.weight"] = ParamSpec((self.num_kv_heads * D, d))
            specs[f"{n['v']}.weight"] = ParamSpec((self.num_kv_heads * D, d))
        if self.bias:
            for key in list(specs):
                w = specs[key]
                specs[key.replace(".weight", ".bias")] = ParamSpec((w.shape[0],), storage="matrix", init="normal")
        return specs

    def load(self, params):
        n = self.names
        keys = ["q"] if self.shares_kv else ["q", "k", "v"]
        self.w_in = torch.cat([params[f"{n[k]}.weight"] for k in keys], dim=0).contiguous()
        self.w_out = params[f"{n['o']}.weight"].contiguous()
        if self.bias:
            self.b_in = torch.cat([params[f"{n[k]}.bias"] for k in keys], dim=0).contiguous()
            self.b_out = params[f"{n['o']}.bias"].contiguous()

    def product_weights(self):
        return [self.w_in, self.w_out]

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_attention", None)
        if check is not None:
            check(dtype, self.num_heads, self.num_kv_heads, self.head_dim, self.page_size or page_size)

    # ---------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window, self.page_size)

    # ---------------------------------------------------------------- step
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        ops = self.ops
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        write = cache.writable and not self.shares_kv
        kv_heads_in_buf = 0 if self.shares_kv else Hkv
        qkv = ops.linear(x, self.w_in, self.b_in, partial_ok=True)   # [T, (Hq + 2*Hkv) * D], or partial sums of it
        T = qkv.shape[-2]
        table = self.position.rotary_table()
        if table is None:
            if qkv.dim() == 3:
                qkv = qkv.sum(0).to(x.dtype)
            q = qkv[:, :Hq * D].view(T, Hq, D)
            k = None if self.shares_kv else qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
            self.position.apply(q, k, ctx.positions)
            inv_freq, style = None, 0
            cs_table = None
        else:
            inv_freq, style = table
            cs_table = self.position.step_table(ctx) if inv_freq is not None else None
        q = qkv
        if qkv.dim() == 3:
            q = torch.empty((T, Hq * D), dtype=x.dtype, device=x.device)
        ops.rope_store(qkv, Hq, kv_heads_in_buf, D, ctx.positions, ctx.token_seq, inv_freq, style,
                       cache.k_pages, cache.v_pages, cache.block_table, cache.page_size, write,
                       q_out=q if qkv.dim() == 3 else None, cs_table=cs_table)
        out = torch.empty((T, Hq * D), dtype=x.dtype, device=x.device)
        # one launch per class of requests (decoded tokens; prompt portions), each planned as if it were alone
        classes = ctx.classes()
        if len(classes) == 1:
            c = classes[0]
            ops.paged_attention(q, Hq, Hkv, D, cache.k_pages, cache.v_pages, cache.block_table, cache.page_size,
                                c.query_start_loc, ctx.seq_lens, ctx.num_seqs, c.max_q_len, c.max_kv_len,
                                self.scale, self.window or 0, out)
        else:
            for ci, c in enumerate(classes):
                key = ("attention class views", id(cache.block_table), ci)    # the same for every layer of a cache group
                views = ctx.step_cache.get(key)
                if views is None:
                    views = ctx.step_cache[key] = (cache.block_table[c.seq_lo:c.seq_hi], ctx.seq_lens[c.seq_lo:c.seq_hi])
                ops.paged_attention(q[c.tok_lo:c.tok_hi], Hq, Hkv, D, cache.k_pages, cache.v_pages, views[0],
                                    cache.page_size, c.query_start_loc, views[1], c.seq_hi - c.seq_lo, c.max_q_len,
                                    c.max_kv_len, self.scale, self.window or 0, out[c.tok_lo:c.tok_hi])
        return ops.linear(out, self.w_out, self.b_out, partial_ok=True)
