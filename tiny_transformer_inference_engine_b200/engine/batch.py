"""Packs a step's entries into one int32 buffer and one host-to-device copy.

The reference builds ``input_ids / positions / query_start_loc / block_tables /
seq_lens`` as Python lists per step (serving/batch.py:18-36) and turns them into
tensors again inside every layer (serving/paged_mqa.py:80,87-96;
serving/fake_paged_attn.py:52-100).  Here they are laid out once in pinned host
memory, copied once, and every kernel of the step reads views of that buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import SeqClass, StepContext


@dataclass
class StepEntry:
    """A request's next tokens: ``tokens`` sit at positions ``start .. start+len-1``;
    ``want`` lists indices into ``tokens`` whose logits are asked for."""
    rid: Hashable
    start: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


def _round4(n: int) -> int:
    return (n + 3) & ~3


class BatchPacker:
    def __init__(self, manager, ops, dtype: torch.dtype, device, vocab_size: int, max_seq_len: int, split_classes: bool = True):
        self.manager, self.ops, self.dtype = manager, ops, dtype
        self.split_classes = bool(split_classes)       # False: a mixed step is one class (every request in the portions' launch)
        self.device = torch.device(device)
        self.vocab_size, self.max_seq_len = vocab_size, max_seq_len
        self._host = None
        self._dev = None
        self._cap = 0
        self._copied = None            # event: the last host-to-device copy has read the host buffer
        self._last = None              # layout of the last fixed-layout decode step (see _repack_decode)

    def _ensure(self, n: int):
        if n > self._cap:
            cap = max(1024, 1 << (n - 1).bit_length())
            pin = self.device.type == "cuda"
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=pin)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._cap = cap

    def validate(self, entries: List[StepEntry]) -> None:
        """Host-side checks of everything a kernel will index with (cf. serving/kv_pool.py:41-53,
        serving/fake_paged_attn.py:61-92, kernels/pagedattn/pagedattn.cu:867-895)."""
        seen = set()
        for en in entries:
            if en.rid in seen:
                raise ValueError(f"request {en.rid!r} appears twice in one step")
            seen.add(en.rid)
            n = len(en.tokens)
            if n < 1:
                raise ValueError(f"request {en.rid!r} brings no tokens")
            if en.start < 0 or en.start + n > self.max_seq_len:
                raise ValueError(f"request {en.rid!r}: positions {en.start}..{en.start + n - 1} exceed "
                                 f"max_seq_len={self.max_seq_len}")
            if min(en.tokens) < 0 or max(en.tokens) >= self.vocab_size:
                bad = [t for t in en.tokens if not 0 <= int(t) < self.vocab_size]
                raise ValueError(f"request {en.rid!r}: token id {bad[0]} outside [0, {self.vocab_size})")
            if en.want and (min(en.want) < 0 or max(en.want) >= n):
                bad = [w for w in en.want if not 0 <= int(w) < n]
                raise ValueError(f"request {en.rid!r}: wanted place {bad[0]} outside its {n} tokens")
            for gi, g in enumerate(self.manager.groups):
                table = g.tables.get(en.rid)
                if table is None:
                    raise KeyError(f"request {en.rid!r} is not admitted")
                first = g.first_needed_page(en.start)
                last = -(-(en.start + n) // g.page_size)
                span = table[first:last]
                if len(table) < last or (span and (min(span) <= 0 or max(span) >= g.num_pages)):
                    raise ValueError(f"request {en.rid!r}: block table of group {gi} does not cover "
                                     f"positions {en.start}..{en.start + n - 1}")

    def _repack_decode(self, entries: List[StepEntry], key) -> bool:
        """A decode step of the same requests in the same order and layout as the last packed one: only the
        tokens, positions, lengths and newly appended pages are written into the host buffer (which still holds
        the rest), with the checks of ``validate`` on what changes.  False: not that case, pack in full."""
        st = self._last
        if st is None or st["key"] != key:
            return False
        mgr, hn = self.manager, st["hn"]
        if self._copied is not None:
            self._copied.synchronize()
        o_tok, o_pos, o_seql = st["o_tok"], st["o_pos"], st["o_seql"]
        for i, en in enumerate(entries):
            tok, start = int(en.tokens[0]), en.start
            if not 0 <= tok < self.vocab_size:
                raise ValueError(f"request {en.rid!r}: token id {tok} outside [0, {self.vocab_size})")
            if start < 0 or start >= self.max_seq_len:
                raise ValueError(f"request {en.rid!r}: positions {start}..{start} exceed max_seq_len={self.max_seq_len}")
            hn[o_tok + i] = tok
            hn[o_pos + i] = start
            hn[o_seql + i] = start + 1
            for gi, g in enumerate(mgr.groups):
                table = g.tables.get(en.rid)
                if table is None:
                    raise KeyError(f"request {en.rid!r} is not admitted")
                have = st["tlen"][gi][i]
                if len(table) * g.page_size <= start or len(table) < have or len(table) > st["widths"][gi]:
                    raise ValueError(f"request {en.rid!r}: block table of group {gi} does not cover positions {start}..{start}")
                if len(table) != have:
                    new = table[have:]
                    if min(new) <= 0 or max(new) >= g.num_pages:
                        raise ValueError(f"request {en.rid!r}: block table of group {gi} does not cover positions {start}..{start}")
                    off = st["o_tab"][gi] + i * st["widths"][gi]
                    hn[off + have:off + len(table)] = new
                    st["tlen"][gi][i] = len(table)
        total = st["total"]
        st["dev"][:total].copy_(st["host"][:total], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        return True

    def feed_tokens(self, tokens: torch.Tensor) -> None:
        """Overwrites the token ids of the fixed-layout decode step packed last with ``tokens`` (int32, on the
        device, one per request in the step's order): the step then runs on tokens the host has not seen yet.
        Ordered on the stream after the step's host-to-device copy."""
        st = self._last
        if st is None:
            raise RuntimeError("no fixed-layout decode step is packed")
        st["dev"][st["o_tok"]:st["o_tok"] + tokens.shape[0]].copy_(tokens)

    def pack(self, entries: List[StepEntry], pad_seqs: int = 0, pages_per_seq: Optional[Dict[int, int]] = None,
             buffers=None, copy_only: bool = False) -> Optional[StepContext]:
        """``pad_seqs``/``pages_per_seq``/``buffers`` give a fixed layout (for a captured
        graph): the batch is padded to ``pad_seqs`` one-token requests that sit on the
        scratch page with length 1, and the tables get ``pages_per_seq[group]`` columns.
        ``copy_only``: fill and copy the buffer but build no context (a graph replay needs none)."""
        key = None
        if buffers is not None and all(len(e.tokens) == 1 and len(e.want) == 1 and e.want[0] == 0 for e in entries):
            # a decode step in a fixed layout: its layout is remembered (tokens may be fed into it on the device), and
            # where no group has a window - a window moves table entries that the short path does not look at - the
            # next step of the same requests rewrites only what changed
            key = (tuple(e.rid for e in entries), pad_seqs, tuple(sorted(pages_per_seq.items())), buffers[0].data_ptr())
            if copy_only and all(g.window is None for g in self.manager.groups) and self._repack_decode(entries, key):
                return None
        self._last = None
        self.validate(entries)
        mgr = self.manager
        N_real = len(entries)
        N = max(N_real, pad_seqs)
        # requests that bring one token are packed first: the two classes of a mixed step (decoded tokens, prompt
        # portions) are then contiguous ranges of requests and of tokens, and a mixer can run each with the kernel
        # that suits it.  Wanted rows keep the order of the entries as given.
        order = sorted(range(N_real), key=lambda i: len(entries[i].tokens) != 1)
        num_single = sum(1 for en in entries if len(en.tokens) == 1)
        tok, pos, tseq, qsl, seql, slots = [], [], [], [0], [], []
        base_of = [0] * N_real
        for i, src in enumerate(order):
            en = entries[src]
            n = len(en.tokens)
            base_of[src] = qsl[-1]
            tok.extend(int(t) for t in en.tokens)
            pos.extend(range(en.start, en.start + n))
            tseq.extend([i] * n)
            qsl.append(qsl[-1] + n)
            seql.append(en.start + n)
            slots.append(mgr.slot_of[en.rid])
        rows = [base_of[i] + int(w) for i, en in enumerate(entries) for w in en.want]
        for i in range(N_real, N):
            tok.append(0); pos.append(0); tseq.append(i); rows.append(qsl[-1]); qsl.append(qsl[-1] + 1); seql.append(1); slots.append(-1)
        q_lens = [qsl[i + 1] - qsl[i] for i in range(N)]
        T = qsl[-1]
        # a mixed step: the second class's query_start_loc counted from its own first token
        mixed = self.split_classes and 0 < num_single < N_real
        qsl_tail = [q - num_single for q in qsl[num_single:]] if mixed else []
        R = len(rows)
        tables, widths = [], []
        for gi, g in enumerate(mgr.groups):
            width = max([len(g.tables[e.rid]) for e in entries] + [1])
            if pages_per_seq is not None:
                if width > pages_per_seq[gi]:
                    raise ValueError("block table wider than the fixed layout")
                width = pages_per_seq[gi]
            tables.append([g.tables[entries[src].rid] for src in order])
            widths.append(width)

        sizes = [T, T, T, N + 1, N, N, max(R, 1), len(qsl_tail)] + [N * w for w in widths]
        offs, total = [], 0
        for s in sizes:
            offs.append(total)
            total += _round4(s)
        if buffers is None:
            self._ensure(total)
            host, dev = self._host, self._dev
        else:
            host, dev = buffers
            if total > host.numel():
                raise ValueError("step does not fit the fixed buffers")
        if self._copied is not None:
            self._copied.synchronize()
        hn = host.numpy()
        for off, data in zip(offs[:8], (tok, pos, tseq, qsl, seql, slots, rows, qsl_tail)):
            hn[off:off + len(data)] = data
        for off, rows_, w in zip(offs[8:], tables, widths):
            block = hn[off:off + N * w].reshape(N, w)
            block[:] = 0
            for i, t in enumerate(rows_):
                block[i, :len(t)] = t
        dev[:total].copy_(host[:total], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()
        if key is not None:
            self._last = {"key": key, "hn": hn, "host": host, "dev": dev, "total": total, "o_tok": offs[0], "o_pos": offs[1],
                          "o_seql": offs[4], "o_tab": offs[8:], "widths": widths,
                          "tlen": [[len(t) for t in rows_] for rows_ in tables]}
        if copy_only:
            return None

        def view(k, n):
            return dev[offs[k]:offs[k] + n]

        ctx = StepContext(
            ops=self.ops, dtype=self.dtype, device=self.device,
            num_tokens=T, num_seqs=N, max_q_len=max(q_lens), max_kv_len=max(seql),
            token_ids=view(0, T), positions=view(1, T), token_seq=view(2, T),
            query_start_loc=view(3, N + 1), seq_lens=view(4, N), slot_ids=view(5, N),
            logit_rows=view(6, R), num_logit_rows=R,
            block_tables={gi: dev[offs[8 + gi]:offs[8 + gi] + N * w].view(N, w) for gi, w in enumerate(widths)},
            host={"q_lens": q_lens, "seq_lens": seql, "query_start_loc": qsl, "positions": pos,
                  "num_real_seqs": N_real},
        )
        if mixed:
            ns = num_single
            ctx.seq_classes = [
                SeqClass(0, ns, 0, ns, 1, max(seql[:ns]), view(3, ns + 1)),
                SeqClass(ns, N, ns, T, max(q_lens[ns:]), max(seql[ns:]), view(7, N - ns + 1)),
            ]
        return ctx
