"""Plain PyTorch stand-ins for the CUDA kernels, one function per kernel with the
kernel's own signature.  They serve two purposes in the tests: (1) each CUDA kernel is
compared with its stand-in at sizes other than the engine's; (2) handed to the engine as
``ops`` they let the cache manager, the batch packer, the step function and the scheduler
be tested on a machine without a GPU.  They are not a product path: the package loads
only the compiled sm_100a library and fails loudly without it.

Everything is computed in float32 (float64 where noted) and rounded to the output dtype
once, so the stand-ins are the "plain float32 reference of the same op".
"""
import math
import struct

import torch


def philox4x32(counter, key, rounds=10):
    """Philox-4x32-10 (Salmon et al. 2011), for checking the sampling kernel's draws."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c, k = list(counter), list(key)
    for _ in range(rounds):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + W0) & 0xFFFFFFFF, (k[1] + W1) & 0xFFFFFFFF]
    return c


def uniform_from_state(seed_lo, seed_hi, draws):
    """The uniform in [0, 1) the sampling kernel draws for (seed, draw counter)."""
    r = philox4x32([draws & 0xFFFFFFFF, 0, 0, 0], [seed_lo & 0xFFFFFFFF, seed_hi & 0xFFFFFFFF])
    return (r[0] >> 8) * (1.0 / 16777216.0)


class PlainOps:
    name = "plain"

    def embed(self, token_ids, table, out):
        out.copy_(table[token_ids.long()].float())

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        if delta is not None:
            resid.add_(delta.float())
        x = resid
        y = x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + eps) * weight.float()
        out.copy_(y.to(out.dtype))

    def rmsnorm_rows(self, resid, delta, rows, num_rows, weight, eps, out):
        x = resid[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
        y = x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + eps) * weight.float()
        out.copy_(y.to(out.dtype))

    def linear(self, x, w, bias, out_dtype=None, partial_ok=False):
        y = x.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        return y.to(out_dtype or x.dtype)

    def linear_swiglu(self, x, w_gu, b_gu, hidden):
        act = torch.empty((x.shape[0], hidden), dtype=x.dtype)
        self.swiglu(self.linear(x, w_gu, b_gu), act)
        return act

    def swiglu(self, gate_up, out):
        F = out.shape[1]
        g, u = gate_up[:, :F].float(), gate_up[:, F:].float()
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def rope_store(self, qkv, num_heads, num_kv_heads, head_dim, positions, token_seq, inv_freq, style,
                   k_pages, v_pages, block_table, page_size, write_kv, q_out=None, cs_table=None):
        T = qkv.shape[0]
        D = head_dim
        n_rot = num_heads + num_kv_heads
        x = qkv[:, :n_rot * D].float().view(T, n_rot, D)
        if inv_freq is not None:
            theta = positions.float()[:, None] * inv_freq.float()[None, :]
            c, s = theta.cos()[:, None, :], theta.sin()[:, None, :]
            y = torch.empty_like(x)
            if style == 0:
                xe, xo = x[..., 0::2], x[..., 1::2]
                y[..., 0::2] = xe * c - xo * s
                y[..., 1::2] = xe * s + xo * c
            else:
                h = D // 2
                y[..., :h] = x[..., :h] * c - x[..., h:] * s
                y[..., h:] = x[..., :h] * s + x[..., h:] * c
            qkv[:, :n_rot * D] = y.view(T, n_rot * D).to(qkv.dtype)
        if write_kv and num_kv_heads:
            pos = positions.long()
            page = block_table[token_seq.long(), pos // page_size].long()
            off = pos % page_size
            k = qkv[:, num_heads * D:(num_heads + num_kv_heads) * D].view(T, num_kv_heads, D)
            v = qkv[:, (num_heads + num_kv_heads) * D:(num_heads + 2 * num_kv_heads) * D].view(T, num_kv_heads, D)
            k_pages[page, :, off, :] = k
            v_pages[page, :, off, :] = v

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table, page_size,
                        query_start_loc, seq_lens, num_seqs, max_q_len, max_kv_len, scale, window, out):
        D, G = head_dim, num_heads // num_kv_heads
        qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
        for i in range(num_seqs):
            a, b, L = qsl[i], qsl[i + 1], sl[i]
            n = b - a
            if n == 0:
                continue
            q = qkv[a:b, :num_heads * D].float().view(n, num_heads, D)
            npages = -(-L // page_size)
            pages = block_table[i, :npages].long()
            k = k_pages[pages].float().permute(0, 2, 1, 3).reshape(npages * page_size, num_kv_heads, D)[:L]
            v = v_pages[pages].float().permute(0, 2, 1, 3).reshape(npages * page_size, num_kv_heads, D)[:L]
            qpos = torch.arange(L - n, L)[:, None]
            kpos = torch.arange(L)[None, :]
            vis = kpos <= qpos
            if window:
                vis = vis & (kpos > qpos - window)
            for h in range(num_heads):
                s = (q[:, h] @ k[:, h // G].T) * scale
                s = s.masked_fill(~vis.to(s.device), float("-inf"))
                out[a:b, h * D:(h + 1) * D] = (torch.softmax(s, dim=-1) @ v[:, h // G]).to(out.dtype)

    # the distribution after temperature / top-k / top-p, as the kernel defines it
    @staticmethod
    def filtered_probs(row, temperature, top_k, top_p):
        x = row.double() / temperature
        if top_k > 0:
            kth = torch.topk(x, min(top_k, x.numel())).values[-1]
            x = x.masked_fill(x < kth, float("-inf"))
        p = torch.softmax(x, dim=-1)
        if top_p < 1.0:
            # keep a token iff the mass of strictly larger values is <= top_p (ties stay together)
            sv, si = torch.sort(x, descending=True)
            sp = p[si]
            cum_before = torch.cumsum(sp, 0) - sp
            first_of_value = torch.ones_like(sv, dtype=torch.bool)
            first_of_value[1:] = sv[1:] != sv[:-1]
            idx = torch.arange(sv.numel())
            start = torch.cummax(torch.where(first_of_value, idx, torch.zeros_like(idx)), 0).values
            keep_sorted = cum_before[start] <= top_p
            keep = torch.zeros_like(keep_sorted)
            keep[si] = keep_sorted
            x = x.masked_fill(~keep, float("-inf"))
            p = torch.softmax(x, dim=-1)
        return p

    def sample(self, logits, slot_ids, state, out, probs_out=None):
        for r in range(logits.shape[0]):
            slot = int(slot_ids[r])
            seed_lo, seed_hi, draws, top_k, t_bits, p_bits, greedy, _ = [int(v) for v in state[slot].tolist()]
            row = logits[r].float().cpu()
            if greedy:
                out[r] = int(torch.argmax(row))
            else:
                temperature = struct.unpack("<f", struct.pack("<i", t_bits))[0]
                top_p = struct.unpack("<f", struct.pack("<i", p_bits))[0]
                p = self.filtered_probs(row, temperature, top_k, top_p)
                if probs_out is not None:
                    probs_out[r] = p.float()
                u = uniform_from_state(seed_lo, seed_hi, draws)
                cdf = torch.cumsum(p, 0)
                tok = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=cdf.dtype), right=True))
                tok = min(tok, int((p > 0).nonzero().max()))
                out[r] = tok
            state[slot, 2] = draws + 1
