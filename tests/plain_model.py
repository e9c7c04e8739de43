"""A plain, slow implementation of the architecture: whole sequences, no cache, one
function per part, float32 (or float64) on the CPU.  It is written from the
reference's formulas (each function cites file:line of the reference) and shares no
code with the engine; ``tests/golden/`` holds a one-time comparison of it with the
reference's own model classes on the CPU.

``cfg`` is a plain dict with the config.json keys; ``w`` maps the reference's
state-dict names to tensors.
"""
import math

import torch


def plain_embedding(w, tokens):
    """models/embedding.py:9-15 - row gather, no scale."""
    return w["embedding.embedding.weight"][torch.as_tensor(tokens, dtype=torch.long)]


def plain_rmsnorm(x, weight, eps):
    """models/rmsnorm.py:13-17 - x * rsqrt(mean(x^2) + eps) * w, eps inside the root."""
    return x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + eps) * weight


def plain_rope_tables(dim, positions, base, dtype=torch.float32):
    """models/rope.py:14-16 - inv_freq = 1/base^(2j/dim) and theta = pos*inv_freq, both in
    32-bit as the reference builds them; cos/sin then in ``dtype``."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
    freqs = torch.outer(torch.as_tensor(positions).float(), inv_freq)
    if dtype == torch.float64:
        freqs = freqs.double()
    return freqs.cos(), freqs.sin()


def plain_rope(x, cos, sin, style="interleaved"):
    """models/rope.py:21-35 - interleaved pairs (2j, 2j+1); x [S, H, D], cos/sin [S, D/2].
    style="half": pairs (j, j+D/2) as kernels/rope_kernel/rope_kernel.cu:133-157."""
    out = torch.empty_like(x)
    c, s = cos[:, None, :], sin[:, None, :]
    if style == "interleaved":
        xe, xo = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = xe * c - xo * s
        out[..., 1::2] = xe * s + xo * c
    else:
        h = x.shape[-1] // 2
        x1, x2 = x[..., :h], x[..., h:]
        out[..., :h] = x1 * c - x2 * s
        out[..., h:] = x1 * s + x2 * c
    return out


def plain_attention(q, k, v, scale, window=None):
    """Causal attention of one whole sequence: q [S, Hq, D], k, v [S, Hkv, D].
    Scores (q.k)*scale with scale 1/sqrt(D) (kernels/pagedattn/pagedattn.cu:930-931), key j
    visible to query i iff j <= i (pagedattn.cu:196-207,256 with ctx_len = 0), softmax in
    32-bit, query head h reads kv head h // (Hq/Hkv) (models/mqa.py:118 num_groups)."""
    S, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.empty_like(q)
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    for h in range(Hq):
        kh, vh = k[:, h // G, :], v[:, h // G, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ vh
    return out


def plain_linear(x, w, name):
    """nn.Linear: y = x @ W.T (+ b) (models/mqa.py:123-126, models/mlp.py:20-22)."""
    y = x @ w[f"{name}.weight"].T
    if f"{name}.bias" in w:
        y = y + w[f"{name}.bias"]
    return y


def plain_mqa(x, w, prefix, cfg, positions, window=None, style="interleaved"):
    """serving/paged_mqa.py:76-113 / models/mqa.py:228-294 for one whole sequence."""
    S = x.shape[0]
    Hq, Hkv = cfg["num_heads"], cfg.get("num_kv_heads", 1)
    D = cfg["d_model"] // Hq
    q = plain_linear(x, w, f"{prefix}.q_proj").view(S, Hq, D)
    k = plain_linear(x, w, f"{prefix}.k_proj").view(S, Hkv, D)
    v = plain_linear(x, w, f"{prefix}.v_proj").view(S, Hkv, D)
    cos, sin = plain_rope_tables(D, positions, cfg.get("rope_theta", 10000.0), x.dtype)
    q, k = plain_rope(q, cos.to(x.dtype), sin.to(x.dtype), style), plain_rope(k, cos.to(x.dtype), sin.to(x.dtype), style)
    o = plain_attention(q, k, v, 1.0 / math.sqrt(D), window)
    return plain_linear(o.reshape(S, Hq * D), w, f"{prefix}.out")


def plain_swiglu(x, w, prefix):
    """models/mlp.py:24-32 - down(silu(gate(x)) * up(x)), silu(g) = g*sigmoid(g)."""
    g = plain_linear(x, w, f"{prefix}.gate_proj")
    u = plain_linear(x, w, f"{prefix}.up_proj")
    return plain_linear(g * torch.sigmoid(g) * u, w, f"{prefix}.down_proj")


def plain_block(x, w, i, cfg, positions):
    """models/transformer_block.py:149-158 - pre-norm block with two residual sums."""
    eps = cfg.get("rms_norm_eps", 1e-5)
    p = f"layers.{i}"
    x = x + plain_mqa(plain_rmsnorm(x, w[f"{p}.attn_norm.weight"], eps), w, f"{p}.attn", cfg, positions)
    x = x + plain_swiglu(plain_rmsnorm(x, w[f"{p}.mlp_norm.weight"], eps), w, f"{p}.mlp")
    return x


def plain_forward(cfg, w, tokens, dtype=torch.float32):
    """models/transformer_block.py:172-182 - logits at every position of one sequence."""
    w = {k: v.to(dtype) for k, v in w.items()}
    x = plain_embedding(w, tokens)
    positions = torch.arange(len(tokens))
    for i in range(cfg["num_layers"]):
        x = plain_block(x, w, i, cfg, positions)
    x = plain_rmsnorm(x, w["final_norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    return x @ w["lm_head.weight"].T


# ------------------------------------------------------------------------- sampling
def plain_top_k(logits, k):
    """sampling.py:75-92 - keep everything >= the k-th largest value (ties stay)."""
    if k <= 0:
        return logits
    kth = torch.topk(logits, min(k, logits.shape[-1]), dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def plain_top_p(logits, p):
    """sampling.py:27-73 - sort descending, softmax, cumulative sum; drop where the sum
    *before* a token already exceeds p (the token that crosses p stays, the first always)."""
    if p >= 1.0:
        return logits
    sl, si = torch.sort(logits, descending=True, dim=-1)
    cum = torch.cumsum(torch.softmax(sl, dim=-1), dim=-1)
    remove = cum > p
    remove[..., 1:] = remove[..., :-1].clone()
    remove[..., 0] = False
    sl = sl.masked_fill(remove, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter_(-1, si, sl)


def plain_sample_probs(logits, temperature=1.0, top_k=0, top_p=1.0):
    """sampling.py:110-127 - the distribution the reference draws from."""
    x = logits.float() / temperature
    x = plain_top_k(x, top_k)
    x = plain_top_p(x, top_p)
    return torch.softmax(x, dim=-1)


def plain_greedy(logits):
    """sampling.py:5-6."""
    return torch.argmax(logits, dim=-1)
