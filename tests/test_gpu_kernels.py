"""Each kernel alone against its plain float32 stand-in, at sizes other than the engine's:
widths and vocabularies that are no power of two, 3 / 5 / 71 heads, head sizes in steps of 16,
page sizes 1..64, pools filled with garbage and shuffled block tables so that a stray read
shows, and inputs made so that one far key, a window's edge or a page's edge decides the result."""
import math
import random
import struct

import pytest
import torch

from plain_ops import PlainOps, uniform_from_state

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PLAIN = PlainOps()


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()


DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 1.2e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,d,V", [(1, 64, 100), (37, 1000, 515), (5, 4544, 77)])
def test_embed(ops, dtype, T, d, V):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, d, generator=g).to(DT[dtype])
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    ids[0] = V - 1
    out = torch.empty(T, d, dtype=torch.float32, device=DEV)
    ops.embed(ids.to(DEV), table.to(DEV), out)
    exp = torch.empty(T, d)
    PLAIN.embed(ids, table, exp)
    assert torch.equal(out.cpu(), exp)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,d,eps", [(1, 64, 1e-5), (19, 1000, 1e-6), (3, 4544, 1e-3), (2, 11008, 1e-5), (64, 4096, 1e-5), (97, 2048, 1e-5)])
def test_add_rmsnorm(ops, dtype, wdtype, T, d, eps):
    g = torch.Generator().manual_seed(1)
    resid = torch.randn(T, d, generator=g) * 3
    delta = (torch.randn(T, d, generator=g)).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(DT[wdtype])
    for dl in (delta, None):
        r_gpu, out = resid.clone().to(DEV), torch.empty(T, d, dtype=DT[dtype], device=DEV)
        ops.add_rmsnorm(r_gpu, None if dl is None else dl.to(DEV), w.to(DEV), eps, out)
        r_cpu, exp = resid.clone(), torch.empty(T, d, dtype=DT[dtype])
        PLAIN.add_rmsnorm(r_cpu, dl, w, eps, exp)
        assert rel(r_gpu.cpu(), r_cpu) < 1e-6                   # the 32-bit residual sum itself
        assert rel(out.float().cpu(), exp.float()) < (1e-5 if dtype == "float32" else 8e-3)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    out = torch.empty(2, d, dtype=DT[dtype], device=DEV)
    r_gpu = resid.clone().to(DEV)
    ops.rmsnorm_rows(r_gpu, delta.to(DEV), rows.to(DEV), 2, w.to(DEV), eps, out)
    exp = torch.empty(2, d, dtype=DT[dtype])
    PLAIN.rmsnorm_rows(resid, delta, rows, 2, w, eps, exp)
    assert torch.equal(r_gpu.cpu(), resid)                        # gathering leaves the stream untouched
    assert rel(out.float().cpu(), exp.float()) < (1e-5 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("M,N,K,bias", [(1, 7, 5, False), (33, 515, 96, True), (130, 64, 1000, False), (5, 200, 4544, True),
                                        (16, 515, 96, True), (2, 50257, 512, False), (9, 33, 1000, True), (1, 3, 4, False), (17, 40, 64, False),
                                        (32, 130, 512, True), (33, 130, 512, True)])
def test_gemm_f32_is_true_32_bit(ops, M, N, K, bias):
    """Both forms of the float32 product: up to 32 rows with aligned operands stream the weights (a warp per four weight
    rows; 17 to 32 rows in two launches), everything else takes the 64 x 64 tile - including the strided, misaligned
    view below."""
    g = torch.Generator().manual_seed(2)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    b = torch.randn(N, generator=g) if bias else None
    out = ops.linear(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV))
    exp = x.double() @ w.double().T + (b.double() if bias else 0)
    # TF32 would leave ~1e-3; FFMA with 32-bit accumulation leaves ~1e-6
    assert rel(out.cpu(), exp) < 3e-6
    # a strided input (a column slice) works too
    big = torch.randn(M, K + 8, generator=g).to(DEV)
    out2 = ops.linear(big[:, 3:3 + K], w.to(DEV), None)
    assert rel(out2.cpu(), big[:, 3:3 + K].cpu().double() @ w.double().T) < 3e-6


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 4352, 4096), (300, 352, 176)])
def test_linear_bf16(ops, M, N, K):
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    b = torch.randn(N, generator=g).bfloat16()
    exp = x.double() @ w.double().T
    assert rel(ops.linear(x.to(DEV), w.to(DEV), None).float().cpu(), exp) < 8e-3
    assert rel(ops.linear(x.to(DEV), w.to(DEV), b.to(DEV)).float().cpu(), exp + b.double()) < 8e-3
    out32 = ops.linear(x.to(DEV), w.to(DEV), None, out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and rel(out32.cpu(), exp) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,F", [(1, 176), (9, 1000), (4, 11008)])
def test_swiglu(ops, dtype, T, F):
    g = torch.Generator().manual_seed(4)
    gu = (torch.randn(T, 2 * F, generator=g) * 4).to(DT[dtype])
    gu[0, 0], gu[0, 1] = -80.0, 80.0
    out = torch.empty(T, F, dtype=DT[dtype], device=DEV)
    ops.swiglu(gu.to(DEV), out)
    exp = torch.empty(T, F, dtype=DT[dtype])
    PLAIN.swiglu(gu, exp)
    assert torch.isfinite(out).all()
    assert rel(out.float().cpu(), exp.float()) < (2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,D,page,style,base", [(4, 1, 16, 16, 0, 1e4), (3, 1, 32, 8, 0, 5e5), (71, 1, 64, 64, 0, 1e4),
                                                      (6, 2, 48, 5, 1, 2e4), (8, 8, 128, 1, 0, 1e4)])
def test_rope_store(ops, dtype, Hq, Hkv, D, page, style, base):
    g = torch.Generator().manual_seed(5)
    lens = [(0, 7), (30, 1), (4090, 3)]                           # (start, new tokens): far positions too
    T = sum(n for _, n in lens)
    positions = torch.tensor([s + i for s, n in lens for i in range(n)], dtype=torch.int32)
    token_seq = torch.tensor([i for i, (_, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    width = max(-(-(s + n) // page) for s, n in lens)
    nb = 3 * width + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    table = perm[:3 * width].view(3, width).to(torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(DT[dtype])
    inv_freq = 1.0 / (base ** (torch.arange(0, D, 2).float() / D))
    kp = torch.full((nb, Hkv, page, D), 777.0).to(DT[dtype])
    vp = kp.clone()
    qkv0, kp0, vp0 = qkv.clone(), kp.clone(), vp.clone()
    q_gpu, kp_gpu, vp_gpu = qkv.clone().to(DEV), kp.clone().to(DEV), vp.clone().to(DEV)
    ops.rope_store(q_gpu, Hq, Hkv, D, positions.to(DEV), token_seq.to(DEV), inv_freq.to(DEV), style, kp_gpu, vp_gpu,
                   table.to(DEV), page, True)
    PLAIN.rope_store(qkv, Hq, Hkv, D, positions, token_seq, inv_freq, style, kp, vp, table, page, True)
    tol = 3e-6 if dtype == "float32" else 8e-3
    assert rel(q_gpu.float().cpu(), qkv.float()) < tol
    assert rel(kp_gpu.float().cpu(), kp.float()) < tol and rel(vp_gpu.float().cpu(), vp.float()) < tol
    assert torch.equal(kp_gpu.cpu()[0], kp[0])                    # the scratch page is untouched
    untouched = (kp == 777.0)
    assert torch.equal(kp_gpu.cpu()[untouched], kp[untouched])    # nothing else was written
    if style == 0 and D % 4 == 0:
        # the vectorised kernel with the step's cos/sin table gives the same
        cs = ops.rope_table(positions.to(DEV), inv_freq.to(DEV))
        theta = positions.float()[:, None] * inv_freq[None, :]
        assert rel(cs.cpu()[..., 0], theta.cos()) < 1e-6 and rel(cs.cpu()[..., 1], theta.sin()) < 1e-6
        q3, kp3, vp3 = qkv0.clone().to(DEV), kp0.clone().to(DEV), vp0.clone().to(DEV)
        ops.rope_store(q3, Hq, Hkv, D, positions.to(DEV), token_seq.to(DEV), inv_freq.to(DEV), 0, kp3, vp3, table.to(DEV),
                       page, True, cs_table=cs)
        assert rel(q3.float().cpu(), qkv.float()) < tol
        assert rel(kp3.float().cpu(), kp.float()) < tol and rel(vp3.float().cpu(), vp.float()) < tol
        assert torch.equal(kp3.cpu()[untouched], kp[untouched])
    # no rotation, no store
    q2 = qkv.clone().to(DEV)
    ops.rope_store(q2, Hq, Hkv, D, positions.to(DEV), token_seq.to(DEV), None, 0, kp_gpu, vp_gpu, table.to(DEV), page, False)
    assert torch.equal(q2.cpu(), qkv)


# ------------------------------------------------------------------------------------------ attention
def attention_case(ops, dtype, Hq, Hkv, D, page, seqs, window=0, plan=None, seed=0, spike=None, split_at=None, plans_seen=None):
    """seqs: list of (kv_len, q_len).  spike=(seq, query index, key position): that query and that
    key are made parallel and large so the key decides the row's output.  split_at: the first
    ``split_at`` requests and the others run as two launches over views of the same step, as the
    attention part runs the two classes of a mixed step."""
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    N = len(seqs)
    T = sum(q for _, q in seqs)
    width = max(-(-L // page) for L, _ in seqs) + 1
    nb = sum(-(-L // page) for L, _ in seqs) + 1
    order = (torch.randperm(nb - 1, generator=g) + 1).tolist()
    kp = torch.full((nb, Hkv, page, D), 1000.0).to(dt)            # garbage everywhere first
    vp = torch.full((nb, Hkv, page, D), -1000.0).to(dt)
    table = torch.zeros(N, width, dtype=torch.int32)
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, generator=g) * 0.7).to(dt)
    dense, qsl = [], [0]
    for i, (L, n) in enumerate(seqs):
        k = (torch.randn(L, Hkv, D, generator=g) * 0.7).to(dt)
        v = torch.randn(L, Hkv, D, generator=g).to(dt)
        if spike is not None and spike[0] == i:
            _, qi, kpos = spike
            u = torch.randn(D, generator=g)
            u = u / u.norm()
            qkv[qsl[-1] + qi, :Hq * D] = (u * 14.0).repeat(Hq).to(dt)
            k[kpos, :, :] = (u * 14.0).to(dt)
        for pg in range(-(-L // page)):
            phys = order.pop()
            table[i, pg] = phys
            lo, hi = pg * page, min(L, (pg + 1) * page)
            kp[phys, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            vp[phys, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        dense.append((k.float(), v.float()))
        qsl.append(qsl[-1] + n)
    seq_lens = torch.tensor([L for L, _ in seqs], dtype=torch.int32)
    qsl_t = torch.tensor(qsl, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    out = torch.full((T, Hq * D), 5.0, dtype=dt, device=DEV)
    max_q, max_kv = max(n for _, n in seqs), max(L for L, _ in seqs)
    if split_at is None:
        ops.paged_attention(qkv.to(DEV), Hq, Hkv, D, kp.to(DEV), vp.to(DEV), table.to(DEV), page, qsl_t.to(DEV),
                            seq_lens.to(DEV), N, max_q, max_kv, scale, window, out, plan=plan)
    else:
        q_d, kp_d, vp_d, table_d, lens_d = qkv.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV), seq_lens.to(DEV)
        for lo, hi in ((0, split_at), (split_at, N)):
            t0, t1 = qsl[lo], qsl[hi]
            mq, mk = max(n for _, n in seqs[lo:hi]), max(L for L, _ in seqs[lo:hi])
            if plans_seen is not None:
                plans_seen.append(ops.attention_plan(dt, hi - lo, Hq, Hkv, D, mq, mk, page))
            ops.paged_attention(q_d[t0:t1], Hq, Hkv, D, kp_d, vp_d, table_d[lo:hi], page, (qsl_t[lo:hi + 1] - t0).to(DEV),
                                lens_d[lo:hi], hi - lo, mq, mk, scale, window, out[t0:t1], plan=plan)
    exp = torch.empty(T, Hq * D)
    G = Hq // Hkv
    for i, (L, n) in enumerate(seqs):
        k, v = dense[i]
        q = qkv[qsl[i]:qsl[i + 1], :Hq * D].float().view(n, Hq, D)
        qpos, kpos = torch.arange(L - n, L)[:, None], torch.arange(L)[None, :]
        vis = kpos <= qpos
        if window:
            vis = vis & (kpos > qpos - window)
        for h in range(Hq):
            s = (q[:, h] @ k[:, h // G].T) * scale
            p = torch.softmax(s.masked_fill(~vis, float("-inf")), -1)
            exp[qsl[i]:qsl[i + 1], h * D:(h + 1) * D] = p @ v[:, h // G]
    return out.float().cpu(), exp, dense, qsl


SCENARIOS = {                                                     # like tests/test.py:33-38 of the reference
    "prefill": [(33, 33), (1, 1), (130, 130)],
    "decode": [(200, 1), (64, 1), (65, 1), (1, 1), (513, 1)],
    "chunked": [(100, 7), (64, 2), (130, 66), (300, 129)],
    "mixed": [(77, 77), (300, 1), (129, 2), (64, 64), (1000, 1)],
}
SHAPES = [(4, 1, 16, 16), (3, 1, 32, 8), (6, 2, 48, 32), (71, 1, 64, 64), (32, 1, 128, 64), (5, 5, 80, 3), (8, 1, 256, 16),
          (2, 2, 20, 7)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scenario", list(SCENARIOS))
@pytest.mark.parametrize("Hq,Hkv,D,page", SHAPES)
def test_paged_attention(ops, dtype, scenario, Hq, Hkv, D, page):
    out, exp, _, _ = attention_case(ops, dtype, Hq, Hkv, D, page, SCENARIOS[scenario])
    assert torch.isfinite(out).all()
    assert rel(out, exp) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,D,page", [(32, 1, 128, 64), (71, 1, 64, 16), (8, 1, 256, 16), (6, 2, 48, 8)])
def test_mixed_step_in_two_classes(ops, dtype, Hq, Hkv, D, page):
    """Decoded tokens with long contexts beside prompt portions, as two launches over one step's buffers:
    each class is planned as if it were alone, and every row equals the float32 reference."""
    seqs = [(4096, 1), (3000, 1), (65, 1), (512, 512), (2600, 512), (130, 2)]
    plans = []
    out, exp, _, _ = attention_case(ops, dtype, Hq, Hkv, D, page, seqs, split_at=3, plans_seen=plans)
    assert torch.isfinite(out).all()
    assert rel(out, exp) < TOL[dtype]
    if dtype == "bfloat16" and D in (64, 128):
        assert plans[0][0] in ("tc", "mma", "mma_c4") and plans[0][1] > 1       # one-token requests: their key range is cut
        assert plans[1][0] in ("tc", "tcpp")


@pytest.mark.parametrize("dtype,kernel,unit", [("float32", "simt", 32), ("bfloat16", "simt", 32), ("bfloat16", "mma", 64)])
@pytest.mark.parametrize("splits", [2, 3, 7])
def test_split_keys_merge(ops, dtype, kernel, unit, splits):
    seqs = [(700, 1), (64, 1), (129, 2), (1, 1)]
    split_len = -(-(-(-700 // splits)) // unit) * unit
    n = -(-700 // split_len)
    out, exp, _, _ = attention_case(ops, dtype, 8, 2, 64, 16, seqs, plan=(kernel, n, split_len))
    assert rel(out, exp) < TOL[dtype]


@pytest.mark.parametrize("dtype,kernel", [("float32", "simt"), ("bfloat16", "simt"), ("bfloat16", "mma")])
@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_window(ops, dtype, kernel, window):
    out, exp, _, _ = attention_case(ops, dtype, 4, 2, 32, 8, [(150, 150), (90, 1), (300, 40)], window=window,
                                    plan=(kernel, 1, 0))
    assert rel(out, exp) < TOL[dtype]


@pytest.mark.parametrize("dtype,kernel", [("float32", "simt"), ("bfloat16", "mma"), ("bfloat16", "simt")])
@pytest.mark.parametrize("kpos,why", [(0, "the first key"), (63, "last key of a page"), (64, "first key of a page"),
                                      (447, "far key among hundreds"), (599, "the query's own position")])
def test_one_key_decides(ops, dtype, kernel, kpos, why):
    """Random inputs give near-uniform attention, which hides a misplaced key; here one key's score
    stands out, so the row's output must be that key's value."""
    seqs = [(50, 1), (600, 1), (64, 3)]
    for plan in ((kernel, 1, 0), (kernel, 3, 256)):
        out, exp, dense, qsl = attention_case(ops, dtype, 4, 1, 64, 64, seqs, plan=plan, spike=(1, 0, kpos))
        row = out[qsl[1]].view(4, 64)
        v = dense[1][1][kpos, 0]
        assert (row - v).abs().max() < 2e-2, why
        assert rel(out, exp) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edge_key(ops, dtype):
    """The key just outside the window must not count although its score would dominate; the key
    just inside must."""
    W = 100
    for kpos, inside in ((500 - W, False), (500 - W + 1, True)):
        out, exp, dense, qsl = attention_case(ops, dtype, 2, 1, 32, 16, [(501, 1)], window=W, spike=(0, 0, kpos))
        v = dense[0][1][kpos, 0]
        close = (out[0].view(2, 32) - v).abs().max() < 2e-2
        assert bool(close) == inside
        assert rel(out, exp) < TOL[dtype]


def test_refuses_sizes_it_cannot_take(ops):
    from tiny_transformer_inference_engine_b200.ops import KernelError
    with pytest.raises(KernelError, match="head size 18"):
        attention_case(ops, "float32", 2, 1, 18, 4, [(5, 5)])
    with pytest.raises(KernelError, match="head size 272"):
        attention_case(ops, "bfloat16", 2, 1, 272, 4, [(5, 5)])
    with pytest.raises(KernelError, match="not supported"):
        ops.linear(torch.zeros(2, 2, dtype=torch.float16, device=DEV), torch.zeros(2, 2, dtype=torch.float16, device=DEV), None) \
            if False else ops.embed(torch.zeros(1, dtype=torch.int32, device=DEV),
                                    torch.zeros(2, 2, dtype=torch.float16, device=DEV),
                                    torch.zeros(1, 2, dtype=torch.float32, device=DEV))


def test_split_decode_attention_in_many_waves_never_waits_in_vain(ops):
    """600 CTAs of six key tiles each, launch after launch: a CTA that starts while the memory system is busy gets its
    value tiles late, and the softmax threads then finish two tiles before the issuing thread has looked at the first.
    With one barrier for "P is written" that looked like no arrival at all and the wait ran out (a second later, with a
    wrong result); the barrier exists per score buffer now.  No wait may run out in 1,500 launches."""
    B, ctx, Hq, D, page = 100, 4096, 32, 128, 64
    pages = ctx // page
    g = torch.Generator().manual_seed(1)
    kp = torch.randn(B * pages + 1, 1, page, D, generator=g).bfloat16().to(DEV)
    vp = torch.randn(B * pages + 1, 1, page, D, generator=g).bfloat16().to(DEV)
    table = (torch.arange(B * pages, dtype=torch.int32) + 1).view(B, pages).to(DEV)
    q = torch.randn(B, Hq * D, generator=g).bfloat16().to(DEV)
    qsl = torch.arange(B + 1, dtype=torch.int32).to(DEV)
    lens = torch.full((B,), ctx, dtype=torch.int32).to(DEV)
    out = torch.empty_like(q)
    for i in range(1500):
        ops.paged_attention(q, Hq, 1, D, kp, vp, table, page, qsl, lens, B, 1, ctx, 1 / math.sqrt(D), 0, out, plan=("tc", 6, 768))
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    r = 7                                                            # one request against the float32 formula
    k = kp[1 + r * pages:1 + (r + 1) * pages, 0].reshape(ctx, D).float()
    v = vp[1 + r * pages:1 + (r + 1) * pages, 0].reshape(ctx, D).float()
    p = torch.softmax(q[r].view(Hq, D).float() @ k.T / math.sqrt(D), dim=-1)
    assert rel(out[r].view(Hq, D).float().cpu(), (p @ v).cpu()) < TOL["bfloat16"]


def test_a_block_table_that_cannot_cover_the_keys_is_refused(ops):
    q = torch.zeros(1, 4 * 64, dtype=torch.bfloat16, device=DEV)
    pages = torch.zeros(4, 1, 16, 64, dtype=torch.bfloat16, device=DEV)
    table = torch.ones(1, 2, dtype=torch.int32, device=DEV)                 # two pages of 16 keys
    qsl = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    lens = torch.tensor([40], dtype=torch.int32, device=DEV)
    from tiny_transformer_inference_engine_b200.ops import KernelError
    with pytest.raises(KernelError, match="cannot cover 40 keys"):
        ops.paged_attention(q, 4, 1, 64, pages, pages, table, 16, qsl, lens, 1, 1, 40, 0.125, 0, torch.empty_like(q))


def test_many_requests_with_grouped_kv_heads_are_cut_into_pieces(ops):
    """Decode steps whose (request, kv head) pairs alone fill the GPU: the tile loop's key range is cut so that the CTAs
    come in whole waves of what the GPU holds at once (5 per SM at head size 128), and the pieces merge to the float32
    reference."""
    assert ops.lib.ttie_attn_mma_ctas_per_sm(128, 1, 32, 8) == 5 and ops.num_sms == 148
    assert ops.attention_plan(torch.bfloat16, 64, 32, 8, 128, 1, 4096, 64) == ("mma", 5, 832)       # 2,560 CTAs, not 512 of 4,096 keys
    assert ops.attention_plan(torch.bfloat16, 32, 32, 8, 128, 1, 4096, 64) == ("mma", 11, 384)      # 2,816 CTAs: 3.8 waves
    assert ops.attention_plan(torch.bfloat16, 24, 32, 8, 128, 1, 2048, 64) == ("mma", 3, 704)       # 576 CTAs in one wave; 4 pieces would be 768
    assert ops.attention_plan(torch.bfloat16, 128, 32, 8, 128, 1, 2048, 64) == ("mma", 4, 512)
    assert ops.attention_plan(torch.bfloat16, 512, 32, 8, 128, 1, 4096, 64) == ("mma", 1, 0)        # 4,096 pairs: enough as they are
    seqs = [(1500 - 37 * i, 1) for i in range(24)]
    plan = ops.attention_plan(torch.bfloat16, len(seqs), 32, 8, 128, 1, 1500, 64)
    assert plan == ("mma", 3, 512)
    out, exp, _, _ = attention_case(ops, "bfloat16", 32, 8, 128, 64, seqs, plan=plan)
    assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]


# ------------------------------------------------------------------------------------------ sampling
def sampler_state(rows):
    st = torch.zeros(len(rows), 8, dtype=torch.int32)
    for i, (seed, draws, top_k, temp, top_p, greedy) in enumerate(rows):
        st[i] = torch.tensor([seed & 0x7fffffff, seed >> 31, draws, top_k,
                              struct.unpack("<i", struct.pack("<f", temp))[0],
                              struct.unpack("<i", struct.pack("<f", top_p))[0], greedy, 0], dtype=torch.int32)
    return st


@pytest.mark.parametrize("V,ctas", [(256, 0), (515, 1), (515, 2), (1000, 4), (1000, 8), (32000, 0), (32000, 1), (65024, 0), (65024, 2),
                                    (50001, 8), (256000, 0), (50000, 1), (337001, 8)])
def test_sampling_distribution_and_draw(ops, V, ctas):
    """``ctas`` CTAs share a row (0: the kernel's own choice); vocabularies that are no multiple of anything, slices
    that fit shared memory and slices that do not (50,000 tokens with one CTA, 337,001 with eight)."""
    g = torch.Generator().manual_seed(V)
    rows = [(1, 0, 0, 1.0, 1.0, 0), (2, 5, 32, 0.8, 1.0, 0), (3, 1, 0, 0.7, 0.9, 0), (4, 9, 50, 1.3, 0.5, 0),
            (5, 2, 1, 1.0, 1.0, 0), (6, 0, 0, 1.0, 1.0, 1), (7, 3, V + 5, 2.0, 0.999, 0), (8, 4, 3, 0.1, 0.3, 0)]
    R = len(rows)
    logits = torch.randn(R, V, generator=g) * 3
    logits[5, 17] = logits[5, 400 % V] = logits[5].max() + 1     # equal maxima: the lowest index wins
    state = sampler_state(rows)
    slot_ids = torch.arange(R, dtype=torch.int32)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    probs = torch.zeros(R, V, device=DEV)
    st_gpu = state.clone().to(DEV)
    ops.sample(logits.to(DEV), slot_ids.to(DEV), st_gpu, out, probs_out=probs, ctas_per_row=ctas)
    # the same draws without asking for the probabilities, and whatever the number of CTAs: the same tokens
    again = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), slot_ids.to(DEV), state.clone().to(DEV), again, ctas_per_row=1 if ctas != 1 else 4)
    assert torch.equal(again, out)
    out, probs, st_after = out.cpu(), probs.cpu(), st_gpu.cpu()
    assert torch.equal(st_after[:, 2], state[:, 2] + 1)           # every draw counter advanced
    for r, (seed, draws, top_k, temp, top_p, greedy) in enumerate(rows):
        if greedy:
            assert out[r] == min(17, 400 % V)
            continue
        exp = PLAIN.filtered_probs(logits[r], temp, top_k, top_p).float()
        assert torch.equal(probs[r] > 0, exp > 0), f"row {r}: kept sets differ"
        assert torch.allclose(probs[r], exp, atol=2e-6, rtol=1e-4)
        u = uniform_from_state(seed & 0x7fffffff, seed >> 31, draws)
        cdf = torch.cumsum(probs[r].double(), 0)
        tok = int(out[r])
        assert probs[r, tok] > 0
        lo = cdf[tok - 1].item() if tok else 0.0
        assert lo - 1e-5 <= u <= cdf[tok].item() + 1e-5, (r, u, lo, cdf[tok].item())
    assert out[4] == int(torch.argmax(logits[4]))                 # top_k = 1 is argmax (tests/test_sampling.py:6-12)


@pytest.mark.parametrize("V,ctas", [(32000, 1), (32000, 2), (32000, 8), (65024, 0), (256000, 0)])
def test_sampling_after_a_top_k_cut(ops, V, ctas):
    """With a small top-k the kernel leaves the row for a short list of candidates: top-k just below, at and above the
    largest value for which it does (256), a much larger one, and cuts that fall into thousands of equal values (the
    list overflows in some CTAs or in all, depending on how many share the row, and the whole row is walked): kept
    sets, probabilities and draws as the plain sampler's, and the same token whatever the number of CTAs."""
    g = torch.Generator().manual_seed(V + 1)
    R = 8
    logits = torch.randn(R, V, generator=g)
    logits[4, ::5] = 2.5                                           # a fifth of the row is equal; about 0.6 % of the rest lies above
    logits[5, 1::3] = 2.5
    logits[7, 100] = logits[7, V - 1] = logits[7].max() + 0.5       # two equal maxima with top_k = 2
    k4, k5 = int((logits[4] > 2.5).sum()) + 40, int((logits[5] > 2.5).sum()) + 7      # cuts inside the equal values
    rows = [(11, 0, 250, 0.9, 0.9, 0), (12, 3, 256, 1.1, 1.0, 0), (13, 1, 257, 0.7, 0.8, 0), (14, 7, 1500, 1.0, 0.95, 0),
            (15, 2, k4, 1.0, 0.9, 0), (16, 4, k5, 1.0, 1.0, 0), (17, 5, 32, 1.0, 0.9, 0), (18, 6, 2, 0.5, 0.6, 0)]
    state = sampler_state(rows)
    slot_ids = torch.arange(R, dtype=torch.int32)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    probs = torch.zeros(R, V, device=DEV)
    st_gpu = state.clone().to(DEV)
    ops.sample(logits.to(DEV), slot_ids.to(DEV), st_gpu, out, probs_out=probs, ctas_per_row=ctas)
    for other in (1, 4):
        again = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample(logits.to(DEV), slot_ids.to(DEV), state.clone().to(DEV), again, ctas_per_row=other)
        assert torch.equal(again, out)
    out, probs = out.cpu(), probs.cpu()
    for r, (seed, draws, top_k, temp, top_p, greedy) in enumerate(rows):
        exp = PLAIN.filtered_probs(logits[r], temp, top_k, top_p).float()
        assert torch.equal(probs[r] > 0, exp > 0), f"row {r}: kept sets differ"
        assert torch.allclose(probs[r], exp, atol=2e-6, rtol=1e-4)
        u = uniform_from_state(seed & 0x7fffffff, seed >> 31, draws)
        cdf = torch.cumsum(probs[r].double(), 0)
        tok = int(out[r])
        assert probs[r, tok] > 0
        lo = cdf[tok - 1].item() if tok else 0.0
        assert lo - 1e-5 <= u <= cdf[tok].item() + 1e-5, (r, u, lo, cdf[tok].item())
    assert int((probs[4] > 0).sum()) > V // 5 and int((probs[5] > 0).sum()) > V // 3 - 1     # the equal values stayed together


@pytest.mark.parametrize("V,ctas", [(515, 1), (32000, 0), (32000, 1), (65024, 2), (256000, 0)])
def test_sampling_with_top_p_alone(ops, V, ctas):
    """Top-p without a top-k: peaked rows, where the tokens of 1/1,024 of the mass or more reach past the cut and the
    kernel leaves the row for them; flat rows, where they do not and the whole row is walked; a row whose listed tokens
    hold just about top_p of the mass; a row of equal values; a row with one token of nearly all the mass.  Kept sets,
    probabilities and draws as the plain sampler's, and the same token whatever the number of CTAs."""
    g = torch.Generator().manual_seed(V + 2)
    R = 8
    logits = torch.randn(R, V, generator=g)
    logits[0] *= 8.0                                               # peaked
    logits[1] *= 5.0
    logits[2] *= 0.5                                               # flat: nearly every token is needed
    logits[3] *= 3.0                                               # in between (the outcome depends on V)
    logits[4] = 1.25                                               # all equal: stay together
    logits[5, 7 % V] = 40.0                                        # one token holds nearly everything
    logits[6] *= 6.0
    logits[6, 1::2] = logits[6, ::2][: logits[6, 1::2].numel()]    # equal pairs at every level
    logits[7] *= 4.0
    rows = [(21, 0, 0, 1.0, 0.9, 0), (22, 3, 0, 0.8, 0.95, 0), (23, 1, 0, 1.0, 0.9, 0), (24, 7, 0, 1.0, 0.92, 0),
            (25, 2, 0, 1.0, 0.5, 0), (26, 4, 0, 1.0, 0.3, 0), (27, 5, V, 1.1, 0.7, 0), (28, 6, 0, 0.6, 0.999, 0)]
    state = sampler_state(rows)
    slot_ids = torch.arange(R, dtype=torch.int32)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    probs = torch.zeros(R, V, device=DEV)
    ops.sample(logits.to(DEV), slot_ids.to(DEV), state.clone().to(DEV), out, probs_out=probs, ctas_per_row=ctas)
    for other in (1, 4):
        again = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample(logits.to(DEV), slot_ids.to(DEV), state.clone().to(DEV), again, ctas_per_row=other)
        assert torch.equal(again, out)
    out, probs = out.cpu(), probs.cpu()
    for r, (seed, draws, top_k, temp, top_p, greedy) in enumerate(rows):
        exp = PLAIN.filtered_probs(logits[r], temp, top_k, top_p).float()
        assert torch.equal(probs[r] > 0, exp > 0), f"row {r}: kept sets differ ({int((probs[r] > 0).sum())} against {int((exp > 0).sum())})"
        assert torch.allclose(probs[r], exp, atol=2e-6, rtol=1e-4)
        u = uniform_from_state(seed & 0x7fffffff, seed >> 31, draws)
        cdf = torch.cumsum(probs[r].double(), 0)
        tok = int(out[r])
        assert probs[r, tok] > 0
        lo = cdf[tok - 1].item() if tok else 0.0
        assert lo - 1e-5 <= u <= cdf[tok].item() + 1e-5, (r, u, lo, cdf[tok].item())
    assert int((probs[4] > 0).sum()) == V and int((probs[5] > 0).sum()) == 1
    assert int((probs[0] > 0).sum()) < 1024 < int((probs[2] > 0).sum()) or V < 2048     # a short nucleus and one no list can hold


def test_sampling_skips_padding_rows(ops):
    """A row whose slot id is -1 (padding of a fixed-size batch) yields token 0 and touches no state."""
    V = 300
    logits = torch.randn(3, V, generator=torch.Generator().manual_seed(2)).to(DEV)
    state = sampler_state([(5, 4, 0, 1.0, 1.0, 1), (6, 9, 0, 1.0, 1.0, 1)]).to(DEV)
    before = state.clone()
    out = torch.full((3,), 77, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.tensor([-1, 1, -1], dtype=torch.int32, device=DEV), state, out)
    assert out.tolist() == [0, int(torch.argmax(logits[1])), 0]
    assert torch.equal(state[0], before[0]) and int(state[1, 2]) == 10


def test_sampling_frequencies(ops):
    """Many draws of one row follow its probabilities."""
    V, n = 50, 4000
    logits = torch.randn(1, V, generator=torch.Generator().manual_seed(0)) * 2
    state = sampler_state([(123, 0, 10, 0.9, 0.95, 0)]).to(DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    lg, counts = logits.to(DEV), torch.zeros(V)
    for _ in range(n):
        ops.sample(lg, slot, state, out)
        counts[int(out)] += 1
    exp = PLAIN.filtered_probs(logits[0], 0.9, 10, 0.95).float()
    assert int(state[0, 2]) == n
    assert (counts[exp == 0] == 0).all()
    assert (counts / n - exp).abs().max() < 0.03


# ------------------------------------------------------------------------------------------ weight-streaming product
@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 4352, 4096), (3, 515, 200), (16, 1000, 176), (9, 4096, 11008),
                                   (5, 72, 8), (16, 33, 4544), (33, 200, 512), (64, 96, 4096), (2, 32000, 4096)])
def test_skinny_gemm_all_epilogues(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    b = torch.randn(N, generator=g).bfloat16()
    exp = x.double() @ w.double().T
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    ops.skinny_max_rows = 64
    assert ops._skinny_ok(xd, wd)
    before = ops.launches
    assert rel(ops.linear(xd, wd, None).float().cpu(), exp) < 8e-3
    assert rel(ops.linear(xd, wd, bd).float().cpu(), exp + b.double()) < 8e-3
    out32 = ops.linear(xd, wd, bd, out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and rel(out32.cpu(), exp + b.double()) < 1e-5
    assert ops.launches == before + 3                              # this package's kernel ran, not the library's
    part = ops.linear(xd, wd, None, partial_ok=True)
    if part.dim() == 3:
        assert part.dtype == torch.float32 and rel(part.sum(0).cpu(), exp) < 1e-5
    # forced K split: partial sums feed add_rmsnorm and rope_store
    for kslice in (128, 256):
        S = -(-K // kslice)
        part = torch.empty(S, M, N, dtype=torch.float32, device=DEV)
        rc = ops.lib.ttie_skinny_gemm(xd.data_ptr(), xd.stride(0), wd.data_ptr(), wd.stride(0), None, part.data_ptr(), N,
                                      M, N, K, kslice, 1, 0, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        assert rel(part.sum(0).cpu(), exp) < 1e-5
    # two sets of 16 weight rows per CTA (the form the load-time measurement may pick): every epilogue, K whole and cut
    stream = torch.cuda.current_stream().cuda_stream
    for kslice in (-(-K // 128) * 128, 256):
        S = -(-K // kslice)
        part = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
        assert ops.lib.ttie_skinny_gemm_tuned(xd.data_ptr(), xd.stride(0), wd.data_ptr(), wd.stride(0), None, part.data_ptr(), N,
                                              M, N, K, kslice, 1, 0, 16, stream) == 0
        assert rel(part.sum(0).cpu(), exp) < 1e-5
    o16 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    o32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    for out, epi, tol in ((o16, 0, 8e-3), (o32, 3, 1e-5)):
        assert ops.lib.ttie_skinny_gemm_tuned(xd.data_ptr(), xd.stride(0), wd.data_ptr(), wd.stride(0), bd.data_ptr(), out.data_ptr(), N,
                                              M, N, K, -(-K // 128) * 128, epi, 0, 16 + 4, stream) == 0
        assert rel(out.float().cpu(), exp + b.double()) < tol
    if N % 2 == 0:
        F = N // 2
        act = ops.linear_swiglu(xd, wd, bd, F)
        gu = exp + b.double()
        ref = gu[:, :F] * torch.sigmoid(gu[:, :F]) * gu[:, F:]
        assert rel(act.float().cpu(), ref) < 1.2e-2
    ops.skinny_max_rows = 8


def test_weight_streaming_form_is_measured_at_load(ops):
    """``tune_products`` on a shape of a model: the product for 8, 16, 32 and 64 rows and, at 8 and 16 rows, the form of this
    package's kernel (K ranges over CTAs, one or two row sets per CTA) are chosen by measurement; a caller that takes
    partial sums and one that wants whole sums are decided apart, and both get the right values."""
    N, K = 2048, 8192
    g = torch.Generator().manual_seed(3)
    ws = [(torch.randn(N, K, generator=g) * 0.02).bfloat16().to(DEV) for _ in range(3)]
    keep = dict(ops._product_choice), dict(ops._skinny_tuned)
    try:
        ops.tune_products(ws)
        for M in (8, 16, 32, 64):
            took = ops.product_timings[(N, K, M)]
            assert took["library"] > 0 and took["skinny"] > 0 and took["skinny"] <= took["skinny_uncut"] * 1.05
            assert ops._product_choice[(N, K, M)] in ("skinny", "library") and ops._product_choice[(N, K, M, "split")] in ("skinny", "library")
        # a narrow deep matrix: this package's kernel with K cut over CTAs wins at 8 and 16 rows
        assert ops._product_choice[(N, K, 8, "split")] == "skinny" and ops._product_choice[(N, K, 16, "split")] == "skinny"
        for M in (3, 8, 13, 16, 40):
            x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
            exp = x.double().cpu() @ ws[1].double().cpu().T
            part = ops.linear(x, ws[1], None, partial_ok=True)
            got = part.sum(0) if part.dim() == 3 else part.float()
            assert rel(got.double().cpu(), exp) < (1e-5 if part.dim() == 3 else 8e-3)
            assert rel(ops.linear(x, ws[1], None).double().cpu(), exp) < 8e-3
    finally:
        ops._product_choice.clear(); ops._product_choice.update(keep[0])
        ops._skinny_tuned.clear(); ops._skinny_tuned.update(keep[1])


def test_swiglu_product_for_few_rows_is_chosen_by_measurement(ops):
    """Up to 8 rows the gate/up product carries SwiGLU in its epilogue or runs K-split-free and hands over to the
    activation kernel, whichever measured faster for the shape at its first use; both give the reference's values."""
    g = torch.Generator().manual_seed(5)
    for F, K in ((1024, 8192), (2752, 1024)):
        x = torch.randn(8, K, generator=g).bfloat16()
        w = (torch.randn(2 * F, K, generator=g) * 0.02).bfloat16()
        gu = x.double() @ w.double().T
        ref = gu[:, :F] * torch.sigmoid(gu[:, :F]) * gu[:, F:]
        xd, wd = x.to(DEV), w.to(DEV)
        ops._swiglu_choice.pop((F, K, "few"), None)
        act = ops.linear_swiglu(xd, wd, None, F)
        took = ops.product_timings[("swiglu", F, K, "few")]
        assert set(took) == {"fused", "unfused"} and ops._swiglu_choice[(F, K, "few")] == (took["fused"] <= 1.03 * took["unfused"])
        assert rel(act.float().cpu(), ref) < 1.2e-2
        for forced in (True, False):                                   # both forms, whatever was measured
            ops._swiglu_choice[(F, K, "few")] = forced
            assert rel(ops.linear_swiglu(xd, wd, None, F).float().cpu(), ref) < 1.2e-2
        del ops._swiglu_choice[(F, K, "few")]
    # 64 CTAs of 512 KB each against a product cut over K: the fused form loses by far on such a shape
    assert ops.product_timings[("swiglu", 1024, 8192, "few")]["unfused"] < ops.product_timings[("swiglu", 1024, 8192, "few")]["fused"]


def test_partial_sums_feed_norm_and_rope(ops):
    g = torch.Generator().manual_seed(7)
    S, T, d = 3, 5, 200
    part = torch.randn(S, T, d, generator=g)
    resid = torch.randn(T, d, generator=g)
    w = 1 + 0.1 * torch.randn(d, generator=g)
    r_gpu, out = resid.clone().to(DEV), torch.empty(T, d, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(r_gpu, part.to(DEV), w.to(DEV), 1e-5, out)
    r_cpu, exp = resid.clone(), torch.empty(T, d, dtype=torch.bfloat16)
    PLAIN.add_rmsnorm(r_cpu, part.sum(0), w, 1e-5, exp)
    assert rel(r_gpu.cpu(), r_cpu) < 1e-6 and rel(out.float().cpu(), exp.float()) < 8e-3
    rows = torch.tensor([4, 1], dtype=torch.int32)
    out2 = torch.empty(2, d, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm_rows(resid.to(DEV), part.to(DEV), rows.to(DEV), 2, w.to(DEV), 1e-5, out2)
    exp2 = torch.empty(2, d, dtype=torch.bfloat16)
    PLAIN.rmsnorm_rows(resid, part.sum(0), rows, 2, w, 1e-5, exp2)
    assert rel(out2.float().cpu(), exp2.float()) < 8e-3
    # rope_store from partial sums == rope_store of their sum
    Hq, Hkv, D, page = 5, 1, 32, 4
    width = (Hq + 2 * Hkv) * D
    part = torch.randn(S, T, width, generator=g)
    positions = torch.tensor([0, 1, 2, 3, 9], dtype=torch.int32)
    token_seq = torch.tensor([0, 0, 0, 0, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0, 0], [1, 3, 4]], dtype=torch.int32)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    kp, vp = torch.zeros(5, Hkv, page, D, dtype=torch.bfloat16, device=DEV), torch.zeros(5, Hkv, page, D, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    ops.rope_store(part.to(DEV), Hq, Hkv, D, positions.to(DEV), token_seq.to(DEV), inv_freq.to(DEV), 0, kp, vp, table.to(DEV),
                   page, True, q_out=q_out)
    summed = part.sum(0)
    kp2, vp2 = torch.zeros(5, Hkv, page, D), torch.zeros(5, Hkv, page, D)
    PLAIN.rope_store(summed, Hq, Hkv, D, positions, token_seq, inv_freq, 0, kp2, vp2, table, page, True)
    assert rel(q_out.float().cpu(), summed[:, :Hq * D]) < 8e-3
    assert rel(kp.float().cpu(), kp2) < 8e-3 and rel(vp.float().cpu(), vp2) < 8e-3


def cluster_plan(ops, groups, cluster, max_kv, D, max_q, Hq, Hkv):
    C = cluster
    while C > 1 and ops.lib.ttie_attn_cluster_active(D, max_q, Hq, Hkv, groups, C) < 1:
        C //= 2
    assert ops.lib.ttie_attn_cluster_active(D, max_q, Hq, Hkv, groups, C) >= 1
    return (f"mma_c{groups}", C, -(-(-(-max_kv // C)) // 64) * 64)


@pytest.mark.parametrize("Hq,Hkv,D,page", [(32, 1, 128, 64), (71, 1, 64, 16), (6, 2, 48, 32), (3, 1, 32, 8), (4, 4, 16, 5), (128, 1, 64, 64)])
@pytest.mark.parametrize("seqs", [[(200, 1), (64, 1), (65, 1), (1, 1), (513, 1)], [(130, 2), (128, 1), (129, 1)], [(4096, 1)] * 2,
                                  [(700, 5), (3, 3), (1100, 1)]])
@pytest.mark.parametrize("groups,cluster", [(4, 16), (4, 4), (2, 8), (2, 1), (4, 1), (2, 2)])
def test_decode_form_attention(ops, Hq, Hkv, D, page, seqs, groups, cluster):
    """One cluster per (request, kv head, row tile): every cluster size, both numbers of key groups, requests
    far shorter than the longest (CTAs and groups without keys), several row tiles, a window."""
    max_kv, max_q = max(L for L, _ in seqs), max(q for _, q in seqs)
    plan = cluster_plan(ops, groups, cluster, max_kv, D, max_q, Hq, Hkv)
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=plan)
    assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=plan, window=70)
    assert rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("kpos", [0, 63, 64, 127, 128, 447, 599])
@pytest.mark.parametrize("groups,cluster", [(4, 4), (2, 16)])
def test_decode_form_one_key_decides(ops, kpos, groups, cluster):
    seqs = [(50, 1), (600, 1), (64, 1)]
    plan = cluster_plan(ops, groups, cluster, 600, 64, 1, 4, 1)
    out, exp, dense, qsl = attention_case(ops, "bfloat16", 4, 1, 64, 64, seqs, plan=plan, spike=(1, 0, kpos))
    assert (out[qsl[1]].view(4, 64) - dense[1][1][kpos, 0]).abs().max() < 2e-2
    assert rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("Hq,Hkv,D,page", [(32, 1, 128, 64), (71, 1, 64, 16), (8, 2, 128, 8), (3, 1, 64, 128), (128, 1, 64, 64), (40, 1, 128, 32)])
@pytest.mark.parametrize("seqs", [[(200, 1), (64, 1), (65, 1), (1, 1), (513, 1)], [(130, 2), (128, 1), (129, 1)], [(4096, 1)] * 2,
                                  [(700, 5), (3, 3), (1100, 1)]])
@pytest.mark.parametrize("split_len", [128, 256, 1024])
def test_tcgen05_attention_with_splits(ops, Hq, Hkv, D, page, seqs, split_len):
    """The tcgen05 kernel on decode-shaped steps: key range cut over CTAs (some of them without a visible key),
    one to four quarters of the 128-row tile in use, partial results merged by the merge kernel."""
    max_kv = max(L for L, _ in seqs)
    n = -(-max_kv // split_len)
    plan = ("tc", n, split_len) if n > 1 else ("tc", 1, 0)
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=plan)
    assert ops.tc_error() == 0
    assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=plan, window=70)
    assert ops.tc_error() == 0
    assert rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("kpos", [0, 127, 128, 447, 599])
def test_tcgen05_splits_one_key_decides(ops, kpos):
    seqs = [(50, 1), (600, 1), (64, 1)]
    out, exp, dense, qsl = attention_case(ops, "bfloat16", 4, 1, 64, 64, seqs, plan=("tc", 5, 128), spike=(1, 0, kpos))
    assert ops.tc_error() == 0
    assert (out[qsl[1]].view(4, 64) - dense[1][1][kpos, 0]).abs().max() < 2e-2
    assert rel(out, exp) < TOL["bfloat16"]


def test_decode_form_is_planned(ops):
    """Decode steps of the bfloat16 path take the tcgen05 kernel with the key range cut over CTAs at head size 64 or 128
    where a request brings 32 rows or more per kv head, or fewer on a nearly empty GPU; otherwise, and at another head size,
    the decode form while a warp has one key tile to walk, and the tile loop with splits beyond; prompt portions the tcgen05
    kernels or the tile loop."""
    kernel, n, split_len = ops.attention_plan(torch.bfloat16, 8, 32, 1, 128, 1, 2048, 64)
    assert kernel == "tc" and n * split_len >= 2048 and 8 * n <= 148
    assert ops.attention_plan(torch.bfloat16, 64, 32, 1, 128, 1, 256, 64) == ("tc", 1, 0)
    assert ops.attention_plan(torch.bfloat16, 256, 32, 1, 128, 1, 4096, 64) == ("tc", 1, 0)       # more requests than SMs: uncut, wave after wave
    assert ops.attention_plan(torch.bfloat16, 512, 32, 1, 128, 1, 512, 64)[0] == "mma"            # ... unless the requests are short
    assert ops.attention_plan(torch.bfloat16, 8, 8, 1, 128, 1, 2048, 64) == ("tc", 16, 128)       # 8 rows per request: while the GPU is far from full
    kernel, C, split_len = ops.attention_plan(torch.bfloat16, 8, 8, 1, 96, 1, 2048, 64)           # ... at a head size the tcgen05 kernel does not take
    assert kernel == "mma_c4" and C * split_len >= 2048 and C & (C - 1) == 0 and split_len <= 256
    assert ops.attention_plan(torch.bfloat16, 96, 40, 2, 128, 1, 2048, 64)[0] == "mma"            # 20 rows per kv head, more CTAs than SMs
    kernel, n, split_len = ops.attention_plan(torch.bfloat16, 24, 32, 8, 128, 1, 2048, 64)        # the tile loop's pieces fill whole waves of
    per_sm = ops.lib.ttie_attn_mma_ctas_per_sm(128, 1, 32, 8)                                     # resident CTAs: not 769 CTAs for 740 places
    assert kernel == "mma" and per_sm >= 4 and (24 * 8 * n) % (per_sm * 148) <= 0.9 * per_sm * 148 and n * split_len >= 2048
    kernel, n, split_len = ops.attention_plan(torch.bfloat16, 96, 32, 1, 128, 1, 8192, 64)        # 96 CTAs would leave a third of the SMs idle
    assert kernel == "tc" and n == 3
    assert ops.attention_plan(torch.bfloat16, 8, 32, 1, 96, 1, 2048, 64)[0] == "mma_c4"           # a head size the tcgen05 kernel does not take
    assert ops.attention_plan(torch.bfloat16, 3, 4, 2, 48, 1, 100, 16)[0] == "mma_c2"
    assert ops.attention_plan(torch.bfloat16, 3, 4, 2, 64, 1, 100, 16) == ("tc", 1, 0)             # two rows per kv head, but the GPU is nearly empty
    assert ops.attention_plan(torch.bfloat16, 64, 8, 1, 128, 1, 256, 64) == ("mma_c4", 1, 256)
    kernel, n, split_len = ops.attention_plan(torch.bfloat16, 8, 32, 1, 128, 1, 32768, 64)
    assert kernel == "tc" and n * split_len >= 32768 and split_len % 128 == 0 and 8 * n <= 148
    assert ops.attention_plan(torch.bfloat16, 8, 32, 1, 96, 1, 32768, 64)[0] == "mma"       # a head size the tcgen05 kernel does not take
    assert ops.attention_plan(torch.bfloat16, 8, 32, 8, 128, 1, 32768, 64)[0] == "mma"      # four rows per kv head
    assert ops.attention_plan(torch.bfloat16, 1, 32, 1, 128, 2048, 2048, 64) == ("tcpp", 1, 0)
    assert ops.attention_plan(torch.bfloat16, 1, 32, 1, 128, 512, 6144, 64) == ("tcpp", 2, 3072)    # a short portion behind a long context
    assert ops.attention_plan(torch.bfloat16, 1, 32, 1, 128, 512, 512, 64) == ("tc", 1, 0)          # a short portion without one
    assert ops.attention_plan(torch.bfloat16, 4, 32, 1, 128, 512, 512, 64) == ("tcpp", 1, 0)
    assert ops.attention_plan(torch.bfloat16, 2, 8, 2, 48, 200, 200, 16)[0] == "mma"


# ------------------------------------------------------------------------------------------ tcgen05 product
@pytest.mark.parametrize("M,N,K,tile_n", [(128, 256, 64, 256), (2048, 4352, 4096, 256), (300, 520, 200, 256), (1, 1000, 64, 128),
                                          (129, 72, 4544, 128), (700, 515 * 8, 176 * 8, 256), (260, 33000, 64, 256)])
def test_gemm_tcgen05(ops, M, N, K, tile_n):
    """TMA + tcgen05.mma + TMEM product against float64; tiles that hang over every edge, many tiles per
    CTA (the persistent loop and both accumulator buffers), bias, float32 output."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    b = torch.randn(N, generator=g).bfloat16().to(DEV)
    ref = x.double() @ w.double().T
    assert rel(ops.linear_tc(x, w, None, None, tile_n).double(), ref) < 8e-3
    assert rel(ops.linear_tc(x, w, b, torch.float32, tile_n).double(), ref + b.double()) < 1e-5
    # a strided activation (column slice of a wider buffer)
    wide = torch.randn(M, K + 64, generator=g).bfloat16().to(DEV)
    xs = wide[:, 8:8 + K]
    assert rel(ops.linear_tc(xs, w, None, torch.float32, tile_n).double(), xs.double() @ w.double().T) < 1e-5
    assert ops.tc_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (2048, 4352, 4096), (300, 520, 200), (1, 1000, 64), (129, 72, 4544),
                                   (700, 515 * 8, 176 * 8), (260, 33000, 64), (513, 4096, 11008), (2048, 4096, 4096),
                                   (1030, 19200, 72), (2048, 5000, 8 * 19), (4100, 4544, 1000)])
def test_gemm_tcgen05_on_cta_pairs(ops, M, N, K):
    """The product on pairs of CTAs (tcgen05.mma.cta_group::2, 256 x 256 tiles) against float64: tiles that hang over
    every edge, many tiles per pair (the persistent loop and both accumulator buffers), bias, float32 output, a
    strided activation."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    b = torch.randn(N, generator=g).bfloat16().to(DEV)
    ref = x.double() @ w.double().T
    tol32 = 1e-5 * max(1.0, (K / 4096) ** 0.5)                    # 32-bit accumulation over K products
    assert rel(ops.linear_tc_pair(x, w, None).double(), ref) < 8e-3
    assert rel(ops.linear_tc_pair(x, w, b, torch.float32).double(), ref + b.double()) < tol32
    wide = torch.randn(M, K + 64, generator=g).bfloat16().to(DEV)
    xs = wide[:, 8:8 + K]
    assert rel(ops.linear_tc_pair(xs, w, None, torch.float32).double(), xs.double() @ w.double().T) < tol32
    assert ops.tc_error() == 0


@pytest.mark.parametrize("M,F,K,bias", [(256, 128, 64, False), (2048, 11008, 4096, False), (300, 176, 200, True), (1, 1000, 64, True),
                                        (515, 18176, 512, False), (130, 200, 4544, True), (2048, 9700, 192, True)])
def test_gemm_tcgen05_pair_with_swiglu(ops, M, F, K, bias):
    """The gate/up product with silu(g) * u in its epilogue: the leader's half of the tile holds gate columns, its
    peer's the matching up columns; widths that are no multiple of the tile, with and without biases."""
    g = torch.Generator().manual_seed(M + F)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(2 * F, K, generator=g) * 0.05).bfloat16().to(DEV)
    b = torch.randn(2 * F, generator=g).bfloat16().to(DEV) if bias else None
    y = x.double() @ w.double().T + (b.double() if bias else 0)
    ref = torch.nn.functional.silu(y[:, :F]) * y[:, F:]
    out = ops.linear_swiglu_tc_pair(x, w, b, F)
    assert out.shape == (M, F) and rel(out.double(), ref) < 8e-3
    assert ops.tc_error() == 0


# ------------------------------------------------------------------------------------------ tcgen05 attention
TC_SHAPES = [(32, 1, 128, 64), (32, 1, 128, 16), (8, 2, 64, 8), (3, 1, 64, 128), (71, 1, 64, 64), (4, 2, 128, 32), (5, 5, 64, 256)]


TC_KERNELS = ["tc", "tcpp"]                                       # one 128-row query tile per CTA; two tiles taken in turns
TC_WIDE_SHAPES = [(8, 1, 256, 16), (8, 1, 256, 64), (3, 3, 256, 128)]   # head size 256: the second kernel with one tile per CTA


@pytest.mark.parametrize("scenario", ["prefill", "chunked", "mixed", "decode"])
@pytest.mark.parametrize("Hq,Hkv,D,page", TC_WIDE_SHAPES)
def test_tcgen05_attention_head_size_256(ops, scenario, Hq, Hkv, D, page):
    seqs = SCENARIOS[scenario] + [(700, 700)]
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=("tcpp", 1, 0))
    assert ops.tc_error() == 0
    assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]
    # and it is what the planner picks at this head size, whatever the step
    assert ops.attention_plan(torch.bfloat16, len(seqs), Hq, Hkv, D, max(n for _, n in seqs), 700, page)[0] == "tcpp"


@pytest.mark.parametrize("Hq,Hkv,D,page", TC_WIDE_SHAPES[:2])
def test_tcgen05_attention_head_size_256_windows_splits_and_one_key(ops, Hq, Hkv, D, page):
    for window in (1, 5, 100, 129, 300):
        out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, [(450, 450), (90, 1), (300, 40)], window=window, plan=("tcpp", 1, 0))
        assert rel(out, exp) < TOL["bfloat16"], window
    for split_len in (128, 512):
        n = -(-1500 // split_len)
        for window in (0, 200):
            out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, [(1500, 200), (300, 300), (900, 1), (64, 64)],
                                            plan=("tcpp", n, split_len), window=window)
            assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"], (split_len, window)
    seqs = [(50, 1), (600, 1), (64, 3), (600, 600)]
    for kpos in (0, 63, 64, 127, 128, 447, 599):
        for sq, qi in ((1, 0), (3, 599)):
            out, exp, dense, qsl = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=("tcpp", 1, 0), spike=(sq, qi, kpos))
            row = out[qsl[sq] + qi].view(Hq, D)
            assert (row - dense[sq][1][kpos, 0]).abs().max() < 2e-2, (kpos, sq)
            assert rel(out, exp) < TOL["bfloat16"]
    # the planner's own choice for decoded tokens with long contexts: the key range cut over CTAs
    plan = ops.attention_plan(torch.bfloat16, 4, Hq, Hkv, D, 1, 3000, page)
    assert plan[0] == "tcpp" and plan[1] > 1
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, [(3000, 1), (2000, 1), (1, 1), (129, 1)])
    assert rel(out, exp) < TOL["bfloat16"]
    assert ops.tc_error() == 0


@pytest.mark.parametrize("kernel", TC_KERNELS)
@pytest.mark.parametrize("scenario", ["prefill", "chunked", "mixed", "decode"])
@pytest.mark.parametrize("Hq,Hkv,D,page", TC_SHAPES)
def test_tcgen05_attention(ops, kernel, scenario, Hq, Hkv, D, page):
    seqs = SCENARIOS[scenario] + [(700, 700)]
    out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=(kernel, 1, 0))
    assert ops.tc_error() == 0
    assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("kernel", TC_KERNELS)
@pytest.mark.parametrize("window", [1, 5, 100, 129, 300])
def test_tcgen05_attention_window(ops, kernel, window):
    out, exp, _, _ = attention_case(ops, "bfloat16", 4, 2, 64, 16, [(450, 450), (90, 1), (300, 40)], window=window, plan=(kernel, 1, 0))
    assert ops.tc_error() == 0 and rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("split_len", [128, 512])
@pytest.mark.parametrize("Hq,Hkv,D,page", [(32, 1, 128, 64), (8, 2, 64, 8), (5, 5, 64, 256)])
def test_tcgen05_two_tile_attention_with_splits(ops, Hq, Hkv, D, page, split_len):
    """The two-tile kernel with the key range cut over CTAs (a long context behind a short portion): partial results
    relative to a maximum that may lag the true one, merged by the merge kernel; splits without a visible key."""
    seqs = [(1500, 200), (300, 300), (900, 1), (64, 64)]
    n = -(-1500 // split_len)
    for window in (0, 200):
        out, exp, _, _ = attention_case(ops, "bfloat16", Hq, Hkv, D, page, seqs, plan=("tcpp", n, split_len), window=window)
        assert ops.tc_error() == 0
        assert torch.isfinite(out).all() and rel(out, exp) < TOL["bfloat16"]


def test_tcgen05_two_tile_attention_rescales(ops):
    """Keys whose scores grow along the sequence, so that the running maximum of every row passes the rescale
    threshold several times, and a row whose output is decided by one late key after large earlier ones."""
    for kpos in (5, 300, 1023):
        out, exp, dense, qsl = attention_case(ops, "bfloat16", 8, 1, 128, 64, [(1024, 1024), (700, 64)], plan=("tcpp", 1, 0),
                                              spike=(0, 1023, kpos))
        assert ops.tc_error() == 0
        assert (out[qsl[0] + 1023].view(8, 128) - dense[0][1][kpos, 0]).abs().max() < 2e-2
        assert rel(out, exp) < TOL["bfloat16"]


@pytest.mark.parametrize("kernel", TC_KERNELS)
@pytest.mark.parametrize("kpos", [0, 63, 64, 127, 128, 447, 599])
def test_tcgen05_attention_one_key_decides(ops, kernel, kpos):
    seqs = [(50, 1), (600, 1), (64, 3), (600, 600)]
    for spike_q in ((1, 0), (3, 599)):
        out, exp, dense, qsl = attention_case(ops, "bfloat16", 4, 1, 64, 64, seqs, plan=(kernel, 1, 0), spike=(spike_q[0], spike_q[1], kpos))
        row = out[qsl[spike_q[0]] + spike_q[1]].view(4, 64)
        assert (row - dense[spike_q[0]][1][kpos, 0]).abs().max() < 2e-2
        assert rel(out, exp) < TOL["bfloat16"]
    assert ops.tc_error() == 0


def test_tcgen05_attention_refuses(ops):
    from tiny_transformer_inference_engine_b200.ops import KernelError
    with pytest.raises(KernelError, match="not supported"):
        attention_case(ops, "bfloat16", 4, 1, 32, 16, [(40, 40)], plan=("tc", 1, 0))
    with pytest.raises(KernelError, match="not supported"):
        attention_case(ops, "bfloat16", 4, 1, 64, 24, [(40, 40)], plan=("tc", 1, 0))
    with pytest.raises(KernelError, match="prompt-portion form only"):
        attention_case(ops, "bfloat16", 4, 1, 256, 16, [(40, 40)], plan=("tc", 1, 0))
