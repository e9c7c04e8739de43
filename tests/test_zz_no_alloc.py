"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of the library cannot allocate device memory at the time they need attention computed
(all memory already handed to their own pools, another runtime's allocator in charge, or a loop
in which an allocation's latency is not acceptable).  For them the library keeps the split-key
scratch in a device array of its own.  This test calls that entry point twice in a row, with
different inputs, and compares each result with the regular entry point's (which gets its scratch
from the caller), within the tolerance the other attention tests use; it also checks that a size
beyond the library's array is refused with a message.  The file is named to be collected last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1.2e-2


def _case(seed, seqs, Hq, Hkv, D, page):
    g = torch.Generator().manual_seed(seed)
    N, T = len(seqs), sum(n for _, n in seqs)
    width = max(-(-L // page) for L, _ in seqs)
    nb = sum(-(-L // page) for L, _ in seqs) + 1
    order = (torch.randperm(nb - 1, generator=g) + 1).tolist()
    table = torch.zeros(N, width, dtype=torch.int32)
    for i, (L, _) in enumerate(seqs):
        for pg in range(-(-L // page)):
            table[i, pg] = order.pop()
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, generator=g) * 0.7).bfloat16()
    kp = (torch.randn(nb, Hkv, page, D, generator=g) * 0.7).bfloat16()
    vp = torch.randn(nb, Hkv, page, D, generator=g).bfloat16()
    qsl = [0]
    for _, n in seqs:
        qsl.append(qsl[-1] + n)
    return dict(qkv=qkv.to(DEV), kp=kp.to(DEV), vp=vp.to(DEV), table=table.to(DEV),
                qsl=torch.tensor(qsl, dtype=torch.int32, device=DEV),
                seq_lens=torch.tensor([L for L, _ in seqs], dtype=torch.int32, device=DEV),
                N=N, T=T, max_q=max(n for _, n in seqs), max_kv=max(L for L, _ in seqs))


def _call_noalloc(lib, c, Hq, Hkv, D, page, num_splits, split_len, out):
    fn = lib.ttie_paged_attention_mma_noalloc
    V, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [V, LL, V, V, V, I, I, V, V, V, I, I, I, I, I, I, F, I, I, I, V]
    fn.restype = I
    return fn(c["qkv"].data_ptr(), c["qkv"].stride(0), c["kp"].data_ptr(), c["vp"].data_ptr(), c["table"].data_ptr(),
              c["table"].shape[1], page, c["qsl"].data_ptr(), c["seq_lens"].data_ptr(), out.data_ptr(), c["T"], c["N"],
              Hq, Hkv, D, c["max_q"], 1.0 / math.sqrt(D), 0, num_splits, split_len,
              torch.cuda.current_stream().cuda_stream)


def test_noalloc_entry_point_matches_the_regular_one_twice():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    ops = get_ops(DEV)
    lib = ctypes.CDLL(ops.lib_path)
    lib.ttie_last_error.restype = ctypes.c_char_p
    Hq, Hkv, D, page = 32, 1, 128, 16
    calls = [(1, [(700, 1), (64, 1), (513, 1), (1, 1)], 3, 256),        # decode, three splits
             (2, [(900, 1), (130, 2), (300, 1)], 8, 128)]               # other inputs, other split: stale scratch must not matter
    for seed, seqs, num_splits, split_len in calls:
        c = _case(seed, seqs, Hq, Hkv, D, page)
        ref = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention(c["qkv"], Hq, Hkv, D, c["kp"], c["vp"], c["table"], page, c["qsl"], c["seq_lens"], c["N"],
                            c["max_q"], c["max_kv"], 1.0 / math.sqrt(D), 0, ref, plan=("mma", num_splits, split_len))
        out = torch.full_like(ref, 7.0)
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, c, Hq, Hkv, D, page, num_splits, split_len, out)
        assert rc == 0, lib.ttie_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
        assert torch.isfinite(out).all() and err < TOL, err
    # a single split needs no scratch at all
    c = _case(3, [(40, 40)], Hq, Hkv, D, page)
    ref = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(c["qkv"], Hq, Hkv, D, c["kp"], c["vp"], c["table"], page, c["qsl"], c["seq_lens"], c["N"],
                        c["max_q"], c["max_kv"], 1.0 / math.sqrt(D), 0, ref, plan=("mma", 1, 0))
    out = torch.empty_like(ref)
    assert _call_noalloc(lib, c, Hq, Hkv, D, page, 1, 0, out) == 0
    assert ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item() < TOL


def test_noalloc_entry_point_refuses_what_its_array_cannot_hold():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    ops = get_ops(DEV)
    lib = ctypes.CDLL(ops.lib_path)
    lib.ttie_last_error.restype = ctypes.c_char_p
    Hq, Hkv, D, page = 32, 1, 128, 64
    c = _case(4, [(4096, 1)] * 64, Hq, Hkv, D, page)                  # 64 x 32 x 16 x 130 floats > 4 Mi
    out = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
    rc = _call_noalloc(lib, c, Hq, Hkv, D, page, 16, 256, out)
    assert rc != 0
    msg = lib.ttie_last_error().decode()
    assert "exceed" in msg and "4194304" in msg
