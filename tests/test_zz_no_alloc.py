"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of the library cannot allocate device memory at the time they need attention computed
(all memory already handed to their own pools, another runtime's allocator in charge, or a loop
in which an allocation's latency is not acceptable).  For them the library keeps the split-key
scratch in a device array of its own.  This test calls that entry point twice in a row, with
different inputs, and compares each result with the regular entry point's (which gets its scratch
from the caller) and with a float32 computation of the same attention, within the tolerance the
other attention tests use; it checks that the device's free memory (as the driver reports it, so an
allocation by any route would show) is the same after the calls as before; and that a size beyond
the library's array is refused with a message.  The file is named to be collected last.
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
    # the same attention in float32 on the host: the expectation that owes nothing to the library
    from plain_ops import PlainOps
    exp = torch.empty(T, Hq * D)
    PlainOps().paged_attention(qkv, Hq, Hkv, D, kp, vp, table, page, torch.tensor(qsl, dtype=torch.int32),
                               torch.tensor([L for L, _ in seqs], dtype=torch.int32), N, max(n for _, n in seqs),
                               max(L for L, _ in seqs), 1.0 / math.sqrt(D), 0, exp)
    return dict(qkv=qkv.to(DEV), kp=kp.to(DEV), vp=vp.to(DEV), table=table.to(DEV), exp=exp,
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
    # a first call of each shape up front (the first call on a device also looks up the array's address), so that
    # what the driver has to load or set up once is not mistaken for an allocation below
    cases = [_case(seed, seqs, Hq, Hkv, D, page) for seed, seqs, _, _ in calls]
    for c, (_, _, num_splits, split_len) in zip(cases, calls):
        warm = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
        assert _call_noalloc(lib, c, Hq, Hkv, D, page, num_splits, split_len, warm) == 0, lib.ttie_last_error().decode()
    torch.cuda.synchronize()
    for c, (_, _, num_splits, split_len) in zip(cases, calls):
        ref = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention(c["qkv"], Hq, Hkv, D, c["kp"], c["vp"], c["table"], page, c["qsl"], c["seq_lens"], c["N"],
                            c["max_q"], c["max_kv"], 1.0 / math.sqrt(D), 0, ref, plan=("mma", num_splits, split_len))
        out = torch.full_like(ref, 7.0)
        torch.cuda.synchronize()
        for attempt in range(3):                                        # (the GPU's free memory is device-wide: look again if it moved)
            torch_before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
            rc = _call_noalloc(lib, c, Hq, Hkv, D, page, num_splits, split_len, out)
            assert rc == 0, lib.ttie_last_error().decode()
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
            assert torch.cuda.memory_allocated() == torch_before
            if free_after >= free_before:
                break
        assert free_after >= free_before, (free_before, free_after)     # no allocation by any route: the driver's own count
        err = ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
        assert torch.isfinite(out).all() and err < TOL, err
        err32 = ((out.float().cpu() - c["exp"]).abs().max() / c["exp"].abs().max()).item()
        assert err32 < TOL, err32                                       # and against float32 on the host
    # a single split needs no scratch at all
    c = _case(3, [(40, 40)], Hq, Hkv, D, page)
    ref = torch.empty(c["T"], Hq * D, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(c["qkv"], Hq, Hkv, D, c["kp"], c["vp"], c["table"], page, c["qsl"], c["seq_lens"], c["N"],
                        c["max_q"], c["max_kv"], 1.0 / math.sqrt(D), 0, ref, plan=("mma", 1, 0))
    out = torch.empty_like(ref)
    assert _call_noalloc(lib, c, Hq, Hkv, D, page, 1, 0, out) == 0
    assert ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item() < TOL
    torch.cuda.synchronize()
    assert ((out.float().cpu() - c["exp"]).abs().max() / c["exp"].abs().max()).item() < TOL


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
