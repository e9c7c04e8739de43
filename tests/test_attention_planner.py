"""The attention planners on the host, with stand-ins for the few answers they ask of the kernel library: whatever the
step, a plan names a kernel that takes the head size, its pieces cover the key range with none left empty, piece lengths
are whole tiles of the kernel, cut ranges that would run in several waves keep long pieces, and the same question gets
the same answer.  (Which plan is the fastest is measured on the GPU; these are the properties every plan must have.)"""
import math
import random

import torch

from tiny_transformer_inference_engine_b200.ops import CudaOps


class FakeLibrary:
    """Answers of the kernel library that the planners use, as on a B200."""

    @staticmethod
    def ttie_attn_tc_supported(head_dim, page_size):
        return int(head_dim in (64, 128, 256) and 8 <= page_size <= 256 and page_size & (page_size - 1) == 0)

    @staticmethod
    def ttie_attn_mma_supported(head_dim):
        return int(head_dim % 16 == 0 and 16 <= head_dim <= 128)

    @staticmethod
    def ttie_attn_mma_tile_rows(max_q_len, heads, kv_heads):
        rows = max_q_len * (heads // kv_heads)
        return 16 if rows <= 16 else 32 if rows <= 32 else 64

    @staticmethod
    def ttie_attn_cluster_tile_rows(max_q_len, heads, kv_heads):
        return 16 if max_q_len * (heads // kv_heads) <= 16 else 32

    @staticmethod
    def ttie_attn_cluster_active(head_dim, max_q_len, heads, kv_heads, groups, size):
        return 148 // size if size <= 8 else 7

    @staticmethod
    def ttie_attn_mma_ctas_per_sm(head_dim, max_q_len, heads, kv_heads):
        rows = max_q_len * (heads // kv_heads)
        return 2 if rows > 32 else max(1, 640 // (head_dim + 8))


def planner():
    ops = CudaOps.__new__(CudaOps)
    ops.lib, ops.num_sms = FakeLibrary(), 148
    ops.attn_target_ctas, ops.attn_cluster_max_rows, ops.attn_cluster_max_size, ops.attn_cluster_tiles_per_warp = 592, 64, 8, 1
    ops.attn_tc_min_rows = 256
    ops._cluster_max, ops._mma_per_sm, ops._plans = {}, {}, {}
    return ops


TILE = {"tc": 128, "tcpp": 128, "mma": 64, "simt": 32}


def check(plan, dtype, seqs, heads, kv_heads, head_dim, q_len, kv_len, page):
    kernel, n, split_len = plan
    where = f"{plan} for {seqs} requests x {heads}/{kv_heads} heads of {head_dim}, {q_len} tokens behind {kv_len} keys, pages of {page}"
    if kernel.startswith("mma_c"):                                   # the decode form: (kernel, cluster size, keys per CTA)
        assert dtype == torch.bfloat16 and FakeLibrary.ttie_attn_mma_supported(head_dim), where
        assert n & (n - 1) == 0 and 1 <= n <= 8 and split_len % 64 == 0 and n * split_len >= kv_len, where
        return
    assert kernel in TILE, where
    if kernel in ("tc", "tcpp"):
        assert dtype == torch.bfloat16 and FakeLibrary.ttie_attn_tc_supported(head_dim, page), where
        assert kernel == "tcpp" or head_dim <= 128, where
    if kernel == "mma":
        assert dtype == torch.bfloat16 and FakeLibrary.ttie_attn_mma_supported(head_dim), where
    if n == 1:
        assert split_len == 0, where
        return
    assert split_len % TILE[kernel] == 0 and split_len > 0, where
    assert n * split_len >= kv_len > (n - 1) * split_len, where       # the pieces cover the keys and the last one is not empty


def test_every_plan_is_sound():
    ops, rng = planner(), random.Random(4)
    for _ in range(4000):
        dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float32])
        head_dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 256])
        kv_heads = rng.choice([1, 1, 1, 2, 4, 8])
        heads = kv_heads * rng.choice([1, 2, 4, 8, 16, 20, 32, 71])
        seqs = rng.choice([1, 2, 3, 8, 16, 33, 64, 100, 256, 700])
        q_len = rng.choice([1, 1, 1, 2, 7, 64, 512, 2048])
        kv_len = q_len - 1 + rng.choice([1, 5, 64, 100, 300, 1024, 4096, 8192, 40000, 131072])
        page = rng.choice([8, 16, 64, 128, None]) if head_dim in (64, 128, 256) else rng.choice([5, 16, 64])
        args = (dtype, seqs, heads, kv_heads, head_dim, q_len, kv_len, page)
        plan = ops.attention_plan(*args)
        check(plan, *args)
        assert ops.attention_plan(*args) is plan                     # kept, not planned again


def test_cut_ranges_in_several_waves_keep_long_pieces():
    ops = planner()
    for seqs in (1, 8, 24, 64, 96, 128, 200, 256, 1000):
        for kv_len in (300, 1024, 4096, 8192, 32768, 131072):
            plan = ops.attention_plan(torch.bfloat16, seqs, 32, 1, 128, 1, kv_len, 64)
            if plan[0] != "tc" or plan[1] == 1:
                continue
            _, n, split_len = plan
            assert seqs * n <= 148 or split_len >= 1280, plan
            assert n <= 256


def test_few_rows_per_kv_head_leave_the_tensor_memory_kernel_when_the_gpu_fills():
    ops = planner()
    assert ops.attention_plan(torch.bfloat16, 2, 32, 8, 128, 1, 300, 64)[0] == "tc"           # 4 rows, 16 pairs, 300 keys
    assert ops.attention_plan(torch.bfloat16, 64, 32, 8, 128, 1, 4096, 64)[0] == "mma"        # 512 pairs
    assert ops.attention_plan(torch.bfloat16, 96, 40, 2, 128, 1, 2048, 64)[0] == "mma"        # 20 rows, 192 pairs
    assert ops.attention_plan(torch.bfloat16, 96, 32, 1, 128, 1, 2048, 64)[0] == "tc"         # 32 rows: stays


def test_portions_are_cut_within_one_wave_and_only_behind_a_context():
    ops = planner()
    for seqs in (1, 2, 4):
        for q_len in (128, 256, 512, 1024):
            for kv_len in (q_len, 2 * q_len - 1, 2048, 8192, 32768):
                if kv_len < q_len:
                    continue
                for heads, head_dim in ((32, 128), (8, 256)):
                    kernel, n, split_len = ops.attention_plan(torch.bfloat16, seqs, heads, 1, head_dim, q_len, kv_len, 64)
                    rows = q_len * heads
                    tiles = seqs * math.ceil(rows / (256 if kernel == "tcpp" and head_dim <= 128 else 128))
                    if kv_len < 2 * q_len:
                        assert n == 1, (kernel, n, split_len)
                    if n > 1:
                        assert tiles * n <= 148, (seqs, q_len, kv_len, heads, head_dim, kernel, n)
