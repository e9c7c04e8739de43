"""The kernels of the step, as Python calls on torch tensors.

``get_ops(device)`` loads the compiled sm_100a library (building it first if it is missing
or stale) and returns the one ``CudaOps`` object every part calls.  There is no other
implementation behind these calls: without a CUDA device or without the library they raise.
Every call launches on torch's current stream of the tensors' device and returns at once.

Matrix products of the bfloat16 path go to the library product (cuBLAS through
``torch.mm``), as the reference's ``nn.Linear`` layers do (models/mqa.py:123-126,
models/mlp.py:20-22); the float32 path uses this package's own FFMA kernel so that no
reduced-precision matrix mode can slip in.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_c_int, _c_ll, _c_float, _c_void = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "ttie_embed": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_add_rmsnorm": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ttie_swiglu": [_c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ttie_rope_store": [_c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void,
                        _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_gemm_f32": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_paged_attention": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
                             _c_void, _c_int, _c_void],
    "ttie_paged_attention_mma": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
                                 _c_void, _c_void],
    "ttie_sample": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void],
}

NUM_SMS = 148


class KernelError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine computes only with its sm_100a kernels "
                              "(there is no CPU path)")
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernel library is built for sm_100a (B200); device reports sm_{major}{minor}")
        path = _build.build()
        self.lib_path = path
        self.lib = ctypes.CDLL(path)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = argtypes, _c_int
        self.lib.ttie_last_error.restype = ctypes.c_char_p
        self.launches = 0                     # kernels of this library launched so far
        self.attn_target_ctas = 2 * NUM_SMS
        for name in ("ttie_attn_mma_supported", "ttie_attn_mma_tile_rows"):
            getattr(self.lib, name).restype = _c_int

    # ------------------------------------------------------------------ helpers
    def _check(self, rc: int, what: str):
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.ttie_last_error().decode()}")

    @staticmethod
    def _stream(t: torch.Tensor):
        return torch.cuda.current_stream(t.device).cuda_stream

    @staticmethod
    def _dt(t: torch.Tensor) -> int:
        try:
            return _DT[t.dtype]
        except KeyError:
            raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None

    # ------------------------------------------------------------------ ops
    def embed(self, token_ids, table, out):
        T, d = out.shape
        self._check(self.lib.ttie_embed(_ptr(token_ids), _ptr(table), _ptr(out), T, d, table.shape[0],
                                        self._dt(table), self._stream(out)), "embed")
        self.launches += 1

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        R, d = resid.shape
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), _ptr(delta), None, _ptr(weight), self._dt(weight),
                                              _ptr(out), R, d, float(eps), self._dt(out), self._stream(out)), "add_rmsnorm")
        self.launches += 1

    def rmsnorm_rows(self, resid, delta, rows, num_rows, weight, eps, out):
        d = resid.shape[1]
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), self._dt(weight),
                                              _ptr(out), num_rows, d, float(eps), self._dt(out), self._stream(out)),
                    "rmsnorm_rows")
        self.launches += 1

    def linear(self, x, w, bias, out_dtype=None):
        """y = x @ w.T (+ bias); x [M, K], w [N, K] -> [M, N]."""
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.float32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._check(self.lib.ttie_gemm_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, x.stride(0),
                                               w.stride(0), N, self._stream(x)), "gemm_f32")
            self.launches += 1
            return out
        # bfloat16: the library product, 32-bit accumulation inside
        if out_dtype == torch.float32:
            out = torch.mm(x, w.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            return out
        if bias is not None:
            return torch.addmm(bias, x, w.t())
        return torch.mm(x, w.t())

    def swiglu(self, gate_up, out):
        T, F = out.shape
        self._check(self.lib.ttie_swiglu(_ptr(gate_up), _ptr(out), T, F, self._dt(out), self._stream(out)), "swiglu")
        self.launches += 1

    def rope_store(self, qkv, num_heads, num_kv_heads, head_dim, positions, token_seq, inv_freq, style,
                   k_pages, v_pages, block_table, page_size, write_kv):
        T = qkv.shape[0]
        self._check(self.lib.ttie_rope_store(_ptr(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim,
                                             _ptr(positions), _ptr(token_seq), _ptr(inv_freq), int(style),
                                             _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                             page_size, k_pages.shape[0], 1 if write_kv else 0, self._dt(qkv),
                                             self._stream(qkv)), "rope_store")
        self.launches += 1

    def attention_plan(self, dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len):
        """Which attention kernel runs and how the key range is split: (kernel, num_splits,
        split_len).  bfloat16 with a head size that is a multiple of 16 up to 128 runs on
        tensor cores; everything else runs the general float32-arithmetic kernel.  The key
        range is split only when the query rows alone cannot fill the GPU."""
        G = num_heads // num_kv_heads
        rows = max_q_len * G
        if dtype == torch.bfloat16 and self.lib.ttie_attn_mma_supported(head_dim):
            kernel, tile_rows, unit, min_len = "mma", self.lib.ttie_attn_mma_tile_rows(max_q_len, num_heads, num_kv_heads), 64, 256
        else:
            kernel, tile_rows, unit, min_len = "simt", 32, 32, 128
        base = num_seqs * num_kv_heads * math.ceil(rows / tile_rows)
        if base >= NUM_SMS or max_kv_len <= min_len:
            return kernel, 1, 0
        want = min(math.ceil(self.attn_target_ctas / base), math.ceil(max_kv_len / min_len))
        split_len = math.ceil(math.ceil(max_kv_len / want) / unit) * unit
        num_splits = math.ceil(max_kv_len / split_len)
        return (kernel, num_splits, split_len) if num_splits > 1 else (kernel, 1, 0)

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table, page_size,
                        query_start_loc, seq_lens, num_seqs, max_q_len, max_kv_len, scale, window, out,
                        plan=None):
        T = qkv.shape[0]
        kernel, num_splits, split_len = plan if plan is not None else self.attention_plan(
            qkv.dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len)
        scratch = None
        if num_splits > 1:
            scratch = torch.empty((T * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
        if kernel == "mma":
            self._check(self.lib.ttie_paged_attention_mma(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), int(window), num_splits, split_len, _ptr(scratch),
                self._stream(qkv)), "paged_attention_mma")
        else:
            self._check(self.lib.ttie_paged_attention(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), int(window), num_splits, split_len, _ptr(scratch),
                self._dt(qkv), self._stream(qkv)), "paged_attention")
        self.launches += 2 if num_splits > 1 else 1

    def sample(self, logits, slot_ids, state, out, probs_out=None):
        R, V = logits.shape
        self._check(self.lib.ttie_sample(_ptr(logits), R, V, _ptr(slot_ids), _ptr(state), _ptr(out), _ptr(probs_out),
                                         self._stream(logits)), "sample")
        self.launches += 1


_OPS = {}


def get_ops(device="cuda:0") -> CudaOps:
    """The kernel library for ``device``; raises if it cannot be had."""
    key = str(torch.device(device))
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
