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
    "ttie_add_rmsnorm": [_c_void, _c_void, _c_void, _c_int, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int,
                         _c_float, _c_int, _c_void],
    "ttie_rope_store_partial": [_c_void, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int,
                                _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_rope_table": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ttie_rope_store_vec": [_c_void, _c_ll, _c_void, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void,
                            _c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_skinny_gemm": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_void],
    "ttie_skinny_gemm_tuned": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_void],
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
    "ttie_paged_attention_mma_form": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                      _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
                                      _c_void, _c_int, _c_void],
    "ttie_paged_attention_tc": [_c_void, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, _c_int,
                                _c_void],
    "ttie_gemm_tc": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_gemm_tc_pair": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_sample": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void],
    "ttie_sample_tuned": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void],
}


class KernelError(RuntimeError):
    pass


def _row_bucket(M: int) -> int:
    return 16 if M <= 16 else 32 if M <= 32 else 64


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
        self.num_sms = int(torch.cuda.get_device_properties(self.device).multi_processor_count)   # the plans below are sized for it
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or \
            (lambda index: torch.cuda.current_stream(index).cuda_stream)
        self.attn_target_ctas = 4 * self.num_sms  # decode tiles are small: four CTAs share an SM
        self.attn_cluster_max_rows = 64         # query rows per request (tokens x heads per kv head) up to which the decode form runs
        self.attn_cluster_max_size = 8          # CTAs per cluster (16 is placed on fewer SMs at a time)
        self.attn_cluster_tiles_per_warp = 1    # ... and only while a warp walks at most this many 64-key tiles
        self._cluster_max = {}
        self._mma_per_sm = {}
        self._plans = {}
        self.attn_tc_min_rows = 256             # query rows per request from which the tcgen05 attention kernel is used
        self.skinny_max_rows = 8                # rows up to which the weight-streaming product is the rule (tune_products may hand a shape to the library)
        self._swiglu_choice = {}                # (F, K, row bucket) -> True where the fused tcgen05 gate/up + SwiGLU kernel measured faster
        self._product_choice = {}               # (N, K, row bucket[, "split"]) -> "skinny" | "library" (tune_products; "split": for callers that take partial sums)
        self._skinny_tuned = {}                 # (N, K, row bucket 8 | 16) -> (K range per CTA, form code) where tune_products found a faster form
        self.product_timings = {}               # what tune_products measured: (N, K, rows) -> {"library": ms, "skinny": ms (best form), "skinny_uncut": ms, ...}
        self.lib.ttie_attn_tc_supported.restype = _c_int
        if os.environ.get("TTIE_NVTX", "0") not in ("", "0"):
            self._wrap_in_ranges()
        self._tc_pinned = torch.zeros(2, dtype=torch.int32).pin_memory()       # failure codes of the tcgen05 kernels, written by the device
        self._tc_words = self._tc_pinned.numpy()
        for i, name in enumerate(("ttie_gemm_tc_set_mirror", "ttie_attn_tc_set_mirror")):
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = [_c_void], _c_int
            if fn(self._tc_pinned.data_ptr() + 4 * i):
                raise KernelError(f"{name} failed")
        for name in ("ttie_attn_mma_supported", "ttie_attn_mma_tile_rows", "ttie_attn_cluster_tile_rows", "ttie_attn_cluster_active",
                     "ttie_attn_mma_ctas_per_sm"):
            getattr(self.lib, name).restype = _c_int

    # ------------------------------------------------------------------ helpers
    _RANGED = ("embed", "add_rmsnorm", "rmsnorm_rows", "linear", "linear_swiglu", "swiglu", "rope_table", "rope_store",
               "paged_attention", "sample")

    def _wrap_in_ranges(self):
        """With ``TTIE_NVTX=1`` in the environment every operation below opens an NVTX range of its own name around its
        launches, so a timeline of a step reads op by op (the reference marks the same places with
        ``torch.profiler.record_function`` behind its ``PROFILE_REGIONS`` flag, models/mqa.py:14-18).  Off by
        default: the step's host time is too short to spend on it unasked."""
        push, pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop

        def ranged(name, fn):
            def call(*args, **kwargs):
                push(name)
                try:
                    return fn(*args, **kwargs)
                finally:
                    pop()
            return call

        for name in self._RANGED:
            setattr(self, name, ranged(name, getattr(self, name)))

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.ttie_last_error().decode()}")

    def _stream(self, t: torch.Tensor = None):
        """torch's current stream of the device as a raw handle (asked at every call: a graph capture changes it).
        The direct query is an order of magnitude cheaper than building a ``torch.cuda.Stream`` object, which
        counts on steps that are not replayed from a graph."""
        return self._raw_stream(self._device_index)

    @staticmethod
    def _dt(t: torch.Tensor) -> int:
        try:
            return _DT[t.dtype]
        except KeyError:
            raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None

    # ------------------------------------------------------------------ what the kernels take
    def check_dtype(self, dtype):
        if dtype not in _DT:
            raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)")

    def check_attention(self, dtype, num_heads, num_kv_heads, head_dim, page_size):
        """Raises unless some attention kernel here takes the sizes: the general kernel takes every head size that is
        a multiple of 4 up to 256, any head counts and any page size (the tensor-core kernels cover subsets of that)."""
        self.check_dtype(dtype)
        if head_dim <= 0 or head_dim % 4 or head_dim > 256:
            raise KernelError(f"attention: head size {head_dim} not supported (multiples of 4 up to 256)")
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise KernelError(f"attention: {num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if page_size < 1:
            raise KernelError(f"attention: page size {page_size}")

    def check_norm(self, dtype, dim):
        self.check_dtype(dtype)
        if dim * 4 > 200 * 1024:
            raise KernelError(f"rmsnorm: width {dim} needs {dim * 4} bytes of shared memory (limit 204800)")

    # ------------------------------------------------------------------ ops
    def embed(self, token_ids, table, out):
        T, d = out.shape
        self._check(self.lib.ttie_embed(_ptr(token_ids), _ptr(table), _ptr(out), T, d, table.shape[0],
                                        self._dt(table), self._stream(out)), "embed")
        self.launches += 1

    @staticmethod
    def _delta_args(delta):
        """(delta pointer, partial pointer, S, stride) for a delta that is None, [T, d] in the compute
        dtype, or float32 partial sums [S, T, d]."""
        if delta is None:
            return None, None, 0, 0
        if delta.dim() == 3:
            return None, delta.data_ptr(), delta.shape[0], delta.stride(0)
        return delta.data_ptr(), None, 0, 0

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        R, d = resid.shape
        dp, pp, S, stride = self._delta_args(delta)
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), dp, pp, S, stride, None, _ptr(weight), self._dt(weight),
                                              _ptr(out), R, d, float(eps), self._dt(out), self._stream(out)), "add_rmsnorm")
        self.launches += 1

    def rmsnorm_rows(self, resid, delta, rows, num_rows, weight, eps, out):
        d = resid.shape[1]
        dp, pp, S, stride = self._delta_args(delta)
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), dp, pp, S, stride, _ptr(rows), _ptr(weight), self._dt(weight),
                                              _ptr(out), num_rows, d, float(eps), self._dt(out), self._stream(out)),
                    "rmsnorm_rows")
        self.launches += 1

    # ---- matrix products
    def _skinny_ok(self, x, w, may_split=False):
        """Whether the weight-streaming product takes this product.  ``may_split``: the caller accepts partial sums of a
        K range cut over CTAs; the measured choice for such calls (which may rest on a cut form) is kept apart."""
        M = x.shape[0]
        key = (w.shape[0], w.shape[1], 8 if M <= self.skinny_max_rows else _row_bucket(M)) + (("split",) if may_split else ())
        choice = self._product_choice.get(key)
        if M > self.skinny_max_rows and not (M <= 64 and choice == "skinny"):
            return False
        if M <= self.skinny_max_rows and choice == "library":
            return False
        return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)

    def tune_products(self, weights, iters=8):
        """Which product serves each distinct bfloat16 matrix shape of a model at 8, 16, 32 and 64 rows, by measurement:
        a replayed graph of ``iters`` launches that rotate over the model's matrices of that shape (so that the weights come
        from HBM).  For 9 to 64 rows neither this package's weight-streaming product nor the library's wins at every
        shape (at the Llama-2-7B widths the library is ahead by 10-20 % from 32 rows on; on a narrow, deep matrix such as
        [2048, 16384] it leaves half of the memory bandwidth unused), and the faster one is remembered.  Up to 8 rows the
        weight-streaming product is the rule and is ahead on most shapes, by up to 3x on narrow deep ones; a shape goes to
        the library where that is more than 5 % faster (measured: [10240, 8192] and [8192, 28672] by 9-10 %).  At 8 and
        16 rows the weight-streaming product's own form is measured too - K cut into 1 to 16 ranges over CTAs, one or two
        sets of 16 weight rows per CTA - and a form that beats the rule of thumb (``_kslice``) by 3 % is kept: [4352, 4096]
        at 8 rows takes 7.8 us in 6 ranges with two row sets against 9.1 in 8 ranges with one, [4544, 18176] 28.5 us in 6
        ranges against 38.3 uncut.  Small matrices (under 4 Mi elements) are left alone."""
        groups, launches = {}, self.launches
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.shape[0] * w.shape[1] >= (4 << 20):
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (N, K), ws in groups.items():
            for M in (8, 16, 32, 64):
                if (N, K, M) in self._product_choice:
                    continue
                x = torch.randn(M, K, device=self.device).to(torch.bfloat16)
                if not self._skinny_shape_ok(x, ws[0]):
                    continue

                def measure(kind, form=None, partial_ok=True):
                    self._product_choice[(N, K, M)] = self._product_choice[(N, K, M, "split")] = kind
                    self._skinny_tuned.pop((N, K, M), None)
                    if form is not None:
                        self._skinny_tuned[(N, K, M)] = form
                    return self._graph_time_rotating(lambda i: self.linear(x, ws[i % len(ws)], None, partial_ok=partial_ok), iters)

                def decide(skinny, library):
                    if M == 8:  # up to 8 rows the weight-streaming product is the rule; the library takes a shape only where it is clearly ahead
                        return "library" if library < 0.95 * skinny else "skinny"
                    return "skinny" if skinny < 0.97 * library else "library"

                took = {"library": measure("library"), "skinny_uncut": measure("skinny", partial_ok=False), "skinny": measure("skinny")}
                form = None
                if M <= 16:
                    # up to 16 rows the weight-streaming product's own form is measured as well: one or two sets of 16 weight
                    # rows per CTA, K cut into 1 to 16 ranges
                    for code in (0, 16):
                        for S in (1, 2, 3, 4, 6, 8, 12, 16):
                            kslice = math.ceil(math.ceil(K / S) / 128) * 128
                            if kslice < 256 or math.ceil(K / kslice) != S:
                                continue
                            t = measure("skinny", (kslice, code))
                            if t < 0.97 * took["skinny"]:
                                took["skinny"], form = t, (kslice, code)
                self._skinny_tuned.pop((N, K, M), None)
                if form is not None:
                    self._skinny_tuned[(N, K, M)] = form
                    took["skinny_form"] = {"k_ranges": math.ceil(K / form[0]), "row_sets": 2 if form[1] & 16 else 1}
                # callers that take partial sums of a cut K range, and callers that want the whole sum
                self._product_choice[(N, K, M, "split")] = decide(took["skinny"], took["library"])
                self._product_choice[(N, K, M)] = decide(took["skinny_uncut"], took["library"])
                self.product_timings[(N, K, M)] = took
        self.launches = launches

    @staticmethod
    def _skinny_shape_ok(x, w):
        return x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0

    def _kslice(self, N, K, may_split):
        """K range per CTA of the weight-streaming kernel.  K is split over CTAs (partial sums) when the
        16-row tiles alone are too few to balance the SMs."""
        tiles = math.ceil(N / 16)
        full = math.ceil(K / 128) * 128
        if not may_split or tiles >= 4 * self.num_sms:
            return full
        best, best_eff = full, 0.0
        for S in (1, 2, 3, 4, 6, 8):
            ks = math.ceil(math.ceil(K / S) / 128) * 128
            if ks < 256:
                break
            ctas = tiles * math.ceil(K / ks)
            eff = (ctas / self.num_sms) / math.ceil(ctas / self.num_sms)
            if eff > best_eff + 0.02:
                best, best_eff = ks, eff
        return best

    def linear(self, x, w, bias, out_dtype=None, partial_ok=False):
        """y = x @ w.T (+ bias); x [M, K], w [N, K] -> [M, N].  With ``partial_ok`` the result may
        instead be float32 partial sums [S, M, N] of a K-split product, which ``add_rmsnorm``,
        ``rmsnorm_rows`` and ``rope_store`` accept and add up."""
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.float32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._check(self.lib.ttie_gemm_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, x.stride(0),
                                               w.stride(0), N, self._stream(x)), "gemm_f32")
            self.launches += 1
            return out
        may_split = partial_ok and bias is None and out_dtype is None
        if self._skinny_ok(x, w, may_split):
            tuned = self._skinny_tuned.get((N, K, 8 if M <= 8 else 16)) if (may_split and M <= 16) else None
            kslice, form = tuned if tuned is not None else (self._kslice(N, K, may_split), 0)
            S = math.ceil(K / kslice)
            if S > 1:
                out, epi = torch.empty((S, M, N), dtype=torch.float32, device=x.device), 1
            elif out_dtype == torch.float32:
                out, epi = torch.empty((M, N), dtype=torch.float32, device=x.device), 3
            else:
                out, epi = torch.empty((M, N), dtype=torch.bfloat16, device=x.device), 0
            self._check(self.lib.ttie_skinny_gemm_tuned(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), N,
                                                        M, N, K, kslice, epi, 0, form, self._stream(x)), "skinny_gemm")
            self.launches += 1
            return out
        # bfloat16, many rows: the library product, 32-bit accumulation inside
        if out_dtype == torch.float32:
            out = torch.mm(x, w.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            return out
        if bias is not None:
            return torch.addmm(bias, x, w.t())
        return torch.mm(x, w.t())

    def linear_tc(self, x, w, bias, out_dtype=None, tile_n=256):
        """The tcgen05 / TMA / TMEM product: y = x @ w.T (+ bias) for bfloat16 operands."""
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0),
                                          M, N, K, 1 if out.dtype == torch.float32 else 0, tile_n, self._stream(x)), "gemm_tc")
        self.launches += 1
        return out

    def linear_tc_pair(self, x, w, bias, out_dtype=None):
        """The tcgen05 product on pairs of CTAs (256 x 256 tiles): y = x @ w.T (+ bias) for bfloat16 operands."""
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc_pair(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0),
                                               M, N, K, 1 if out.dtype == torch.float32 else 0, 0, self._stream(x)), "gemm_tc_pair")
        self.launches += 1
        return out

    def linear_swiglu_tc_pair(self, x, w_gu, b_gu, hidden):
        """silu(x @ Wg.T) * (x @ Wu.T) in one kernel: the pair product with the activation in its epilogue."""
        M, K = x.shape
        act = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc_pair(_ptr(x), x.stride(0), _ptr(w_gu), w_gu.stride(0), _ptr(b_gu), _ptr(act), act.stride(0),
                                               M, hidden, K, 0, 1, self._stream(x)), "gemm_tc_pair (SwiGLU)")
        self.launches += 1
        return act

    def tc_error(self) -> int:
        """Error word of the tcgen05 kernels (0 = none; otherwise the code of the first bounded wait that
        ran out: product 1-4, attention 101-110); synchronises the device."""
        g = int(self.lib.ttie_tc_error())
        a = int(self.lib.ttie_attn_tc_error())
        return g or (100 + a if a else 0)

    def check_tc(self):
        """After a point where the host has waited for the device: raises if a bounded wait inside a tcgen05
        kernel ran out since the last check (its result is then not to be trusted).  The kernels also write
        their failure code into two words of pinned host memory, so this costs two loads - it is called
        after every step, graph replays included."""
        if self._tc_words[0] or self._tc_words[1]:
            self._tc_words[:] = 0
            code = self.tc_error() or -1
            raise KernelError(f"a tcgen05 kernel gave up waiting on a barrier (code {code}); its output is invalid")

    def linear_swiglu(self, x, w_gu, b_gu, hidden):
        """silu(x @ Wg.T) * (x @ Wu.T) with w_gu = [Wg; Wu] ([2*hidden, K]) -> [M, hidden]."""
        M, K = x.shape
        act = torch.empty((M, hidden), dtype=x.dtype, device=x.device)
        if self._skinny_ok(x, w_gu) and self._fused_few_rows_wins(x, w_gu, b_gu, hidden):
            return self._linear_swiglu_skinny(x, w_gu, b_gu, hidden, act)
        if M >= 1024 and x.dtype == torch.bfloat16 and self._skinny_shape_ok(x, w_gu) and self._fused_swiglu_wins(x, w_gu, b_gu, hidden):
            return self.linear_swiglu_tc_pair(x, w_gu, b_gu, hidden)
        self.swiglu(self.linear(x, w_gu, b_gu), act)
        return act

    def _linear_swiglu_skinny(self, x, w_gu, b_gu, hidden, act):
        M, K = x.shape
        self._check(self.lib.ttie_skinny_gemm(_ptr(x), x.stride(0), _ptr(w_gu), w_gu.stride(0), _ptr(b_gu), _ptr(act),
                                              hidden, M, hidden, K, math.ceil(K / 128) * 128, 2, hidden,
                                              self._stream(x)), "skinny_gemm_swiglu")
        self.launches += 1
        return act

    def _graph_time_rotating(self, fn, iters=8) -> float:
        """Milliseconds of one replay of a graph of ``iters`` calls ``fn(i)`` (after two plain calls)."""
        for i in range(2):
            fn(i)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        best = None
        for _ in range(3):                                           # the least of three replays
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize(self.device)
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
        return best

    def _graph_time(self, fn, iters=8) -> float:
        """Milliseconds of one replay of a graph of ``iters`` calls of ``fn`` (after two plain calls)."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize(self.device)
        return a.elapsed_time(b)

    def _fused_few_rows_wins(self, x, w_gu, b_gu, hidden) -> bool:
        """Up to 8 rows: whether the weight-streaming product with SwiGLU in its epilogue beats the same product without
        it followed by the activation kernel.  The fused form cannot cut K over CTAs (the activation needs whole sums),
        so it has hidden / 16 CTAs: at the Llama-2-7B widths (688 CTAs) it is 8 % ahead, at a feed-forward width of
        2,048 to 4,096 behind a model width of 4,096 to 8,192 it is 15-40 % behind.  Measured per shape the first time
        it is met outside a graph capture (a step that meets a new batch bucket runs plainly once before it is
        captured), as a replayed graph of eight launches each."""
        key = (hidden, x.shape[1], "few")
        choice = self._swiglu_choice.get(key)
        if choice is None:
            if torch.cuda.is_current_stream_capturing():
                return True
            launches = self.launches
            act = torch.empty((x.shape[0], hidden), dtype=x.dtype, device=x.device)
            took = {"fused": self._graph_time(lambda: self._linear_swiglu_skinny(x, w_gu, b_gu, hidden, act)),
                    "unfused": self._graph_time(lambda: self.swiglu(self.linear(x, w_gu, b_gu), act))}
            self.launches = launches
            choice = self._swiglu_choice[key] = took["fused"] <= 1.03 * took["unfused"]
            self.product_timings[("swiglu",) + key] = took
        return choice

    def _fused_swiglu_wins(self, x, w_gu, b_gu, hidden) -> bool:
        """Whether, for portions of this many rows, the gate/up product with SwiGLU in its epilogue (this package's
        tcgen05 kernel on CTA pairs) is faster than the library's product followed by the activation kernel.  Measured
        the first time a shape and row bucket (1,024 / 2,048 / 4,096 rows and up) is met outside a graph capture: three
        launches of each between events.  At the Llama-2-7B and Falcon-7B widths the two are within 3 % of each other
        at 2,048 rows; below 1,024 rows the pair kernel has too few tiles for the GPU and is not considered."""
        M, K = x.shape
        key = (hidden, K, 4096 if M >= 4096 else 2048 if M >= 2048 else 1024)
        choice = self._swiglu_choice.get(key)
        if choice is None:
            if torch.cuda.is_current_stream_capturing():
                return False
            launches, took = self.launches, {}
            act = torch.empty((M, hidden), dtype=x.dtype, device=x.device)
            for kind, fn in (("library", lambda: self.swiglu(self.linear(x, w_gu, b_gu), act)),
                             ("pair", lambda: self.linear_swiglu_tc_pair(x, w_gu, b_gu, hidden))):
                fn()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(3):
                    fn()
                b.record()
                b.synchronize()
                took[kind] = a.elapsed_time(b)
            self.launches = launches
            choice = self._swiglu_choice[key] = took["pair"] < took["library"]
            self.product_timings[("swiglu",) + key] = took
        return choice

    def swiglu(self, gate_up, out):
        T, F = out.shape
        self._check(self.lib.ttie_swiglu(_ptr(gate_up), _ptr(out), T, F, self._dt(out), self._stream(out)), "swiglu")
        self.launches += 1

    def rope_table(self, positions, inv_freq):
        """cos and sin of pos * inv_freq for every token of the step: float32 [T, D/2, 2]."""
        T, half = positions.shape[0], inv_freq.shape[0]
        cs = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
        self._check(self.lib.ttie_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(cs), T, half, self._stream(cs)), "rope_table")
        self.launches += 1
        return cs

    def rope_store(self, qkv, num_heads, num_kv_heads, head_dim, positions, token_seq, inv_freq, style,
                   k_pages, v_pages, block_table, page_size, write_kv, q_out=None, cs_table=None):
        """Rotates q and k and stores k, v into the pages.  qkv [T, width] is rotated in place; qkv given
        as float32 partial sums [S, T, width] is summed, rotated, and q written to ``q_out`` [T, Hq*D].
        ``cs_table`` (from ``rope_table``) replaces the per-layer sine/cosine evaluation."""
        partial = qkv.dim() == 3
        T = qkv.shape[-2]
        stream = self._stream(qkv)
        vec_ok = head_dim % 4 == 0 and (inv_freq is None or (style == 0 and cs_table is not None)) and \
            (partial or (qkv.stride(0) % 4 == 0 and qkv.stride(1) == 1))
        if vec_ok:
            dst = q_out if partial else qkv
            self._check(self.lib.ttie_rope_store_vec(
                None if partial else _ptr(qkv), 0 if partial else qkv.stride(0), _ptr(qkv) if partial else None,
                qkv.shape[0] if partial else 0, qkv.stride(0) if partial else 0, T, num_heads, num_kv_heads, head_dim,
                _ptr(positions), _ptr(token_seq), None if inv_freq is None else _ptr(cs_table), _ptr(dst), dst.stride(0),
                _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size, k_pages.shape[0],
                1 if write_kv else 0, self._dt(dst), stream), "rope_store_vec")
        elif partial:
            self._check(self.lib.ttie_rope_store_partial(
                _ptr(qkv), qkv.shape[0], qkv.stride(0), T, num_heads, num_kv_heads, head_dim, _ptr(positions), _ptr(token_seq),
                _ptr(inv_freq), int(style), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], page_size, k_pages.shape[0], 1 if write_kv else 0, self._dt(q_out),
                stream), "rope_store_partial")
        else:
            self._check(self.lib.ttie_rope_store(_ptr(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim,
                                                 _ptr(positions), _ptr(token_seq), _ptr(inv_freq), int(style),
                                                 _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                                 page_size, k_pages.shape[0], 1 if write_kv else 0, self._dt(qkv),
                                                 stream), "rope_store")
        self.launches += 1

    def attention_plan(self, dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size=None):
        """Which attention kernel runs and how the key range is split: (kernel, num_splits,
        split_len).  bfloat16 with a head size that is a multiple of 16 up to 128, or 256, runs
        on tensor cores; everything else runs the general float32-arithmetic kernel.  The key
        range is split only when the query rows alone cannot fill the GPU.  Every layer of a step
        asks the same question, so the answers are kept."""
        key = (dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size)
        plan = self._plans.get(key)
        if plan is None:
            if len(self._plans) >= 4096:
                self._plans.clear()
            plan = self._plans[key] = self._attention_plan(*key)
        return plan

    def _attention_plan(self, dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size):
        G = num_heads // num_kv_heads
        rows = max_q_len * G
        if (dtype == torch.bfloat16 and page_size is not None and head_dim > 128
                and self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            return self._tc_wide_plan(num_seqs, num_kv_heads, rows, max_kv_len, max_q_len)
        if (dtype == torch.bfloat16 and page_size is not None and rows >= self.attn_tc_min_rows
                and self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            # prompt portions: the tcgen05 kernel with two query tiles per CTA, uncut, where its CTAs fill half of the GPU
            # or more.  Below that the choice is between that kernel and the one-tile kernel (twice the CTAs), each with the
            # key range uncut or cut, by a cost model fitted to measurements (32 heads of 128; 1 to 8 portions of 128 to
            # 2,048 tokens behind 2,048 to 32,768 keys): waves of one CTA per SM at 3.5 us and 12 ns (one tile) or 17 ns (two)
            # per key, 2 us for the launch, and for cut ranges 3 us and the partial results' way through memory at 4 TB/s.
            # (512 tokens alone: one tile uncut, 14.3 against 18.4 us; the last 512 of 8,192: two tiles in two pieces, 83
            # against 103 one tile uncut and 134 two tiles uncut; the last 128 of 2,048: one tile in four pieces, 18.4
            # against 30.4 two tiles in two.)
            base = num_seqs * num_kv_heads * math.ceil(rows / 256)
            if base > self.num_sms // 2:
                return "tcpp", 1, 0
            return self._portion_pieces(num_seqs * num_kv_heads * rows, head_dim, max_kv_len,
                                        (("tc", num_seqs * num_kv_heads * math.ceil(rows / 128), 0.012), ("tcpp", base, 0.017)),
                                        max_kv_len >= 2 * max_q_len)
        if dtype == torch.bfloat16 and self.lib.ttie_attn_mma_supported(head_dim):
            # few rows per request: the tcgen05 kernel with the key range cut over CTAs where it applies (16 rows and more
            # per kv head, head size 64 or 128) - since it stages only the rows in use and sets itself up while its
            # predecessor finishes it is ahead of the decode form at every context (8 requests x 32 heads: 7.1 against
            # 10.7 us at 100 keys, 8.8 against 10.6 at 1,024, 9.6 against 10.7 at 2,048) -, else the decode form
            plan = self._tc_split_plan(num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size)
            if plan is not None:
                return plan
            plan = self._cluster_plan(num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len)
            if plan is not None:
                return plan
            kernel, tile_rows, unit, min_len = "mma", self.lib.ttie_attn_mma_tile_rows(max_q_len, num_heads, num_kv_heads), 64, 128
        else:
            kernel, tile_rows, unit, min_len = "simt", 32, 32, 32      # (one 32-key tile per CTA where the GPU has room: 10.6 us
                                                                      # against 21 for 200 keys in two pieces of 128)
        base = num_seqs * num_kv_heads * math.ceil(rows / tile_rows)
        if kernel == "mma" and rows <= 64:      # (one row tile per request and kv head: decoded tokens and the like)
            return self._mma_split_plan(base, head_dim, max_q_len, num_heads, num_kv_heads, max_kv_len)
        if base >= self.num_sms or max_kv_len <= min_len:
            return kernel, 1, 0
        # as many splits as fit one wave of resident CTAs, none shorter than min_len keys
        want = max(1, min(self.attn_target_ctas // base, math.ceil(max_kv_len / min_len)))
        split_len = math.ceil(math.ceil(max_kv_len / want) / unit) * unit
        num_splits = math.ceil(max_kv_len / split_len)
        return (kernel, num_splits, split_len) if num_splits > 1 else (kernel, 1, 0)

    def _portion_pieces(self, all_rows, head_dim, max_kv_len, kernels, may_cut):
        """The cheapest of ``kernels`` (name, CTAs per piece, us per key) and cuts of the key range for prompt portions whose
        CTAs fill less than half of the GPU: one wave of CTAs at 3.5 us + the keys of a piece, 2 us for the launch, and for
        a cut range 3 us and the partial results' way through memory at 4 TB/s.  A cut range stays within one wave; a
        portion that is most of its own context (``may_cut`` false) is not cut: behind the diagonal a piece has no work."""
        best, best_cost = (kernels[0][0], 1, 0), None
        for kernel, tiles, per_key in kernels:
            for want in range(1, (min(16, math.ceil(max_kv_len / 128)) if may_cut else 1) + 1):
                split_len = math.ceil(math.ceil(max_kv_len / want) / 128) * 128
                n = math.ceil(max_kv_len / split_len)
                if n != want or (n > 1 and tiles * n > self.num_sms):
                    continue                                         # (a cut range in several waves lost wherever it was measured)
                cost = math.ceil(tiles / self.num_sms) * (3.5 + min(split_len, max_kv_len) * per_key) + 2.0
                if n > 1:
                    cost += 3.0 + all_rows * (n * (4 * head_dim + 8) + 2 * head_dim) / 4e6
                if best_cost is None or cost < best_cost - 1e-9:
                    best, best_cost = ((kernel, n, split_len) if n > 1 else (kernel, 1, 0)), cost
        return best

    def _mma_split_plan(self, base, head_dim, max_q_len, num_heads, num_kv_heads, max_kv_len):
        """Pieces of the key range for the mma.sync tile loop, by a cost model fitted to measurements (head size 128,
        16-row tiles, 8 to 200 requests on 2 and 8 kv heads, 300 to 8,192 keys).  An SM holds a handful of the kernel's
        CTAs (5 at head size 128) and all of them together stream at a fixed rate, so the CTAs run in waves of
        ``resident``: a wave costs about 4.3 us and 74 ns per key of its pieces (58 ns when the wave fills less than a
        third of the GPU: a CTA alone on its SM runs faster), and 769 CTAs take as long as 1,480.  From three waves on the
        waves blur and the cost is proportional to the CTAs.  Merging costs 2 us.  Against picking the pieces by a fixed
        target of CTAs this is 16 % faster on average over those measurements and up to 70 % (24 requests x 8 kv heads at
        300 keys: 12.5 us in 3 pieces against 19.7 uncut; at 2,048 keys 54.6 against 71.4)."""
        key = (head_dim, max_q_len * (num_heads // num_kv_heads) <= 16, max_q_len * (num_heads // num_kv_heads) <= 32)
        per_sm = self._mma_per_sm.get(key)
        if per_sm is None:
            per_sm = self._mma_per_sm[key] = max(1, self.lib.ttie_attn_mma_ctas_per_sm(head_dim, max_q_len, num_heads, num_kv_heads))
        resident = per_sm * self.num_sms
        full_key = 0.0743 * (head_dim + 8) / 136

        def per_key(fill):
            return full_key * (0.78 + max(0.0, min(fill, 0.86) - 0.3) * 0.4)

        best, best_cost = ("mma", 1, 0), None
        shortest = 64 if max_q_len * (num_heads // num_kv_heads) <= 16 else 128      # (32 rows, 16 requests at 2,048 keys: 10.9 us in pieces of 128, 13.6 of 64)
        for want in range(1, min(128, math.ceil(max_kv_len / shortest)) + 1):
            split_len = math.ceil(math.ceil(max_kv_len / want) / 64) * 64
            n = math.ceil(max_kv_len / split_len)
            if n != want:
                continue
            ctas, keys = base * n, min(split_len, max_kv_len)
            if ctas >= 3 * resident:
                cost = ctas / resident * (4.3 + keys * full_key)
            else:
                whole, rest = divmod(ctas, resident)
                cost = whole * (4.3 + keys * full_key) + ((4.3 + keys * per_key(rest / resident)) if rest else 0.0)
            cost += 2.0 if n > 1 else 0.0
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = (("mma", n, split_len) if n > 1 else ("mma", 1, 0)), cost
        return best

    def _tc_wide_plan(self, num_seqs, num_kv_heads, rows, max_kv_len, max_q_len):
        """Head size 256: every step takes the prompt-portion tcgen05 kernel with one 128-row tile per CTA.  Steps of few
        rows (decoded tokens) have their key range cut by the cost model of the one-tile decode kernel, at 20 ns per key
        (8 heads on one kv head, 2 requests at 1,024 keys: 9.3 us in 8 pieces of 128 against 11.5 in 4; 96 requests at
        8,192 keys: 132 us in 3 pieces against 153 uncut).  Portions whose row tiles fill less than half of the GPU are cut
        by the portions' cost model at 21 ns per key (512 tokens behind 2,048 keys: 25.5 us in 4 pieces against 33.0 in 2)."""
        base = num_seqs * num_kv_heads * math.ceil(rows / 128)
        if rows <= 128:
            return self._one_per_sm_pieces("tcpp", base, max_kv_len, 0.020, waves_min_keys=640)
        if base > self.num_sms // 2:
            return "tcpp", 1, 0
        return self._portion_pieces(num_seqs * num_kv_heads * rows, 256, max_kv_len, (("tcpp", base, 0.021),),
                                    max_kv_len >= 2 * max_q_len)

    def _tc_split_plan(self, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size):
        """The tcgen05 kernel for steps with few query rows per request: the key range of every request is cut into
        pieces, one CTA each (the kernel takes a whole SM), and the merge kernel adds the pieces.  None where the head
        or page size is not the kernel's, the rows exceed one 128-row tile, or there are so few rows per kv head and so
        many requests that the mma.sync kernel's 16-row tiles waste less."""
        rows = max_q_len * (num_heads // num_kv_heads)
        base = num_seqs * num_kv_heads
        if (page_size is None or rows > 128 or head_dim > 128
                or not self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            return None
        # 16 rows or fewer fill an eighth of the kernel's row tile: it still wins while the GPU is far from full (2 requests
        # x 8 kv heads at 300 keys: 8.0 us against 10.0 for the decode form), the tile loop's 16-row CTAs win beyond (32
        # requests x 2 kv heads at 2,048 keys: 19.6 us against 22.9)
        if rows <= 16 and (base > 32 or base * max_kv_len > (32768 if rows == 16 else 16384)):
            return None
        if rows < 32 and base > self.num_sms:
            return None              # (40 heads on 2 kv heads, 96 requests at 2,048 keys: 72.7 us uncut against 56.8 for the tile loop)
        if base > self.num_sms and max_kv_len < 1024:
            return None              # more requests than SMs with short contexts: the tile loop is ahead (measured at 512 keys)
        # The number of pieces by a cost model fitted to measurements (32 heads of 128 and 71 heads of 64 on one kv head, 2
        # to 200 requests, 300 to 8,192 keys).  CTAs run in waves of one per SM; a wave costs about 3.5 us to set up and
        # finish and 12.5 ns per key (more with more than 64 query rows); the launch costs 2 us, merging the pieces 2
        # (5.5 with more than 32 pieces, which the general merge kernel adds up).  So few requests get pieces down to 128
        # keys (2 requests at 1,024 keys: 7.7 us in 8 pieces against 8.9 in 4), and where the requests alone leave the
        # last wave half empty the key range is cut although every SM has a CTA already (96 requests at 8,192 keys: 81 us
        # in 3 pieces against 99 uncut; 200 requests: 165 in 2 against 194) - but into pieces of 1,280 keys at least:
        # shorter ones in several waves lose (200 requests at 1,024 keys: 43.6 us in 2 pieces against 34.8 uncut).
        return self._one_per_sm_pieces("tc", base, max_kv_len, 0.0125 * (1.15 if rows > 64 else 1.0))

    def _one_per_sm_pieces(self, kernel, base, max_kv_len, per_key, waves_min_keys=1280):
        """The cheapest cut of ``max_kv_len`` keys into pieces of a multiple of 128 keys for a kernel that runs one CTA per
        SM, ``base`` CTAs per piece: waves of ``num_sms`` CTAs at 3.5 us + ``per_key`` us per key of a piece, 2 us for the
        launch, 2 for merging (5.5 with more than 32 pieces); pieces that run in several waves hold ``waves_min_keys`` or more."""
        best, best_cost = (kernel, 1, 0), None
        for want in range(1, min(256, math.ceil(max_kv_len / 128)) + 1):
            split_len = math.ceil(math.ceil(max_kv_len / want) / 128) * 128
            n = math.ceil(max_kv_len / split_len)
            if n != want or (n > 1 and base * n > self.num_sms and split_len < waves_min_keys):
                continue                                             # (the same cut as a smaller count; short pieces in several waves)
            cost = (math.ceil(base * n / self.num_sms) * (3.5 + min(split_len, max_kv_len) * per_key) + 2.0
                    + (0.0 if n == 1 else 2.0 if n <= 32 else 5.5))
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = ((kernel, n, split_len) if n > 1 else (kernel, 1, 0)), cost
        return best

    def _clusters_active(self, head_dim, max_q_len, num_heads, num_kv_heads, groups, size):
        key = (head_dim, max_q_len * (num_heads // num_kv_heads) <= 16, groups, size)
        if key not in self._cluster_max:
            self._cluster_max[key] = self.lib.ttie_attn_cluster_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, size)
        return self._cluster_max[key]

    def _cluster_plan(self, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len):
        """The decode form ("mma_c4" / "mma_c2": one thread-block cluster per request and kv head, 4 or 2 key
        groups per CTA) for steps whose requests bring few query rows: (kernel, cluster size, keys per CTA),
        or None where the tile loop serves better (many rows; a long context with too few requests to
        fill the GPU with clusters)."""
        rows = max_q_len * (num_heads // num_kv_heads)
        if rows > self.attn_cluster_max_rows:
            return None
        tile_rows = self.lib.ttie_attn_cluster_tile_rows(max_q_len, num_heads, num_kv_heads)
        base = num_seqs * num_kv_heads * math.ceil(rows / tile_rows)
        groups = 4 if max_kv_len > 128 else 2
        want = max(1, min(self.attn_cluster_max_size, (self.num_sms + base // 2) // base, math.ceil(max_kv_len / (64 * groups))))
        C = 1 << (want.bit_length() - 1)                       # a power of two
        while C > 1 and self._clusters_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, C) < base:
            C //= 2                                            # all clusters of the step have to run at once
        if self._clusters_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, C) < 1:
            return None
        split_len = math.ceil(math.ceil(max_kv_len / C) / 64) * 64
        # measured: the form pays while a warp walks few tiles; beyond that the tile loop with more, smaller CTAs
        # and a merge kernel is as fast or faster
        if split_len > self.attn_cluster_tiles_per_warp * 64 * groups:
            return None
        return f"mma_c{groups}", C, split_len

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table, page_size,
                        query_start_loc, seq_lens, num_seqs, max_q_len, max_kv_len, scale, window, out,
                        plan=None):
        T = qkv.shape[0]
        if max_kv_len > block_table.shape[1] * page_size:
            raise KernelError(f"paged_attention: a block table of {block_table.shape[1]} pages of {page_size} keys cannot cover {max_kv_len} keys")
        kernel, num_splits, split_len = plan if plan is not None else self.attention_plan(
            qkv.dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size)
        if kernel in ("tc", "tcpp"):
            scratch = None
            if num_splits > 1:
                scratch = torch.empty((T * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
            self._check(self.lib.ttie_paged_attention_tc(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table),
                block_table.shape[1], page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads,
                num_kv_heads, head_dim, max_q_len, float(scale), int(window), num_splits, split_len, _ptr(scratch),
                1 if kernel == "tcpp" else 0, self._stream(qkv)), "paged_attention_tc")
            self.launches += 2 if num_splits > 1 else 1
            return
        form = {"mma": 0, "mma_c2": 2, "mma_c4": 4}.get(kernel)
        scratch = None
        if num_splits > 1 and not form:
            scratch = torch.empty((T * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
        if form is not None:
            self._check(self.lib.ttie_paged_attention_mma_form(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), int(window), num_splits, split_len, _ptr(scratch),
                form, self._stream(qkv)), "paged_attention_mma")
            self.launches += 2 if (num_splits > 1 and not form) else 1
            return
        else:
            self._check(self.lib.ttie_paged_attention(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), int(window), num_splits, split_len, _ptr(scratch),
                self._dt(qkv), self._stream(qkv)), "paged_attention")
        self.launches += 2 if num_splits > 1 else 1

    def sample(self, logits, slot_ids, state, out, probs_out=None, ctas_per_row=0):
        """``ctas_per_row``: 0 = chosen from the vocabulary's size; 1, 2, 4 or 8 CTAs (a cluster) share a row."""
        R, V = logits.shape
        self._check(self.lib.ttie_sample_tuned(_ptr(logits), R, V, _ptr(slot_ids), _ptr(state), _ptr(out), _ptr(probs_out),
                                               int(ctas_per_row), self._stream(logits)), "sample")
        self.launches += 1


_OPS = {}


def get_ops(device="cuda:0") -> CudaOps:
    """The kernel library for ``device``; raises if it cannot be had."""
    key = str(torch.device(device))
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
