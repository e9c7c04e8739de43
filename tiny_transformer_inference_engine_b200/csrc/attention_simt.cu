// Paged causal attention, general form: any mix of prompt portions and single decoded tokens,
// any number of heads and kv heads, head sizes that are multiples of 4 up to 256, any page
// size, optional window, float32 or bfloat16 storage with float32 arithmetic throughout
// (scores, running maximum and sum, output accumulators; expf, not a fast approximation).
// It is the attention of the float32 path and the fallback of the bfloat16 path.
//
// Mask and scale as kernels/pagedattn/pagedattn.cu:196-207,256 of the reference: a request
// with kv_len keys and q_len new tokens has ctx = kv_len - q_len; query row r sits at position
// p = ctx + r and sees keys j <= p (and j > p - window if a window is set); scores are
// (q.k) * scale.  Keys are found through the block table: page = table[j / page_size].
//
// Work split: one CTA = one (request, kv head, tile of 32 query rows) x one split of the key
// range; a query row is a (token, head of the kv head's group) pair, so with multi-query
// attention all heads of a token share each key/value tile loaded into shared memory.  With
// more than one split the CTAs leave unnormalised partial outputs and (max, sum) pairs in
// scratch memory and a second kernel merges them.
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {
constexpr int WARPS = 8, RPW = 4, ROWS = WARPS * RPW, BK = 32;

struct AttnParams {
    const void* q; long long q_stride;
    const void* k_pages; const void* v_pages;
    const int* block_table; int table_width; int page_size;
    const int* qsl; const int* seq_lens;
    void* out;
    int num_seqs, Hq, Hkv, D;
    float scale; int window;
    int row_tiles;                 // tiles of ROWS query rows per (request, kv head)
    int num_splits, split_len;
    float* ws_o; float* ws_ml;     // [T*Hq, num_splits, D] and [T*Hq, num_splits, 2]
};

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int DPL>
__global__ void __launch_bounds__(WARPS * 32)
paged_attn_simt_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.D, G = p.Hq / p.Hkv, KS = D + 4;
    float* Qs = smem;                       // [ROWS][D]
    float* Ks = Qs + ROWS * D;              // [BK][D+4]
    float* Vs = Ks + BK * KS;               // [BK][D+4]

    int tile = blockIdx.x;
    const int split = blockIdx.y;
    const int rt = tile % p.row_tiles; tile /= p.row_tiles;
    const int kvh = tile % p.Hkv;
    const int seq = tile / p.Hkv;
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G;
    const int row0 = rt * ROWS;
    if (row0 >= nrows) return;
    const int ctx = kv_len - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int tok_lo = row0 / G;
    const int tok_hi = (min(nrows, row0 + ROWS) - 1) / G;
    int k_hi = ctx + tok_hi + 1;
    int k_lo = p.window > 0 ? max(0, ctx + tok_lo - p.window + 1) : 0;
    if (p.num_splits > 1) {
        const int piece = piece_len(kv_len, p.num_splits, p.split_len, BK);
        k_lo = max(k_lo, split * piece);
        k_hi = min(k_hi, (split + 1) * piece);
    }

    // per-row state of this warp's rows
    float m[RPW], l[RPW], o[RPW][DPL];
    int pos[RPW], lo[RPW];
    bool valid[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int row = row0 + warp * RPW + r;
        valid[r] = row < nrows;
        const int tok = valid[r] ? row / G : 0;
        pos[r] = ctx + tok;
        lo[r] = p.window > 0 ? max(0, pos[r] - p.window + 1) : 0;
        m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[r][i] = 0.f;
    }

    if (k_lo < k_hi) {
        const T* qp = (const T*)p.q;
        for (int idx = threadIdx.x; idx < ROWS * D; idx += blockDim.x) {
            const int r = idx / D, d = idx - r * D;
            const int row = row0 + r;
            float v = 0.f;
            if (row < nrows) {
                const int tok = row / G, g = row - tok * G;
                v = to_f32<T>(qp[(size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + d]);
            }
            Qs[idx] = v;
        }
        const T* kp = (const T*)p.k_pages;
        const T* vp = (const T*)p.v_pages;
        const int* table = p.block_table + (size_t)seq * p.table_width;

        for (int kt = k_lo; kt < k_hi; kt += BK) {
            __syncthreads();
            // four consecutive elements of a key and of a value per step (head sizes are multiples of 4): one page look-up
            // and one 16-byte (float32) or 8-byte (bfloat16) load of each
            const int D4 = D >> 2;
            for (int idx = threadIdx.x; idx < BK * D4; idx += blockDim.x) {
                const int j = idx / D4, d = (idx - j * D4) << 2;
                const int key = kt + j;
                float4 kval = make_float4(0.f, 0.f, 0.f, 0.f), vval = kval;
                if (key < k_hi) {
                    const int pg = key / p.page_size;
                    const int page = pg < p.table_width ? table[pg] : 0;         // (a table that is too short: the scratch page, not a wild read)
                    const int off = key - pg * p.page_size;
                    const size_t src = (((size_t)page * p.Hkv + kvh) * p.page_size + off) * D + d;
                    kval = load4(kp + src); vval = load4(vp + src);
                }
                *reinterpret_cast<float4*>(Ks + j * KS + d) = kval;
                *reinterpret_cast<float4*>(Vs + j * KS + d) = vval;
            }
            __syncthreads();

            const int key = kt + lane;
            float s[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) s[r] = 0.f;
            const float4* k4 = reinterpret_cast<const float4*>(Ks + lane * KS);
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float4 kv = k4[d4];
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    const float4 qv = reinterpret_cast<const float4*>(Qs + (warp * RPW + r) * D)[d4];
                    s[r] = fmaf(qv.x, kv.x, s[r]); s[r] = fmaf(qv.y, kv.y, s[r]);
                    s[r] = fmaf(qv.z, kv.z, s[r]); s[r] = fmaf(qv.w, kv.w, s[r]);
                }
            }
            float pr[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const bool vis = valid[r] && key < k_hi && key <= pos[r] && key >= lo[r];
                const float sc = vis ? s[r] * p.scale : -INFINITY;
                const float m_new = fmaxf(m[r], warp_max(sc));
                const float alpha = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
                pr[r] = vis ? expf(sc - m_new) : 0.f;
                l[r] = l[r] * alpha + warp_sum(pr[r]);
                m[r] = m_new;
#pragma unroll
                for (int i = 0; i < DPL; ++i) o[r][i] *= alpha;
            }
            const int nk = min(BK, k_hi - kt);
            for (int j = 0; j < nk; ++j) {
                float vv[DPL];
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int d = lane + 32 * i;
                    vv[i] = d < D ? Vs[j * KS + d] : 0.f;
                }
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    const float pj = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
                    for (int i = 0; i < DPL; ++i) o[r][i] = fmaf(pj, vv[i], o[r][i]);
                }
            }
        }
    }

    // results
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        if (!valid[r]) continue;
        const int row = row0 + warp * RPW + r;
        const int tok = row / G, g = row - tok * G;
        const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
        if (p.num_splits == 1) {
            T* op = (T*)p.out + grow * D;
            const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) op[d] = from_f32<T>(o[r][i] * inv);
            }
        } else {
            float* wo = p.ws_o + (grow * p.num_splits + split) * D;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) wo[d] = o[r][i];
            }
            if (lane == 0) {
                float* ml = p.ws_ml + (grow * p.num_splits + split) * 2;
                ml[0] = m[r]; ml[1] = l[r];
            }
        }
    }
}

// out[row] = sum_s exp(m_s - M) O_s / sum_s exp(m_s - M) l_s over the splits of the row.
// One block per row: the first warp turns the (max, sum) pairs into one weight per split (kept in
// shared memory); then the block's MERGE_GROUPS groups of threads each take every MERGE_GROUPS-th split - a thread
// owns output columns and adds its splits' partial outputs with independent loads, so a row of a hundred splits costs
// a few memory latencies, not a dozen - and the groups' sums are added in group order.  The order of the additions
// is fixed.
constexpr int MERGE_GROUPS = 4;
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, T* __restrict__ out,
                                  int num_splits, int D) {
    extern __shared__ float wgt[];                                  // [num_splits], then the groups' sums [MERGE_GROUPS][D]
    float* part = wgt + num_splits;
    TTIE_PDL_ENTRY();
    const size_t row = blockIdx.x;
    const float* ml = ws_ml + row * num_splits * 2;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int s = lane; s < num_splits; s += 32) {
            const float2 v = *reinterpret_cast<const float2*>(ml + 2 * s);
            if (v.y > 0.f) M = fmaxf(M, v.x);
        }
        M = warp_max(M);
        float den = 0.f;
        for (int s = lane; s < num_splits; s += 32) {
            const float2 v = *reinterpret_cast<const float2*>(ml + 2 * s);
            const float e = v.y > 0.f ? expf(v.x - M) : 0.f;
            wgt[s] = e;
            den += e * v.y;
        }
        den = warp_sum(den);
        const float inv = den > 0.f ? 1.f / den : 0.f;
        for (int s = lane; s < num_splits; s += 32) wgt[s] *= inv;
    }
    __syncthreads();
    const float* o = ws_o + row * num_splits * D;
    const int cols = blockDim.x / MERGE_GROUPS, g = threadIdx.x / cols, c = threadIdx.x - g * cols;
    for (int d = c; d < D; d += cols) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = g; s < num_splits; s += MERGE_GROUPS) acc = fmaf(wgt[s], o[(size_t)s * D + d], acc);
        part[g * D + d] = acc;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = part[d];
#pragma unroll
        for (int k = 1; k < MERGE_GROUPS; ++k) acc += part[k * D + d];
        out[row * D + d] = from_f32<T>(acc);
    }
}

// Up to NS <= 32 splits: every thread asks for all (max, sum) pairs of its row and for its column of every split's
// partial output at once, so the whole merge costs one memory latency; weights are computed redundantly per thread.
template <typename T, int NS>
__global__ void __launch_bounds__(128)
attn_merge_small_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, T* __restrict__ out, int num_splits, int D) {
    TTIE_PDL_ENTRY();
    const size_t row = blockIdx.x;
    const int d = blockIdx.y * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const float2* ml = reinterpret_cast<const float2*>(ws_ml + row * num_splits * 2);
    const float* o = ws_o + row * num_splits * D + d;
    float2 v[NS];
    float x[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        v[s] = s < num_splits ? ml[s] : make_float2(-INFINITY, 0.f);
        x[s] = s < num_splits ? o[(size_t)s * D] : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < NS; ++s) if (v[s].y > 0.f) M = fmaxf(M, v[s].x);
    float acc = 0.f, den = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s) {                               // fixed order
        const float e = v[s].y > 0.f ? expf(v[s].x - M) : 0.f;
        acc = fmaf(e, v[s].y > 0.f ? x[s] : 0.f, acc);
        den = fmaf(e, v[s].y, den);
    }
    out[row * D + d] = from_f32<T>(den > 0.f ? acc / den : 0.f);
}

// The same for up to 8 splits with four columns per thread and the rows packed into blocks of 256 threads: a prompt
// portion whose key range was cut brings thousands of rows, and one small block per row (16,384 rows x 2 splits: 24 us)
// spends its time on block launches, not on the 21 MB it moves.  The arithmetic per element is that of the kernel above.
template <int NS>
__global__ void __launch_bounds__(256)
attn_merge_vec_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, __nv_bfloat16* __restrict__ out,
                      long long rows, int num_splits, int D) {
    TTIE_PDL_ENTRY();
    const int per_row = D / 4;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = t / per_row;
    if (row >= rows) return;
    const int d = (int)(t - row * per_row) * 4;
    const float2* ml = reinterpret_cast<const float2*>(ws_ml + row * num_splits * 2);
    const float* o = ws_o + row * num_splits * D + d;
    float2 v[NS];
    float4 x[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        v[s] = s < num_splits ? ml[s] : make_float2(-INFINITY, 0.f);
        x[s] = s < num_splits ? *reinterpret_cast<const float4*>(o + (size_t)s * D) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < NS; ++s) if (v[s].y > 0.f) M = fmaxf(M, v[s].x);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s) {                               // fixed order
        const bool live = v[s].y > 0.f;
        const float e = live ? expf(v[s].x - M) : 0.f;
        acc.x = fmaf(e, live ? x[s].x : 0.f, acc.x);
        acc.y = fmaf(e, live ? x[s].y : 0.f, acc.y);
        acc.z = fmaf(e, live ? x[s].z : 0.f, acc.z);
        acc.w = fmaf(e, live ? x[s].w : 0.f, acc.w);
        den = fmaf(e, v[s].y, den);
    }
    const bool any = den > 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(any ? acc.x / den : 0.f, any ? acc.y / den : 0.f);
    __nv_bfloat162 hi = __floats2bfloat162_rn(any ? acc.z / den : 0.f, any ? acc.w / den : 0.f);
    uint2 packed;
    packed.x = *reinterpret_cast<unsigned*>(&lo);
    packed.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(out + row * D + d) = packed;
}

}  // namespace

namespace ttie {
int attn_merge_bf16(const float* ws_o, const float* ws_ml, void* out, int rows, int num_splits, int D, cudaStream_t s) {
    const dim3 grid(rows, ceil_div(D, 128));
    const bool vec = D % 4 == 0 && ((reinterpret_cast<uintptr_t>(ws_o) | reinterpret_cast<uintptr_t>(ws_ml)) & 15) == 0
                     && (reinterpret_cast<uintptr_t>(out) & 7) == 0;
    if (vec && num_splits <= 8) {
        const long long threads = (long long)rows * (D / 4);
        const unsigned blocks = (unsigned)((threads + 255) / 256);
        if (num_splits <= 2) { TTIE_LAUNCH(attn_merge_vec_kernel<2>, blocks, 256, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, (long long)rows, num_splits, D); }
        else if (num_splits <= 4) { TTIE_LAUNCH(attn_merge_vec_kernel<4>, blocks, 256, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, (long long)rows, num_splits, D); }
        else { TTIE_LAUNCH(attn_merge_vec_kernel<8>, blocks, 256, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, (long long)rows, num_splits, D); }
    } else if (num_splits <= 4) {
        TTIE_LAUNCH((attn_merge_small_kernel<__nv_bfloat16, 4>), grid, 128, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, num_splits, D);
    } else if (num_splits <= 8) {
        TTIE_LAUNCH((attn_merge_small_kernel<__nv_bfloat16, 8>), grid, 128, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, num_splits, D);
    } else if (num_splits <= 16) {
        TTIE_LAUNCH((attn_merge_small_kernel<__nv_bfloat16, 16>), grid, 128, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, num_splits, D);
    } else if (num_splits <= 32) {
        TTIE_LAUNCH((attn_merge_small_kernel<__nv_bfloat16, 32>), grid, 128, 0, s, ws_o, ws_ml, (__nv_bfloat16*)out, num_splits, D);
    } else {
        TTIE_LAUNCH(attn_merge_kernel<__nv_bfloat16>, rows, MERGE_GROUPS * (D >= 128 ? 128 : 64), (num_splits + MERGE_GROUPS * D) * sizeof(float), s,
                    ws_o, ws_ml, (__nv_bfloat16*)out, num_splits, D);
    }
    TTIE_CHECK_LAUNCH("attention merge");
    return 0;
}
}  // namespace ttie

namespace {
template <typename T, int DPL>
int launch(const AttnParams& p, int T_tokens, cudaStream_t s) {
    const size_t smem = ((size_t)ROWS * p.D + 2 * (size_t)BK * (p.D + 4)) * sizeof(float);
    auto k = paged_attn_simt_kernel<T, DPL>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(p.num_seqs * p.Hkv * p.row_tiles, p.num_splits);
    k<<<grid, WARPS * 32, smem, s>>>(p);
    TTIE_CHECK_LAUNCH("paged_attention");
    if (p.num_splits > 1) {
        attn_merge_kernel<T><<<T_tokens * p.Hq, MERGE_GROUPS * (p.D >= 128 ? 128 : 64), (p.num_splits + MERGE_GROUPS * p.D) * sizeof(float), s>>>(
            p.ws_o, p.ws_ml, (T*)p.out, p.num_splits, p.D);
        TTIE_CHECK_LAUNCH("attention merge");
    }
    return 0;
}

template <typename T>
int dispatch(const AttnParams& p, int T_tokens, cudaStream_t s) {
    switch ((p.D + 31) / 32) {
        case 1: return launch<T, 1>(p, T_tokens, s);
        case 2: return launch<T, 2>(p, T_tokens, s);
        case 3: return launch<T, 3>(p, T_tokens, s);
        case 4: return launch<T, 4>(p, T_tokens, s);
        case 5: return launch<T, 5>(p, T_tokens, s);
        case 6: return launch<T, 6>(p, T_tokens, s);
        case 7: return launch<T, 7>(p, T_tokens, s);
        case 8: return launch<T, 8>(p, T_tokens, s);
    }
    TTIE_FAIL("paged_attention: head size %d not supported (multiples of 4 up to 256)", p.D);
}
}  // namespace

// Scratch floats needed for `num_splits` splits: the caller allocates ws_o and ws_ml.
extern "C" long long ttie_attn_scratch_floats(int T, int Hq, int D, int num_splits) {
    return num_splits > 1 ? (long long)T * Hq * num_splits * (D + 2) : 0;
}

extern "C" int ttie_paged_attention(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                    const int* block_table, int table_width, int page_size, const int* qsl,
                                    const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                    int max_q_len, float scale, int window, int num_splits, int split_len,
                                    float* scratch, int dtype, void* stream) {
    if (T <= 0 || num_seqs <= 0) return 0;
    if (D % 4 || D > 256 || D <= 0) TTIE_FAIL("paged_attention: head size %d not supported (multiples of 4 up to 256)", D);
    if (Hkv <= 0 || Hq % Hkv) TTIE_FAIL("paged_attention: %d heads are not a multiple of %d kv heads", Hq, Hkv);
    if (page_size <= 0) TTIE_FAIL("paged_attention: page size %d", page_size);
    if (num_splits < 1) num_splits = 1;
    if (num_splits > 1 && (split_len <= 0 || !scratch)) TTIE_FAIL("paged_attention: splits need split_len and scratch");
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.k_pages = k_pages; p.v_pages = v_pages;
    p.block_table = block_table; p.table_width = table_width; p.page_size = page_size;
    p.qsl = qsl; p.seq_lens = seq_lens; p.out = out;
    p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.scale = scale; p.window = window;
    const int G = Hq / Hkv;
    p.row_tiles = ceil_div(max_q_len * G, ROWS);
    p.num_splits = num_splits; p.split_len = split_len;
    p.ws_o = scratch;
    p.ws_ml = scratch ? scratch + (size_t)T * Hq * num_splits * D : nullptr;
    if ((long long)p.num_seqs * p.Hkv * p.row_tiles > 2147483647LL) TTIE_FAIL("paged_attention: grid too large");
    if (num_splits > 65535) TTIE_FAIL("paged_attention: too many splits (%d)", num_splits);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kF32) return dispatch<float>(p, T, s);
    if (dtype == kBF16) return dispatch<__nv_bfloat16>(p, T, s);
    TTIE_FAIL("paged_attention: unknown dtype %d", dtype);
}
