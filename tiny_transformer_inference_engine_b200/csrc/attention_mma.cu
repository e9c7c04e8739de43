// Paged causal attention on tensor cores for the bfloat16 path: one kernel for prompt portions
// and for decoded tokens.
//
// A query row is a (token, head of a kv head's group) pair, so with multi-query attention the
// 16*NWARPS rows of a CTA are a few tokens times all their heads and every key/value tile that
// the CTA brings into shared memory serves all of them (the reference's kernel takes one head
// per CTA, kernels/pagedattn/pagedattn.cu:921-922, and reads each key tile once per head).
// Prompt portions use 64-row tiles; decode steps use the smallest tile that holds a token's
// heads and split the key range over CTAs, whose partial results a second kernel merges.
//
// Mask, scale and block-table lookup as kernels/pagedattn/pagedattn.cu:196-207,256: ctx =
// kv_len - q_len, the row of token t sees keys j <= ctx + t (and j > ctx + t - window).
// Scores, running maximum, running sum and the output accumulate in float32; probabilities are
// rounded to bfloat16 for the second product, as the reference rounds them to half
// (pagedattn.cu:379-382).  Tiles arrive by 16-byte cp.async copies, two stages; products are
// mma.sync m16n8k16 fed by ldmatrix from rows padded by 16 bytes (conflict-free for every head
// size that is a multiple of 16).
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {
constexpr int BN = 64;

struct MmaParams {
    const __nv_bfloat16* q; long long q_stride;
    const __nv_bfloat16* k_pages; const __nv_bfloat16* v_pages;
    const int* block_table; int table_width; int page_size;
    const int* qsl; const int* seq_lens;
    __nv_bfloat16* out;
    int num_seqs, Hq, Hkv;
    float scale_log2; int window;
    int row_tiles, num_splits, split_len;
    float* ws_o; float* ws_ml;
};

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                                   // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// STAGES = 2: the next key/value tile is in flight while the current one is used (prompt portions: few,
// long-running CTAs).  STAGES = 1: half the shared memory, so more CTAs of a decode step share an SM and
// hide each other's load latency.
template <int D, int NWARPS, int STAGES>
__global__ void __launch_bounds__(NWARPS * 32)
paged_attn_mma_kernel(const MmaParams p) {
    constexpr int BM = NWARPS * 16, LDS = D + 8, NT = NWARPS * 32, CH = D / 8;      // CH: 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                // [BM][LDS]
    __nv_bfloat16* Ks = Qs + BM * LDS;                                             // [2][BN][LDS]
    __nv_bfloat16* Vs = Ks + STAGES * BN * LDS;                                    // [STAGES][BN][LDS]
    long long* rowoff = reinterpret_cast<long long*>(Vs + STAGES * BN * LDS);      // [STAGES][BN] element offset of a key's row, -1: none
    TTIE_PDL_ENTRY();

    const int G = p.Hq / p.Hkv;
    int tile = blockIdx.x;
    const int split = blockIdx.y;
    const int rt = p.row_tiles - 1 - tile % p.row_tiles;                            // late (long) tiles first
    tile /= p.row_tiles;
    const int kvh = tile % p.Hkv;
    const int seq = tile / p.Hkv;
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G;
    const int row0 = rt * BM;
    if (row0 >= nrows) return;
    const int ctx = kv_len - q_len;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int tok_lo = row0 / G, tok_hi = (min(nrows, row0 + BM) - 1) / G;
    int k_hi = ctx + tok_hi + 1;
    int k_lo = p.window > 0 ? max(0, ctx + tok_lo - p.window + 1) : 0;
    if (p.num_splits > 1) {
        k_lo = max(k_lo, split * p.split_len);
        k_hi = min(k_hi, (split + 1) * p.split_len);
    }
    k_lo = k_lo / BN * BN;                                                          // tiles start on multiples of BN

    // the two rows of this thread
    int rpos[2], rlo[2]; bool rvalid[2]; int rrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + warp * 16 + (lane >> 2) + 8 * h;
        rrow[h] = row;
        rvalid[h] = row < nrows;
        rpos[h] = rvalid[h] ? ctx + row / G : -1;
        rlo[h] = p.window > 0 ? max(0, rpos[h] - p.window + 1) : 0;
    }
    // position range of the warp's rows (uniform over the warp)
    const int wrow_lo = row0 + warp * 16, wrow_hi = min(nrows, wrow_lo + 16) - 1;
    const bool warp_active = wrow_lo < nrows;
    const int wpos_hi = warp_active ? ctx + wrow_hi / G : -1;
    const int wpos_lo = warp_active ? ctx + wrow_lo / G : -1;
    const int wkey_lo = p.window > 0 ? max(0, wpos_lo - p.window + 1) : 0;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    const int ntiles = k_lo < k_hi ? (k_hi - k_lo + BN - 1) / BN : 0;
    const int* table = p.block_table + (size_t)seq * p.table_width;

    auto fill_rowoff = [&](int stage, int kt) {
        for (int j = tid; j < BN; j += NT) {
            const int key = kt + j;
            long long off = -1;
            if (key < k_hi) {
                const int pg = key / p.page_size;
                const int page = table[pg];
                off = (((long long)page * p.Hkv + kvh) * p.page_size + (key - pg * p.page_size)) * D;
            }
            rowoff[stage * BN + j] = off;
        }
    };
    auto issue_tile = [&](int stage) {
        __nv_bfloat16* kd = Ks + stage * BN * LDS;
        __nv_bfloat16* vd = Vs + stage * BN * LDS;
        for (int c = tid; c < BN * CH; c += NT) {
            const int j = c / CH, part = c - j * CH;
            const long long off = rowoff[stage * BN + j];
            const bool ok = off >= 0;
            const long long src = ok ? off + part * 8 : 0;
            cp_async16(kd + j * LDS + part * 8, p.k_pages + src, ok);
            cp_async16(vd + j * LDS + part * 8, p.v_pages + src, ok);
        }
    };

    if (ntiles > 0) {
        // queries of the tile
        for (int c = tid; c < BM * CH; c += NT) {
            const int r = c / CH, part = c - r * CH;
            const int row = row0 + r;
            const bool ok = row < nrows;
            const int tok = ok ? row / G : 0, g = ok ? row - tok * G : 0;
            const __nv_bfloat16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + part * 8;
            cp_async16(Qs + r * LDS + part * 8, ok ? src : p.q, ok);
        }
        fill_rowoff(0, k_lo);
        __syncthreads();
        issue_tile(0);
        cp_async_commit();
    }

    unsigned qf[D / 16][4];
    for (int t = 0; t < ntiles; ++t) {
        const int stage = STAGES == 2 ? (t & 1) : 0, kt = k_lo + t * BN;
        if (STAGES == 2) {
            if (t + 1 < ntiles) fill_rowoff(stage ^ 1, kt + BN);
            __syncthreads();                       // row offsets visible; everyone is done with the other stage
            if (t + 1 < ntiles) issue_tile(stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (t > 0) {
                __syncthreads();                   // everyone is done with the previous tile
                fill_rowoff(0, kt);
                __syncthreads();
                issue_tile(0);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        __syncthreads();                           // tile t (and the queries) have landed for every thread
        if (t == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qf[ks], Qs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));
        }
        const bool needed = warp_active && kt <= wpos_hi && kt + BN > wkey_lo;
        if (needed) {
            const __nv_bfloat16* kb = Ks + stage * BN * LDS;
            const __nv_bfloat16* vb = Vs + stage * BN * LDS;
            float s[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < BN / 16; ++np) {
                    unsigned b[4];
                    ldmatrix_x4(b, kb + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
                    mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
                }
            }
            // scale, mask, running maximum
            const bool full = kt + BN - 1 <= wpos_lo && kt >= (p.window > 0 ? max(0, wpos_hi - p.window + 1) : 0) && kt + BN <= k_hi
                              && wrow_hi - wrow_lo == 15;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    float v = s[i][e] * p.scale_log2;
                    if (!full) {
                        const int key = kt + i * 8 + 2 * (lane & 3) + (e & 1);
                        if (!(rvalid[h] && key <= rpos[h] && key >= rlo[h] && key < k_hi)) v = -INFINITY;
                    }
                    s[i][e] = v;
                    mx[h] = fmaxf(mx[h], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            const float msub[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[i][e] - msub[e >> 1]);           // exp2(-inf) = 0 for masked keys
                    s[i][e] = pv;
                    l_run[e >> 1] += pv;
                }
            }
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                unsigned pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vb + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                    mma_bf16(o[2 * dp], pf, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // results: each thread owns columns 2*(lane&3), +1 of every 8-wide slice, for its two rows
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!rvalid[h]) continue;
        const int row = rrow[h];
        const int tok = row / G, g = row - tok * G;
        const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
        if (p.num_splits == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* op = p.out + grow * D + 2 * (lane & 3);
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
                *reinterpret_cast<__nv_bfloat162*>(op + i * 8) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        } else {
            float* wo = p.ws_o + (grow * p.num_splits + split) * D + 2 * (lane & 3);
#pragma unroll
            for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(wo + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
            if ((lane & 3) == 0) {
                float* ml = p.ws_ml + (grow * p.num_splits + split) * 2;
                ml[0] = m_run[h] * 0.6931471805599453f;             // back to natural-log units for the merge
                ml[1] = l;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------ decode form
// Few query rows per request (one decoded token times the heads of a kv head's group, or a short
// portion): there is too little work per key tile for the tile loop above to hide latency, so the
// key range is cut finer.  A CTA takes DEC_KEYS keys of one (request, kv head); each of its four
// warps loads its own 32 keys (cp.async, no CTA-wide barrier) and computes all query rows against
// them, 16 rows at a time; the four partial results of a 16-row tile are merged in shared memory
// and leave as one partial result per CTA (or as the final output if the request has one split).
constexpr int DEC_WARPS = 4, DEC_WKEYS = 32, DEC_KEYS = DEC_WARPS * DEC_WKEYS, DEC_MAX_ROWS = 128;

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_attn_decode_kernel(const MmaParams p) {
    constexpr int LDS = D + 8, CH = D / 8, NT = DEC_WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int G = p.Hq / p.Hkv;
    const int kvh = blockIdx.x % p.Hkv, seq = blockIdx.x / p.Hkv, split = blockIdx.y;
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G;
    if (nrows <= 0) return;
    const int nmt = (nrows + 15) / 16;
    const int rows_pad = nmt * 16;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [rows_pad][LDS]
    __nv_bfloat16* Ks = Qs + p.row_tiles * LDS;                                     // [4 warps][32][LDS]; row_tiles holds the padded row capacity here
    __nv_bfloat16* Vs = Ks + DEC_WARPS * DEC_WKEYS * LDS;
    float* Op = reinterpret_cast<float*>(Vs + DEC_WARPS * DEC_WKEYS * LDS);         // [4 warps][16][D] partial outputs
    float* MLp = Op + DEC_WARPS * 16 * D;                                           // [4 warps][16][2]
    const int ctx = kv_len - q_len;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kbase = split * DEC_KEYS;
    const bool cta_has_keys = kbase < kv_len;

    if (cta_has_keys) {
        for (int c = tid; c < rows_pad * CH; c += NT) {
            const int r = c / CH, part = c - r * CH;
            const bool ok = r < nrows;
            const int tok = ok ? r / G : 0, g = ok ? r - tok * G : 0;
            const __nv_bfloat16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + part * 8;
            cp_async16(Qs + r * LDS + part * 8, ok ? src : p.q, ok);
        }
        // this warp's 32 keys
        const int key = kbase + warp * DEC_WKEYS + lane;
        long long off = -1;
        if (key < kv_len) {
            const int pg = key / p.page_size;
            const int page = p.block_table[(size_t)seq * p.table_width + pg];
            off = (((long long)page * p.Hkv + kvh) * p.page_size + (key - pg * p.page_size)) * D;
        }
        __nv_bfloat16* kd = Ks + warp * DEC_WKEYS * LDS;
        __nv_bfloat16* vd = Vs + warp * DEC_WKEYS * LDS;
#pragma unroll
        for (int i = 0; i < DEC_WKEYS * CH / 32; ++i) {
            const int c = lane + 32 * i;
            const int j = c / CH, part = c - j * CH;
            const long long o = __shfl_sync(0xffffffffu, off, j);
            const bool ok = o >= 0;
            const long long src = ok ? o + part * 8 : 0;
            cp_async16(kd + j * LDS + part * 8, p.k_pages + src, ok);
            cp_async16(vd + j * LDS + part * 8, p.v_pages + src, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
    }
    __syncthreads();

    const int wkey0 = kbase + warp * DEC_WKEYS;
    const __nv_bfloat16* kb = Ks + warp * DEC_WKEYS * LDS;
    const __nv_bfloat16* vb = Vs + warp * DEC_WKEYS * LDS;
    for (int mt = 0; mt < nmt; ++mt) {
        float o[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
        float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
        int rpos[2], rlo[2]; bool rvalid[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = mt * 16 + (lane >> 2) + 8 * h;
            rvalid[h] = row < nrows;
            rpos[h] = rvalid[h] ? ctx + row / G : -1;
            rlo[h] = p.window > 0 ? max(0, rpos[h] - p.window + 1) : 0;
        }
        const int mt_pos_hi = ctx + (min(nrows, mt * 16 + 16) - 1) / G;
        const int mt_key_lo = p.window > 0 ? max(0, ctx + (mt * 16) / G - p.window + 1) : 0;
        const bool needed = cta_has_keys && wkey0 < kv_len && wkey0 <= mt_pos_hi && wkey0 + DEC_WKEYS > mt_key_lo;
        if (needed) {
            float s[DEC_WKEYS / 8][4];
#pragma unroll
            for (int i = 0; i < DEC_WKEYS / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                unsigned qf[4];
                ldmatrix_x4(qf, Qs + (mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));
#pragma unroll
                for (int np = 0; np < DEC_WKEYS / 16; ++np) {
                    unsigned b[4];
                    ldmatrix_x4(b, kb + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
                    mma_bf16(s[2 * np], qf, b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < DEC_WKEYS / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int key = wkey0 + i * 8 + 2 * (lane & 3) + (e & 1);
                    float v = s[i][e] * p.scale_log2;
                    if (!(rvalid[h] && key <= rpos[h] && key >= rlo[h] && key < kv_len)) v = -INFINITY;
                    s[i][e] = v;
                    mx[h] = fmaxf(mx[h], v);
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                mrow[h] = mx[h];
            }
            const float msub[2] = {mrow[0] == -INFINITY ? 0.f : mrow[0], mrow[1] == -INFINITY ? 0.f : mrow[1]};
#pragma unroll
            for (int i = 0; i < DEC_WKEYS / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[i][e] - msub[e >> 1]);
                    s[i][e] = pv;
                    lrow[e >> 1] += pv;
                }
#pragma unroll
            for (int kk = 0; kk < DEC_WKEYS / 16; ++kk) {
                unsigned pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vb + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                    mma_bf16(o[2 * dp], pf, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
                }
            }
        }
        // this warp's partial result of the 16 rows -> shared memory
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = lrow[h];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const int r = (lane >> 2) + 8 * h;
            float* op = Op + (warp * 16 + r) * D + 2 * (lane & 3);
#pragma unroll
            for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(op + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
            if ((lane & 3) == 0) { MLp[(warp * 16 + r) * 2] = mrow[h]; MLp[(warp * 16 + r) * 2 + 1] = l; }
        }
        __syncthreads();
        // merge the four warps' partial results (maxima are in log2 units)
        for (int e = tid; e < 16 * D; e += NT) {
            const int r = e / D, d = e - r * D;
            const int row = mt * 16 + r;
            if (row >= nrows) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) if (MLp[(w * 16 + r) * 2 + 1] > 0.f) M = fmaxf(M, MLp[(w * 16 + r) * 2]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float lw = MLp[(w * 16 + r) * 2 + 1];
                if (lw > 0.f) {
                    const float f = exp2f(MLp[(w * 16 + r) * 2] - M);
                    acc += f * Op[(w * 16 + r) * D + d];
                    L += f * lw;
                }
            }
            const int tok = row / G, g = row - tok * G;
            const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
            if (p.num_splits == 1) {
                p.out[grow * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            } else {
                p.ws_o[(grow * p.num_splits + split) * D + d] = acc;
                if (d == 0) {
                    float* ml = p.ws_ml + (grow * p.num_splits + split) * 2;
                    ml[0] = M * 0.6931471805599453f;                // natural-log units for the merge kernel
                    ml[1] = L;
                }
            }
        }
        __syncthreads();
    }
}

template <int D>
int launch_decode(const MmaParams& p, cudaStream_t s) {
    constexpr int LDS = D + 8;
    const size_t smem = ((size_t)p.row_tiles * LDS + 2 * (size_t)DEC_KEYS * LDS) * sizeof(__nv_bfloat16)
                        + (size_t)DEC_WARPS * 16 * (D + 2) * sizeof(float);
    auto k = paged_attn_decode_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) TTIE_FAIL("paged_attention_decode: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid(p.num_seqs * p.Hkv, p.num_splits);
    k<<<grid, DEC_WARPS * 32, smem, s>>>(p);
    TTIE_CHECK_LAUNCH("paged_attention_decode");
    return 0;
}

template <int D, int NWARPS>
int launch(const MmaParams& p, cudaStream_t s) {
    constexpr int BM = NWARPS * 16, LDS = D + 8, STAGES = NWARPS >= 4 ? 2 : 1;
    const size_t smem = ((size_t)BM * LDS + 2 * STAGES * (size_t)BN * LDS) * sizeof(__nv_bfloat16) + STAGES * BN * sizeof(long long);
    auto k = paged_attn_mma_kernel<D, NWARPS, STAGES>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) TTIE_FAIL("paged_attention_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid(p.num_seqs * p.Hkv * p.row_tiles, p.num_splits);
    TTIE_LAUNCH(k, grid, NWARPS * 32, smem, s, p);
    TTIE_CHECK_LAUNCH("paged_attention_mma");
    return 0;
}

template <int D>
int pick_rows(const MmaParams& p, int rows_per_seq_max, cudaStream_t s, int* bm) {
    if (rows_per_seq_max <= 16) { *bm = 16; return launch<D, 1>(p, s); }
    if (rows_per_seq_max <= 32) { *bm = 32; return launch<D, 2>(p, s); }
    *bm = 64; return launch<D, 4>(p, s);
}
}  // namespace

// Rows per CTA tile the kernel will use for a batch whose longest request brings max_q_len tokens.
extern "C" int ttie_attn_mma_tile_rows(int max_q_len, int Hq, int Hkv) {
    const int rows = max_q_len * (Hq / Hkv);
    return rows <= 16 ? 16 : (rows <= 32 ? 32 : 64);
}

extern "C" int ttie_attn_mma_supported(int D) { return D % 16 == 0 && D >= 16 && D <= 128; }

// The decode form takes requests that bring at most this many query rows (tokens x heads per kv head)
// and splits keys in pieces of ttie_attn_decode_split_len().
extern "C" int ttie_attn_decode_max_rows() { return DEC_MAX_ROWS; }
extern "C" int ttie_attn_decode_split_len() { return DEC_KEYS; }

// form 0: tile loop (prompt portions; decode with caller-chosen splits).  form 1: decode form.
extern "C" int ttie_paged_attention_mma_form(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                             const int* block_table, int table_width, int page_size, const int* qsl,
                                             const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                             int max_q_len, float scale, int window, int num_splits, int split_len,
                                             float* scratch, int form, void* stream);

extern "C" int ttie_paged_attention_mma(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_width, int page_size, const int* qsl,
                                        const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                        int max_q_len, float scale, int window, int num_splits, int split_len,
                                        float* scratch, void* stream) {
    return ttie_paged_attention_mma_form(q, q_stride, k_pages, v_pages, block_table, table_width, page_size, qsl, seq_lens, out,
                                         T, num_seqs, Hq, Hkv, D, max_q_len, scale, window, num_splits, split_len, scratch, 0, stream);
}

extern "C" int ttie_paged_attention_mma_form(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                             const int* block_table, int table_width, int page_size, const int* qsl,
                                             const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                             int max_q_len, float scale, int window, int num_splits, int split_len,
                                             float* scratch, int form, void* stream) {
    if (T <= 0 || num_seqs <= 0) return 0;
    if (!ttie_attn_mma_supported(D)) TTIE_FAIL("paged_attention_mma: head size %d not supported (multiples of 16 up to 128)", D);
    if (Hkv <= 0 || Hq % Hkv) TTIE_FAIL("paged_attention_mma: %d heads are not a multiple of %d kv heads", Hq, Hkv);
    if (q_stride % 8) TTIE_FAIL("paged_attention_mma: query row stride %lld must be a multiple of 8 elements", q_stride);
    if (((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) TTIE_FAIL("paged_attention_mma: pointers must be 16-byte aligned");
    if (num_splits < 1) num_splits = 1;
    if (num_splits > 1 && (split_len <= 0 || split_len % BN || !scratch))
        TTIE_FAIL("paged_attention_mma: splits need scratch and a split length that is a multiple of %d", BN);
    if (num_splits > 65535) TTIE_FAIL("paged_attention_mma: too many splits (%d)", num_splits);
    MmaParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
    p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.block_table = block_table; p.table_width = table_width; p.page_size = page_size;
    p.qsl = qsl; p.seq_lens = seq_lens; p.out = (__nv_bfloat16*)out;
    p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv;
    p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
    p.num_splits = num_splits; p.split_len = split_len;
    p.ws_o = scratch; p.ws_ml = scratch ? scratch + (size_t)T * Hq * num_splits * D : nullptr;
    const int rows = max_q_len * (Hq / Hkv);
    if (form == 1) {
        if (rows > DEC_MAX_ROWS) TTIE_FAIL("paged_attention_mma: the decode form takes at most %d query rows per request, got %d", DEC_MAX_ROWS, rows);
        if (num_splits > 1 && split_len != DEC_KEYS) TTIE_FAIL("paged_attention_mma: the decode form splits keys by %d", DEC_KEYS);
        p.row_tiles = ceil_div(rows, 16) * 16;                  // padded query-row capacity of the CTA's shared memory
        int rc;
        switch (D) {
            case 16: rc = launch_decode<16>(p, (cudaStream_t)stream); break;
            case 32: rc = launch_decode<32>(p, (cudaStream_t)stream); break;
            case 48: rc = launch_decode<48>(p, (cudaStream_t)stream); break;
            case 64: rc = launch_decode<64>(p, (cudaStream_t)stream); break;
            case 80: rc = launch_decode<80>(p, (cudaStream_t)stream); break;
            case 96: rc = launch_decode<96>(p, (cudaStream_t)stream); break;
            case 112: rc = launch_decode<112>(p, (cudaStream_t)stream); break;
            case 128: rc = launch_decode<128>(p, (cudaStream_t)stream); break;
            default: TTIE_FAIL("paged_attention_mma: head size %d", D);
        }
        if (rc) return rc;
        if (num_splits > 1) return attn_merge_bf16(p.ws_o, p.ws_ml, out, T * Hq, num_splits, D, (cudaStream_t)stream);
        return 0;
    }
    const int bm = ttie_attn_mma_tile_rows(max_q_len, Hq, Hkv);
    p.row_tiles = ceil_div(rows, bm);
    if ((long long)num_seqs * Hkv * p.row_tiles > 2147483647LL) TTIE_FAIL("paged_attention_mma: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    int used = 0, rc;
    switch (D) {
        case 16: rc = pick_rows<16>(p, rows, s, &used); break;
        case 32: rc = pick_rows<32>(p, rows, s, &used); break;
        case 48: rc = pick_rows<48>(p, rows, s, &used); break;
        case 64: rc = pick_rows<64>(p, rows, s, &used); break;
        case 80: rc = pick_rows<80>(p, rows, s, &used); break;
        case 96: rc = pick_rows<96>(p, rows, s, &used); break;
        case 112: rc = pick_rows<112>(p, rows, s, &used); break;
        case 128: rc = pick_rows<128>(p, rows, s, &used); break;
        default: TTIE_FAIL("paged_attention_mma: head size %d", D);
    }
    if (rc) return rc;
    if (num_splits > 1) return attn_merge_bf16(p.ws_o, p.ws_ml, out, T * Hq, num_splits, D, s);
    return 0;
}
