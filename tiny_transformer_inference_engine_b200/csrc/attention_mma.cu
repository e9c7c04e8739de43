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
// 2^x on the special-function unit (ex2(-inf) = 0); exp2f() wraps the same instruction in range handling
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
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
        const int piece = piece_len(kv_len, p.num_splits, p.split_len, BN);
        k_lo = max(k_lo, split * piece);
        k_hi = min(k_hi, (split + 1) * piece);
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
                const int page = pg < p.table_width ? table[pg] : 0;             // (a table that is too short: the scratch page, not a wild read)
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
                    float v = s[i][e];                                 // raw scores; the scale (positive) goes into the exponent's fma
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
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2)) * p.scale_log2;
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = (m_new == -INFINITY) ? 1.f : ex2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            const float msub[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ex2(fmaf(s[i][e], p.scale_log2, -msub[e >> 1]));           // exp2(-inf) = 0 for masked keys
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
// portion).  A thread-block cluster takes one (request, kv head, row tile): its C CTAs cut the key range
// into C pieces, and inside a CTA KG groups of RW warps walk their piece in 64-key tiles, group g taking
// tiles g, g + KG, ...  A group loads its own tile (cp.async) and synchronises only with itself (a named
// barrier), so one group's loads run under another's products.  At the end the groups' partial results
// are merged in shared memory, then the C CTAs' results through distributed shared memory: CTA r reads
// rows r, r + C, ... of every CTA, adds them in rank order and writes the output.  No scratch in global
// memory and no second kernel.
constexpr int CL_MAX_ROWS = 32;

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned map_to_rank(const void* local, unsigned rank) {
    unsigned remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_cluster_f32x4(unsigned addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_cluster_f32x2(unsigned addr, float2 v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}
// bytes of the key/value tiles and their row offsets (the area that later holds the groups' partial results)
template <int D, int RW, int KG>
__host__ __device__ constexpr size_t cluster_tile_bytes() {
    constexpr size_t tiles = (size_t)KG * 2 * BN * (D + 8) * 2;
    constexpr size_t part = (size_t)KG * RW * 16 * (D + 8 + 2) * 4;
    return ((tiles > part ? tiles : part) + 15) / 16 * 16;
}
template <int D, int RW, int KG>
__global__ void __launch_bounds__(RW * KG * 32)
paged_attn_cluster_kernel(const MmaParams p) {
    constexpr int BM = RW * 16, LDS = D + 8, CH = D / 8, NT = RW * KG * 32, GT = RW * 32;     // GT: threads of a key group
    constexpr int LDO = D + 8;                                                     // float row stride of the exchange buffers (no bank conflicts)
    constexpr int NI = BN * CH / GT;                                               // 16-byte pieces of a tile per thread
    static_assert(BN == 64 && (BN * CH) % GT == 0, "a lane holds the row offsets of keys lane and lane + 32");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(smem_raw);                // [KG][2][BN][LDS]
    // after the key loop the tile area holds the partial results
    float* Op = reinterpret_cast<float*>(KV);                                      // [KG][BM][LDO]
    float* MLp = Op + KG * BM * LDO;                                               // [KG][BM][2]
    // Rows that the other CTAs of the cluster send here (never aliased: they may arrive while this CTA still
    // works on its tiles): slot = sender's rank * rows per owner + local row
    float* Recv = reinterpret_cast<float*>(smem_raw + cluster_tile_bytes<D, RW, KG>());   // [BM + 16][LDO]
    float* MLrecv = Recv + (BM + 16) * LDO;                                        // [BM + 16][2]
    TTIE_PDL_ENTRY();

    const int G = p.Hq / p.Hkv;
    int tile = blockIdx.x;
    const int rt = tile % p.row_tiles;
    tile /= p.row_tiles;
    const int kvh = tile % p.Hkv, seq = tile / p.Hkv;
    const unsigned rank = cluster_rank(), C = cluster_size();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kg = warp / RW, rw = warp - kg * RW, gtid = tid - kg * GT;
    const int* table = p.block_table + (size_t)seq * p.table_width;
    // Without a window the first tile of this group is known before the request's lengths are: its page
    // numbers are asked for together with the lengths (one memory latency instead of two).
    const int kt_guess = (int)rank * p.split_len + kg * BN;
    int page_guess[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pg = (kt_guess + lane + 32 * i) / p.page_size;
        page_guess[i] = pg < p.table_width ? table[pg] : 0;
    }
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G;
    const int row0 = rt * BM;
    if (row0 >= nrows) return;                                                     // the same for every CTA of the cluster
    // "I have started": a CTA may write into another's shared memory only once that CTA is known to run, and a CTA
    // with no keys of its own reaches the exchange at once.  The matching wait stands before the first remote
    // store; the key loop lies between them, so it costs nothing.
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int ctx = kv_len - q_len;

    const int tok_lo = row0 / G, tok_hi = (min(nrows, row0 + BM) - 1) / G;
    int k_hi = ctx + tok_hi + 1;
    int k_lo = p.window > 0 ? max(0, ctx + tok_lo - p.window + 1) : 0;
    k_lo = max(k_lo, (int)rank * p.split_len);
    k_hi = min(k_hi, ((int)rank + 1) * p.split_len);
    k_lo = k_lo / BN * BN;

    int rpos[2], rlo[2]; bool rvalid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + rw * 16 + (lane >> 2) + 8 * h;
        rvalid[h] = row < nrows;
        rpos[h] = rvalid[h] ? ctx + row / G : -1;
        rlo[h] = p.window > 0 ? max(0, rpos[h] - p.window + 1) : 0;
    }
    const int wrow_lo = row0 + rw * 16, wrow_hi = min(nrows, wrow_lo + 16) - 1;
    const bool warp_active = wrow_lo < nrows;
    const int wpos_hi = warp_active ? ctx + wrow_hi / G : -1;
    const int wpos_lo = warp_active ? ctx + wrow_lo / G : -1;
    const int wkey_lo = p.window > 0 ? max(0, wpos_lo - p.window + 1) : 0;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    const int kt0 = k_lo + kg * BN;                                                // this group's first tile
    // this warp's 16 query rows straight into mma A fragments (4-byte loads; no shared memory, no barrier):
    // fragment registers 0,1 hold columns 2q, 2q+1 of rows g and g+8, registers 2,3 the same 8 columns on
    unsigned qf[D / 16][4];
    {
        const __nv_bfloat16* qrow[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = row0 + rw * 16 + (lane >> 2) + 8 * h;
            const int tok = rvalid[h] ? row / G : 0, g = rvalid[h] ? row - tok * G : 0;
            qrow[h] = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + 2 * (lane & 3);
        }
        const bool any_keys = kt0 < k_hi;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                qf[ks][j] = (any_keys && rvalid[j & 1]) ? *reinterpret_cast<const unsigned*>(qrow[j & 1] + ks * 16 + 8 * (j >> 1)) : 0u;
    }
    __nv_bfloat16* kb = KV + (kg * 2) * BN * LDS;
    __nv_bfloat16* vb = kb + BN * LDS;
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(kg + 1), "r"(GT) : "memory"); };
    // Row offsets of tile `kt`: lane l of every warp holds those of keys l and l + 32 (-1: no such key); the
    // copy loop fetches the one it needs by shuffle, so no shared memory and no barrier come between the
    // page numbers and the copies.  `pages`: page numbers already loaded for exactly this tile, or null.
    // (unsigned row numbers: a pool of 2^32 rows of keys and as many of values would not fit the GPU's memory)
    constexpr unsigned NO_ROW = 0xffffffffu;
    auto row_offsets = [&](unsigned (&off)[2], int kt, const int* pages) {  // in rows of D elements
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int key = kt + lane + 32 * i;
            off[i] = NO_ROW;
            if (key < k_hi) {
                const int pg = key / p.page_size;
                const int page = pages ? pages[i] : (pg < p.table_width ? table[pg] : 0);
                off[i] = ((unsigned)page * (unsigned)p.Hkv + (unsigned)kvh) * (unsigned)p.page_size + (unsigned)(key - pg * p.page_size);
            }
        }
    };
    auto issue = [&](__nv_bfloat16* dst, const __nv_bfloat16* pages, const unsigned (&off)[2]) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int c = gtid + i * GT;
            const int j = c / CH, part = c - j * CH;
            const unsigned lo = __shfl_sync(0xffffffffu, off[0], j & 31), hi = __shfl_sync(0xffffffffu, off[1], j & 31);
            const unsigned o = j < 32 ? lo : hi;
            const bool ok = o != NO_ROW;
            cp_async16(dst + j * LDS + part * 8, pages + (ok ? (size_t)o * D + part * 8 : 0), ok);
        }
        cp_async_commit();
    };
    // Keys and values are separate copy groups: the next tile's keys are asked for as soon as this tile's
    // scores are done, its values after the second product, so most of their latency hides behind arithmetic.
    unsigned off_cur[2], off_next[2] = {NO_ROW, NO_ROW};
    if (kt0 < k_hi) {
        row_offsets(off_cur, kt0, kt0 == kt_guess ? page_guess : nullptr);
        issue(kb, p.k_pages, off_cur);
        issue(vb, p.v_pages, off_cur);
    }
    for (int kt = kt0; kt < k_hi; kt += KG * BN) {
        const int kt_next = kt + KG * BN;
        const bool more = kt_next < k_hi;
        if (more) row_offsets(off_next, kt_next, nullptr);      // (its page loads overlap the wait below)
        cp_async_wait<1>();                                     // this tile's keys (its values may still be on their way)
        group_sync();
        const bool needed = warp_active && kt <= wpos_hi && kt + BN > wkey_lo;
        float s[BN / 8][4];
        if (needed) {
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
        }
        group_sync();                                           // the group has read the keys: their buffer is free
        if (more) issue(kb, p.k_pages, off_next); else cp_async_commit();
        if (needed) {
            const bool full = kt + BN - 1 <= wpos_lo && kt >= (p.window > 0 ? max(0, wpos_hi - p.window + 1) : 0) && kt + BN <= k_hi
                              && wrow_hi - wrow_lo == 15;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    float v = s[i][e];                                 // raw scores; the scale (positive) goes into the exponent's fma
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
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2)) * p.scale_log2;
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = (m_new == -INFINITY) ? 1.f : ex2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            const float msub[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ex2(fmaf(s[i][e], p.scale_log2, -msub[e >> 1]));
                    s[i][e] = pv;
                    l_run[e >> 1] += pv;
                }
            }
            if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
                for (int i = 0; i < D / 8; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
            }
        }
        cp_async_wait<1>();                                     // this tile's values (the next keys may still be on their way)
        group_sync();
        if (needed) {
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
        group_sync();                                           // the group has read the values
        if (more) issue(vb, p.v_pages, off_next); else cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();                               // every group is done with its tiles: the area becomes the exchange buffers

    // each warp's partial result -> shared memory
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int r = rw * 16 + (lane >> 2) + 8 * h;
        float* op = Op + ((size_t)kg * BM + r) * LDO + 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(op + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
        if ((lane & 3) == 0) { MLp[(kg * BM + r) * 2] = m_run[h]; MLp[(kg * BM + r) * 2 + 1] = l; }
    }
    __syncthreads();
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");                    // every CTA of the cluster has started
    // the groups of this CTA, in group order (maxima are in log2 units)
    const int rows_per_owner = (BM + (int)C - 1) / (int)C;
    for (int e = tid; e < BM * (D / 4); e += NT) {
        const int r = e / (D / 4), c4 = e - r * (D / 4);
        float mg[KG], lg[KG];
        float4 vg[KG];
#pragma unroll
        for (int g2 = 0; g2 < KG; ++g2) {
            const float2 ml = *reinterpret_cast<const float2*>(MLp + (g2 * BM + r) * 2);
            mg[g2] = ml.x; lg[g2] = ml.y;
            vg[g2] = *reinterpret_cast<const float4*>(Op + ((size_t)g2 * BM + r) * LDO + c4 * 4);
        }
        float M = -INFINITY;
#pragma unroll
        for (int g2 = 0; g2 < KG; ++g2) if (lg[g2] > 0.f) M = fmaxf(M, mg[g2]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (int g2 = 0; g2 < KG; ++g2) {
            const float f = lg[g2] > 0.f ? ex2(mg[g2] - M) : 0.f;
            acc.x += f * vg[g2].x; acc.y += f * vg[g2].y; acc.z += f * vg[g2].z; acc.w += f * vg[g2].w;
            L += f * lg[g2];
        }
        // row r belongs to CTA r % C of the cluster, which adds the C partial results
        const unsigned owner = (unsigned)r % C;
        const int slot = (int)rank * rows_per_owner + r / (int)C;
        st_cluster_f32x4(map_to_rank(Recv + (size_t)slot * LDO + c4 * 4, owner), acc);
        if (c4 == 0) st_cluster_f32x2(map_to_rank(MLrecv + slot * 2, owner), make_float2(M, L));
    }
    cluster_sync_all();                            // release / acquire: what was sent is visible to its owner
    // the CTAs of the cluster, in rank order: this CTA finishes rows rank, rank + C, ... (from its own shared memory)
    const int my_rows = (BM - (int)rank + (int)C - 1) / (int)C;
    for (int e = tid; e < my_rows * (D / 4); e += NT) {
        const int lr = e / (D / 4), c4 = e - lr * (D / 4);
        const int r = (int)rank + lr * (int)C;
        const int row = row0 + r;
        if (row >= nrows) continue;
        float M = -INFINITY;
        for (unsigned k = 0; k < C; ++k) {
            const float2 ml = *reinterpret_cast<const float2*>(MLrecv + (k * rows_per_owner + lr) * 2);
            if (ml.y > 0.f) M = fmaxf(M, ml.x);
        }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (unsigned k = 0; k < C; ++k) {
            const float2 ml = *reinterpret_cast<const float2*>(MLrecv + (k * rows_per_owner + lr) * 2);
            const float f = ml.y > 0.f ? ex2(ml.x - M) : 0.f;
            const float4 v = *reinterpret_cast<const float4*>(Recv + (size_t)(k * rows_per_owner + lr) * LDO + c4 * 4);
            acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
            L += f * ml.y;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        const int tok = row / G, g = row - tok * G;
        __nv_bfloat16* dst = p.out + ((size_t)(q0 + tok) * p.Hq + kvh * G + g) * D + c4 * 4;
        uint2 w;
        w.x = pack_bf16(acc.x * inv, acc.y * inv);
        w.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(dst) = w;
    }
}

template <int D, int RW, int KG>
size_t cluster_smem() {
    return cluster_tile_bytes<D, RW, KG>() + (size_t)(RW * 16 + 16) * (D + 8 + 2) * sizeof(float);
}

// How many clusters of `size` CTAs (a power of two up to 16) the device holds at once; 0: such a cluster cannot
// be placed.  Asked once per kernel and size.
template <int D, int RW, int KG>
int active_clusters(int size) {
    static int cached[5] = {-1, -1, -1, -1, -1};                 // sizes 1, 2, 4, 8, 16
    int slot = 0;
    while ((1 << slot) < size) ++slot;
    if (slot > 4 || (1 << slot) != size) return 0;
    if (cached[slot] >= 0) return cached[slot];
    auto k = paged_attn_cluster_kernel<D, RW, KG>;
    const size_t smem = cluster_smem<D, RW, KG>();
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return cached[slot] = 0; }
    if (cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) cudaGetLastError();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, size); cfg.blockDim = dim3(RW * KG * 32); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = (unsigned)size; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    return cached[slot] = n;
}

template <int D, int RW, int KG>
int launch_cluster(const MmaParams& p, cudaStream_t s) {
    if (active_clusters<D, RW, KG>(p.num_splits) < 1)
        TTIE_FAIL("paged_attention (decode form): the device places no cluster of %d CTAs for this kernel", p.num_splits);
    dim3 grid(p.num_seqs * p.Hkv * p.row_tiles, p.num_splits);
    TTIE_LAUNCH_CLUSTER((paged_attn_cluster_kernel<D, RW, KG>), grid, RW * KG * 32, (cluster_smem<D, RW, KG>()), s, dim3(1, p.num_splits, 1), p);
    TTIE_CHECK_LAUNCH("paged_attention (decode form)");
    return 0;
}

template <int D>
int pick_cluster(const MmaParams& p, int rows, int key_groups, cudaStream_t s) {
    if (rows <= 16) return key_groups >= 4 ? launch_cluster<D, 1, 4>(p, s) : launch_cluster<D, 1, 2>(p, s);
    return key_groups >= 4 ? launch_cluster<D, 2, 4>(p, s) : launch_cluster<D, 2, 2>(p, s);
}
template <int D>
int active_clusters_of(int rows, int key_groups, int size) {
    if (rows <= 16) return key_groups >= 4 ? active_clusters<D, 1, 4>(size) : active_clusters<D, 1, 2>(size);
    return key_groups >= 4 ? active_clusters<D, 2, 4>(size) : active_clusters<D, 2, 2>(size);
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

// CTAs of the tile loop that one SM holds at once (0 if the question fails)
template <int D, int NWARPS>
int resident_per_sm() {
    constexpr int BM = NWARPS * 16, LDS = D + 8, STAGES = NWARPS >= 4 ? 2 : 1;
    const size_t smem = ((size_t)BM * LDS + 2 * STAGES * (size_t)BN * LDS) * sizeof(__nv_bfloat16) + STAGES * BN * sizeof(long long);
    auto k = paged_attn_mma_kernel<D, NWARPS, STAGES>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return 0; }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, NWARPS * 32, smem) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}
template <int D>
int resident_per_sm_of(int rows) { return rows <= 16 ? resident_per_sm<D, 1>() : rows <= 32 ? resident_per_sm<D, 2>() : resident_per_sm<D, 4>(); }

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

// CTAs of the tile loop that one SM holds at once, for this head size and row count per request and kv head.
extern "C" int ttie_attn_mma_ctas_per_sm(int D, int max_q_len, int Hq, int Hkv) {
    const int rows = max_q_len * (Hq / Hkv);
    switch (D) {
        case 16: return resident_per_sm_of<16>(rows);
        case 32: return resident_per_sm_of<32>(rows);
        case 48: return resident_per_sm_of<48>(rows);
        case 64: return resident_per_sm_of<64>(rows);
        case 80: return resident_per_sm_of<80>(rows);
        case 96: return resident_per_sm_of<96>(rows);
        case 112: return resident_per_sm_of<112>(rows);
        case 128: return resident_per_sm_of<128>(rows);
    }
    return 0;
}

// The decode form tiles query rows (tokens x heads per kv head) by at most this many per cluster.
extern "C" int ttie_attn_cluster_tile_rows(int max_q_len, int Hq, int Hkv) { return max_q_len * (Hq / Hkv) <= 16 ? 16 : CL_MAX_ROWS; }
// How many clusters of `size` CTAs (1, 2, 4, 8 or 16: the CTAs over which one request's keys are cut) the device
// holds at once, for this head size, row count per request and number of key groups (2 or 4); 0: none.
extern "C" int ttie_attn_cluster_active(int D, int max_q_len, int Hq, int Hkv, int key_groups, int size) {
    const int rows = max_q_len * (Hq / Hkv);
    switch (D) {
        case 16: return active_clusters_of<16>(rows, key_groups, size);
        case 32: return active_clusters_of<32>(rows, key_groups, size);
        case 48: return active_clusters_of<48>(rows, key_groups, size);
        case 64: return active_clusters_of<64>(rows, key_groups, size);
        case 80: return active_clusters_of<80>(rows, key_groups, size);
        case 96: return active_clusters_of<96>(rows, key_groups, size);
        case 112: return active_clusters_of<112>(rows, key_groups, size);
        case 128: return active_clusters_of<128>(rows, key_groups, size);
    }
    return 0;
}

// form 0: tile loop (prompt portions; decode with caller-chosen splits and a merge kernel).  form 2 or 4: decode form
// with that many key groups; num_splits is then the cluster size and split_len the keys per CTA (no scratch).
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
    if (form == 0 && num_splits > 1 && (split_len <= 0 || split_len % BN || !scratch))
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
    if (form == 2 || form == 4) {
        if (num_splits > 1 && (split_len <= 0 || split_len % BN)) TTIE_FAIL("paged_attention_mma: the split length must be a multiple of %d", BN);
        if (num_splits == 1) p.split_len = 1 << 30;
        const int tile_rows = ttie_attn_cluster_tile_rows(max_q_len, Hq, Hkv);
        p.row_tiles = ceil_div(rows, tile_rows);
        if ((long long)num_seqs * Hkv * p.row_tiles > 2147483647LL) TTIE_FAIL("paged_attention_mma: grid too large");
        cudaStream_t s = (cudaStream_t)stream;
        switch (D) {
            case 16: return pick_cluster<16>(p, rows, form, s);
            case 32: return pick_cluster<32>(p, rows, form, s);
            case 48: return pick_cluster<48>(p, rows, form, s);
            case 64: return pick_cluster<64>(p, rows, form, s);
            case 80: return pick_cluster<80>(p, rows, form, s);
            case 96: return pick_cluster<96>(p, rows, form, s);
            case 112: return pick_cluster<112>(p, rows, form, s);
            case 128: return pick_cluster<128>(p, rows, form, s);
            default: TTIE_FAIL("paged_attention_mma: head size %d", D);
        }
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
