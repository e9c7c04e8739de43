// bfloat16 matrix product for prompt portions on pairs of SMs:
// C[M,N] = A[M,K] * W[N,K]^T (+ bias), or silu(A Wg^T) * (A Wu^T) for the gate/up pair, float32 accumulation in
// tensor memory.
//
// Two CTAs (a thread-block cluster of 2, on neighbouring SMs) own one 256 x 256 output tile and share its operands:
// each CTA copies 128 rows of A and 128 rows of W per 64-wide K block into its own shared memory, and the leader's
// tensor-core instruction (tcgen05.mma.cta_group::2, M = 256, N = 256, K = 16) reads both halves of W from both CTAs
// and each CTA's half of A, and writes each CTA's 128 x 256 half of the accumulator into that CTA's tensor memory.
// Per product a CTA therefore brings in 32 KB instead of the 48 KB a lone 128 x 256 tile needs - the operand stream
// through L2 is what bounds the one-CTA kernel (gemm_tcgen05.cu).
//
//   warp 0   (both CTAs) one thread copies this CTA's operand halves (cp.async.bulk.tensor.2d.cta_group::2, 128-byte
//            swizzle, no multicast) through a ring of stages; the bytes of both CTAs are counted on the leader's
//            barrier.  The warp also allocates and frees the pair's tensor memory (a collective of both CTAs).
//   warp 1   (leader only) one thread issues the products and hands stages back to both producers and finished tiles
//            to both epilogues with tcgen05.commit ... .multicast::cluster
//   warps 2-5  (both CTAs) read this CTA's half of the accumulator (tcgen05.ld), apply the epilogue and store; the
//            accumulator is double-buffered, so a tile's epilogue overlaps the next tile's products
// SwiGLU epilogue: W holds the gate rows [0, F) and then the up rows [F, 2F).  The leader copies 128 gate rows and its
// peer the matching 128 up rows, so accumulator column j is gate column j and column 128 + j its up column, and the
// epilogue writes silu(g) * u (models/mlp.py:24-32; silu in 32-bit as kernels/fused_swiglu/kernel.py:20-25) without
// the [T, 2F] round trip through memory.
// Every mbarrier wait is bounded by a clock deadline; a wait that runs out records a code in the error word of the
// tensor-core product kernels and the CTA leaves its loops; both CTAs meet at the end before tensor memory is freed.
#include "common.cuh"
#include <cuda.h>
using namespace ttie;

namespace ttie {
// the error word of the tensor-core product kernels, its mirror in pinned host memory, and the tensor-map builder
// (gemm_tcgen05.cu)
int gemm_tc_error_words(int** word, int** mirror);
int gemm_tc_make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows);
}  // namespace ttie

namespace {
constexpr int HM = 128, HN = 128, BK = 64, UMMA_K = 16;          // a CTA's halves of the 256 x 256 tile
constexpr long long WAIT_CYCLES = 2000000000LL;                 // about one second
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;                     // clears the bit that tells the pair's CTAs apart: the leader's address

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {       // on the leader's copy of this barrier
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_MASK) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
struct ErrorWords { int* word; int* mirror; };
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code, const ErrorWords& e) {
    if (mbar_try(bar, parity)) return true;
    const long long deadline = clock64() + WAIT_CYCLES;
    while (!mbar_try(bar, parity)) {
        if (clock64() > deadline) {
            atomicCAS(e.word, 0, code);
            if (e.mirror) { *reinterpret_cast<volatile int*>(e.mirror) = code; __threadfence_system(); }
            return false;
        }
    }
    return true;
}
// this CTA's tile into its own shared memory; the bytes are counted on the leader's barrier
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & PEER_MASK), "r"(x), "r"(y) : "memory");
}
// K-major tile, rows of 64 bfloat16 (128 bytes) with 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives, once the products issued so far have finished, on the barrier at this address in both CTAs of the pair
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct PairParams {
    void* C; long long ldc;
    const __nv_bfloat16* bias;
    int M, N, K;              // N: output columns (SwiGLU: F)
    int up_offset;            // SwiGLU: row of W (and entry of bias) where the up projection starts
    ErrorWords err;           // where a wait that runs out leaves its code
};

// EPI 0: C = A W^T (+ bias) as OutT; EPI 1: C = silu(A Wg^T + bg) * (A Wu^T + bu) as bfloat16 (OutT)
// KPS: 64-wide K blocks per stage of the ring (one barrier round trip of the issuing thread per stage)
template <int STAGES, int KPS, int EPI, typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PairParams p) {
    constexpr uint32_t A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2, BLOCK_BYTES = A_BYTES + B_BYTES, STAGE_BYTES = KPS * BLOCK_BYTES;
    constexpr int TILE_N = EPI == 1 ? HN : 2 * HN;               // output columns of a tile
    constexpr uint32_t ACC_COLS = 2 * HN, TMEM_COLS = 2 * ACC_COLS;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned rank;
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (p.M + 2 * HM - 1) / (2 * HM), tiles_n = (p.N + TILE_N - 1) / TILE_N, num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + KPS * BK - 1) / (KPS * BK);        // stages per tile
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t accfull0 = smem_u32(&bars[2 * STAGES]), accempty0 = smem_u32(&bars[2 * STAGES + 2]);

    if (threadIdx.x == 0) {
        // full: the leader's own arrival (with the byte count of both CTAs); empty, accfull: one commit; accempty (the
        // leader's is used): the four epilogue warps of both CTAs
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accfull0 + 8 * a, 1); mbar_init(accempty0 + 8 * a, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                          // the peer's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    // Tiles are dealt round-robin to the resident pairs; M tiles are the fast index, so pairs that run together share a
    // W tile (read from HBM once) and the activations stay in L2.
    if (warp == 0) {
        if (lane == 0) {
            int kc = 0;
            for (int tile = pair; tile < num_tiles; tile += num_pairs) {
                const int m0 = (tile % tiles_m) * (2 * HM) + (int)rank * HM;
                const int tn = tile / tiles_m;
                const int w0 = EPI == 1 ? (int)rank * p.up_offset + tn * HN : tn * (2 * HN) + (int)rank * HN;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    if (!mbar_wait(empty0 + 8 * s, ((kc / STAGES) & 1) ^ 1, 21, p.err)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
#pragma unroll
                    for (int q = 0; q < KPS; ++q) {              // (a block past the end of K is filled with zeros)
                        const uint32_t a_dst = smem_u32(smem + (size_t)s * STAGE_BYTES + q * BLOCK_BYTES), b_dst = a_dst + A_BYTES;
                        tma_load_pair(a_dst, &tmA, full0 + 8 * s, (kb * KPS + q) * BK, m0);
                        tma_load_pair(b_dst, &tmB, full0 + 8 * s, (kb * KPS + q) * BK, w0);
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 256 (over the pair)
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * HN) >> 3) << 17) | ((uint32_t)((2 * HM) >> 4) << 24);
            int kc = 0, lt = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++lt) {
                const int ab = lt & 1;
                if (!mbar_wait(accempty0 + 8 * ab, ((lt >> 1) & 1) ^ 1, 24, p.err)) { ok = false; break; }   // both epilogues have drained this buffer
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(ab * ACC_COLS);
                for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    if (!mbar_wait(full0 + 8 * s, (kc / STAGES) & 1, 22, p.err)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < KPS; ++q) {
                        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES + q * BLOCK_BYTES), b_addr = a_addr + A_BYTES;
                        const uint64_t da = umma_desc(a_addr), db = umma_desc(b_addr);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_pair(tmem_acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, (kb | q | k) != 0);
                    }
                    umma_commit_both(empty0 + 8 * s);           // both producers may refill the stage once these products have read it
                }
                if (ok) umma_commit_both(accfull0 + 8 * ab);    // both epilogues: the tile is complete
            }
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31 = rows of this CTA's half of the tile
        const int quarter = warp & 3;
        int lt = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
            const int m0 = (tile % tiles_m) * (2 * HM) + (int)rank * HM, n0 = (tile / tiles_m) * TILE_N;
            const int ab = lt & 1;
            const int row = m0 + quarter * 32 + lane;
            bool ok = mbar_wait(accfull0 + 8 * ab, (lt >> 1) & 1, 23, p.err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_acc = tmem_base + (uint32_t)(ab * ACC_COLS) + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < TILE_N / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_acc + (uint32_t)(c * 32), v);
                if (EPI == 1) {
                    uint32_t u[32];
                    tmem_ld32(tmem_acc + (uint32_t)(HN + c * 32), u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float g = __uint_as_float(v[j]), up = __uint_as_float(u[j]);
                        if (p.bias) {
                            const int col = min(n0 + c * 32 + j, p.N - 1);
                            g += __bfloat162float(p.bias[col]); up += __bfloat162float(p.bias[p.up_offset + col]);
                        }
                        v[j] = __float_as_uint(g / (1.f + __expf(-g)) * up);
                    }
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(p.bias[min(n0 + c * 32 + j, p.N - 1)]));
                    }
                }
                const int col0 = n0 + c * 32;
                if (row < p.M && col0 < p.N) {
                    OutT* dst = reinterpret_cast<OutT*>(p.C) + (long long)row * p.ldc + col0;
                    const bool full = col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
                    if (full) {
                        if (sizeof(OutT) == 2) {
                            uint32_t packed[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                                packed[j] = *reinterpret_cast<uint32_t*>(&h);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<float4*>(dst)[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                                                __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        }
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = from_f32<OutT>(__uint_as_float(v[j]));
                    }
                }
            }
            // hand the accumulator buffer back to the issuer (the leader's barrier counts the warps of both CTAs)
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) mbar_arrive_leader(accempty0 + 8 * ab);
        }
    }
    // Nobody leaves before both CTAs are done: the leader's products read the peer's shared memory, the peer's warps
    // arrive on the leader's barriers, and the tensor memory of the pair is freed together.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int STAGES, int KPS, int EPI, typename OutT>
int launch(const CUtensorMap& a, const CUtensorMap& b, const PairParams& p, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * KPS * (HM * BK * 2 + HN * BK * 2) + 1024;
    auto k = gemm_tc_pair_kernel<STAGES, KPS, EPI, OutT>;
    static bool allowed[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!allowed[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) TTIE_FAIL("gemm_tc_pair: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        allowed[dev] = true;
    }
    const int tile_n = EPI == 1 ? HN : 2 * HN;
    const int tiles = ceil_div(p.M, 2 * HM) * ceil_div(p.N, tile_n);
    const int pairs = tiles < num_sms() / 2 ? tiles : num_sms() / 2;
    cudaError_t e = launch_kernel(k, dim3(2 * pairs), dim3(192), smem, s, dim3(2, 1, 1), a, b, p);
    if (e != cudaSuccess) TTIE_FAIL("gemm_tc_pair: launch failed: %s", cudaGetErrorString(e));
    return 0;
}
}  // namespace

// C[M,N] = A[M,K] * W[N,K]^T (+ bias) on pairs of CTAs.  A, W bfloat16 with row strides lda, ldw (multiples of 8,
// 16-byte aligned bases); out_f32 selects float32 output.
// swiglu != 0: W is [2F, K] (gate rows, then up rows), N = F, C[M, F] = silu(A Wg^T) * (A Wu^T) in bfloat16.
extern "C" int ttie_gemm_tc_pair(const void* A, long long lda, const void* W, long long ldw, const void* bias, void* C,
                                 long long ldc, int M, int N, int K, int out_f32, int swiglu, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) TTIE_FAIL("gemm_tc_pair: K and the row strides must be positive multiples of 8");
    if (((uintptr_t)A | (uintptr_t)W) & 15) TTIE_FAIL("gemm_tc_pair: operand pointers must be 16-byte aligned");
    if (swiglu && out_f32) TTIE_FAIL("gemm_tc_pair: the SwiGLU epilogue writes bfloat16");
    CUtensorMap ma, mb;
    if (gemm_tc_make_map(&ma, A, M, K, lda, HM)) return -1;
    if (gemm_tc_make_map(&mb, W, swiglu ? 2LL * N : N, K, ldw, HN)) return -1;
    PairParams p;
    p.C = C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias; p.M = M; p.N = N; p.K = K; p.up_offset = swiglu ? N : 0;
    if (gemm_tc_error_words(&p.err.word, &p.err.mirror)) TTIE_FAIL("gemm_tc_pair: the error word's address is not to be had");
    cudaStream_t s = (cudaStream_t)stream;
    // (measured at 2,048 rows: two K blocks per stage with three stages, or seven stages, change nothing - the issuing
    // thread's barrier round trips are not what bounds this kernel)
    if (swiglu) return launch<6, 1, 1, __nv_bfloat16>(ma, mb, p, s);
    return out_f32 ? launch<6, 1, 0, float>(ma, mb, p, s) : launch<6, 1, 0, __nv_bfloat16>(ma, mb, p, s);
}
