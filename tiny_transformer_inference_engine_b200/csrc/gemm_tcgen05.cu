// bfloat16 matrix product for prompt portions on Blackwell's 5th-generation tensor cores:
// C[M,N] = A[M,K] * W[N,K]^T (+ bias), float32 accumulation in tensor memory.
//
// Structure (persistent: one CTA per SM walks over 128 x BN output tiles; warp-specialised; the
// accumulator is double-buffered in tensor memory so a tile's epilogue overlaps the next tile's products):
//   warp 0   one elected thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the
//            A and W tiles of each 64-wide K block into a ring of shared-memory stages; the warp also
//            allocates and frees the CTA's tensor-memory columns
//   warp 1   one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16) from
//            shared-memory descriptors into the TMEM accumulator and commits each stage back to the
//            producer (tcgen05.commit -> mbarrier) and the finished tile to the epilogue
//   warps 2-5  read the accumulator with tcgen05.ld (each warp its 32 TMEM lanes = 32 output rows),
//            add the bias, round once, and store
// Every mbarrier wait is bounded by a clock deadline; a wait that runs out records a code in the
// error word, the CTA leaves its loops, frees its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
using namespace ttie;

namespace {
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr long long WAIT_CYCLES = 2000000000LL;            // about one second

__device__ int g_tc_error = 0;                             // first failure code of any launch since the last read
__device__ int* g_tc_error_mirror = nullptr;                // the same word in pinned host memory, if the host gave one

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the code recorded) if the phase does not complete within the deadline.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long deadline = clock64() + WAIT_CYCLES;
    while (!mbar_try(bar, parity)) {
        if (clock64() > deadline) {
            atomicCAS(&g_tc_error, 0, code);
            if (g_tc_error_mirror) { *reinterpret_cast<volatile int*>(g_tc_error_mirror) = code; __threadfence_system(); }
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor: K-major tile, rows of 64 bfloat16 (128 bytes) with 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);                // start address
    d |= (uint64_t)1 << 16;                                 // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                 // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                 // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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

struct TcParams {
    void* C; long long ldc;
    const __nv_bfloat16* bias;
    int M, N, K;
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int NACC = (2 * BN <= 512) ? 2 : 1;               // accumulator buffers in tensor memory
    constexpr uint32_t TMEM_COLS = NACC * BN;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 2 * NACC];
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN, num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + BK - 1) / BK;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t accfull0 = smem_u32(&bars[2 * STAGES]), accempty0 = smem_u32(&bars[2 * STAGES + NACC]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < NACC; ++a) { mbar_init(accfull0 + 8 * a, 1); mbar_init(accempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    // Tiles are dealt round-robin to the resident CTAs; M tiles are the fast index, so CTAs that run
    // together share a W tile (read from HBM once) and the activations stay in L2.
    if (warp == 0) {
        if (lane == 0) {
            int kc = 0;                                          // K blocks loaded so far, over all tiles
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    const uint32_t parity = ((kc / STAGES) & 1) ^ 1;
                    if (!mbar_wait(empty0 + 8 * s, parity, 1)) { ok = false; break; }
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(smem + (size_t)s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    tma_load_2d(a_dst, &tmA, full0 + 8 * s, kb * BK, m0);
                    tma_load_2d(b_dst, &tmB, full0 + 8 * s, kb * BK, n0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int kc = 0, lt = 0;                                  // K blocks consumed; tiles done by this CTA
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
                const int ab = lt % NACC;
                const uint32_t use = lt / NACC;
                if (!mbar_wait(accempty0 + 8 * ab, (use & 1) ^ 1, 4)) { ok = false; break; }   // the epilogue has drained this buffer
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(ab * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    if (!mbar_wait(full0 + 8 * s, (kc / STAGES) & 1, 2)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
                    const uint64_t da = umma_desc(a_addr), db = umma_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(tmem_acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, (kb | k) != 0);
                    umma_commit(empty0 + 8 * s);               // the stage may be refilled once these products have read it
                }
                if (ok) umma_commit(accfull0 + 8 * ab);        // the tile is complete once all products have finished
            }
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31
        const int quarter = warp & 3;
        int lt = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const int ab = lt % NACC;
            const uint32_t use = lt / NACC;
            const int row = m0 + quarter * 32 + lane;
            bool ok = mbar_wait(accfull0 + 8 * ab, use & 1, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_acc = tmem_base + (uint32_t)(ab * BN) + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_acc + (uint32_t)(c * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col0 = n0 + c * 32;
                if (row < p.M && col0 < p.N) {
                    OutT* dst = reinterpret_cast<OutT*>(p.C) + (long long)row * p.ldc + col0;
                    const bool full = col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
                    if (full) {
                        if (sizeof(OutT) == 2) {
                            uint32_t packed[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
                                if (p.bias) { a += __bfloat162float(p.bias[col0 + 2 * j]); b += __bfloat162float(p.bias[col0 + 2 * j + 1]); }
                                __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                                packed[j] = *reinterpret_cast<uint32_t*>(&h);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float4 o;
                                o.x = __uint_as_float(v[4 * j]); o.y = __uint_as_float(v[4 * j + 1]);
                                o.z = __uint_as_float(v[4 * j + 2]); o.w = __uint_as_float(v[4 * j + 3]);
                                if (p.bias) {
                                    o.x += __bfloat162float(p.bias[col0 + 4 * j]); o.y += __bfloat162float(p.bias[col0 + 4 * j + 1]);
                                    o.z += __bfloat162float(p.bias[col0 + 4 * j + 2]); o.w += __bfloat162float(p.bias[col0 + 4 * j + 3]);
                                }
                                reinterpret_cast<float4*>(dst)[j] = o;
                            }
                        }
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                            float a = __uint_as_float(v[j]);
                            if (p.bias) a += __bfloat162float(p.bias[col0 + j]);
                            dst[j] = from_f32<OutT>(a);
                        }
                    }
                }
            }
            // hand the accumulator buffer back to the issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(accempty0 + 8 * ab) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D map over a row-major [rows][K] bfloat16 matrix with row stride ld; box = 64 (K) x box_rows.
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) TTIE_FAIL("gemm_tc: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TTIE_FAIL("gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int BN, int STAGES, typename OutT>
int launch(const CUtensorMap& a, const CUtensorMap& b, const TcParams& p, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
    auto k = gemm_tc_kernel<BN, STAGES, OutT>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TTIE_FAIL("gemm_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    const int tiles = ceil_div(p.M, BM) * ceil_div(p.N, BN);
    k<<<tiles < num_sms() ? tiles : num_sms(), 192, smem, s>>>(a, b, p);
    TTIE_CHECK_LAUNCH("gemm_tc");
    return 0;
}
}  // namespace

// Reads and clears the error word of the tensor-core kernels (0: none; 1 producer, 2 issuer, 3 epilogue
// wait ran out).  Synchronises the device.
// A word of pinned host memory (device-accessible) that also receives the failure code, so the host can look at it
// after every step without a call into the runtime.  nullptr: none.
static int* h_tc_error_mirror = nullptr;                       // host copy of the pointer the device holds
extern "C" int ttie_gemm_tc_set_mirror(int* host_word) {
    h_tc_error_mirror = host_word;
    return cudaMemcpyToSymbol(g_tc_error_mirror, &host_word, sizeof(int*)) == cudaSuccess ? 0 : 1;
}

namespace ttie {
// For the other product kernels of this library (other files): the device address of the error word, the host mirror's
// address (or nullptr), and the tensor-map builder.
int gemm_tc_error_words(int** word, int** mirror) {
    static int* addr[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!addr[dev] && cudaGetSymbolAddress((void**)&addr[dev], g_tc_error) != cudaSuccess) return -1;
    *word = addr[dev];
    *mirror = h_tc_error_mirror;
    return 0;
}
int gemm_tc_make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    return make_map(map, base, rows, K, ld, box_rows);
}
}  // namespace ttie

extern "C" int ttie_tc_error() {
    int v = 0, zero = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}

// C[M,N] = A[M,K] * W[N,K]^T (+ bias).  A, W bfloat16 with row strides lda, ldw (multiples of 8, 16-byte aligned
// bases); out_f32 selects float32 output.  tile_n: 128 or 256.
extern "C" int ttie_gemm_tc(const void* A, long long lda, const void* W, long long ldw, const void* bias, void* C,
                            long long ldc, int M, int N, int K, int out_f32, int tile_n, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) TTIE_FAIL("gemm_tc: K and the row strides must be positive multiples of 8");
    if (((uintptr_t)A | (uintptr_t)W) & 15) TTIE_FAIL("gemm_tc: operand pointers must be 16-byte aligned");
    if (tile_n != 128 && tile_n != 256) TTIE_FAIL("gemm_tc: tile_n must be 128 or 256");
    CUtensorMap ma, mb;
    if (make_map(&ma, A, M, K, lda, BM)) return -1;
    if (make_map(&mb, W, N, K, ldw, tile_n)) return -1;
    TcParams p;
    p.C = C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias; p.M = M; p.N = N; p.K = K;
    cudaStream_t s = (cudaStream_t)stream;
    if (tile_n == 256) return out_f32 ? launch<256, 4, float>(ma, mb, p, s) : launch<256, 4, __nv_bfloat16>(ma, mb, p, s);
    return out_f32 ? launch<128, 6, float>(ma, mb, p, s) : launch<128, 6, __nv_bfloat16>(ma, mb, p, s);
}
