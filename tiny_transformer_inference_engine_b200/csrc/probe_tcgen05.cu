// Timing probe for the tensor-core kernels' issuing threads: how long one thread's stream of tcgen05.mma takes, by
// shape and operand source, and which of the instructions that follow it wait for the products to finish.
// The kernels' structure rests on what this measures (one issuing thread per independent product chain), so it is
// kept with them: `python -m tiny_transformer_inference_engine_b200.ops.microbench --what issue`.
// Operands are whatever shared and tensor memory hold; only clocks are reported.  Every wait is bounded.
#include "common.cuh"
using namespace ttie;

namespace {
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);    // 8-row groups 1024 bytes apart, sm_100 descriptor, 128-byte swizzle
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
template <bool ACC>
__device__ __forceinline__ void umma_ss(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
                 ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const long long deadline = clock64() + 200000000LL;           // a tenth of a second
    while (!mbar_try(bar, parity)) if (clock64() > deadline) return false;
    return true;
}

// after: what follows every batch of 8 products in the issuing thread
//   0 nothing   1 tcgen05.commit   2 commit + wait for that commit   3 commit + wait on a barrier that completed long ago
//   4 commit + tcgen05.fence::after_thread_sync   5 commit + poll of a shared-memory flag that is set
//   6 as 3, with a second thread (another warp) doing the same into an accumulator of its own
template <int N, bool ATMEM, int AFTER>
__global__ void __launch_bounds__(128, 1) issue_probe_kernel(int batches, long long* out) {
    constexpr int after = AFTER;
    extern __shared__ unsigned char dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bars[5];
    __shared__ uint32_t slot;
    __shared__ volatile int flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
    const uint32_t bar0 = smem_u32(&bars[0]);
    if (threadIdx.x == 0) {
        flag = 1;
        for (int i = 0; i < 5; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8 * i), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar0 + 8) : "memory");      // bars[1]: phase 0 is over for good
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = slot;
    const bool issuer = lane == 0 && (warp == 1 || (warp == 2 && after == 6));
    if (issuer) {
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        // A: 128 rows x 128 columns (two 64-column blocks of 16 KB); B: up to 256 rows (two blocks of 32 KB)
        const uint32_t a_lo = desc_lo(smem_u32(smem)), b_lo = desc_lo(smem_u32(smem + 32 * 1024));
        const uint32_t acc = tm + (warp == 2 ? 128u : 0u);       // the second thread's products are 64 wide in every instantiation used with after == 6
        const uint32_t mine = bar0 + (warp == 2 ? 16u : 0u), last = bar0 + (warp == 2 ? 32u : 24u);
        bool ok = true;
        const long long t0 = clock64();
        for (int r = 0; r < batches && ok; ++r) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t a_off = (k >> 2) * 1024 + (k & 3) * 2, b_off = (k >> 2) * 2048 + (k & 3) * 2;   // 8 K steps over the two blocks, in 16-byte units
                if (ATMEM) { if (k) umma_ts<true>(acc, tm + 256 + k * 8, b_lo + b_off, idesc); else umma_ts<false>(acc, tm + 256, b_lo, idesc); }
                else { if (k) umma_ss<true>(acc, a_lo + a_off, b_lo + b_off, idesc); else umma_ss<false>(acc, a_lo, b_lo, idesc); }
            }
            if (after >= 1) commit(mine);
            if (after == 2) ok = mbar_wait(mine, r & 1);
            if (after == 3 || after == 6) ok = mbar_wait(bar0 + 8, 0);
            if (after == 4) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (after == 5) { const long long dl = clock64() + 200000000LL; while (flag == 0) if (clock64() > dl) { ok = false; break; } }
        }
        const long long t1 = clock64();
        commit(last);
        const bool fin = mbar_wait(last, 0);
        const long long t2 = clock64();
        if (blockIdx.x == 0 && warp == 1) { out[0] = t1 - t0; out[1] = (ok && fin) ? t2 - t0 : -1; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
}

template <int N, bool ATMEM, int AFTER>
int launch_probe(int batches, long long* out, cudaStream_t s) {
    const size_t smem = 98 * 1024;
    auto k = issue_probe_kernel<N, ATMEM, AFTER>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TTIE_FAIL("issue probe: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    k<<<148, 128, smem, s>>>(batches, out);
    TTIE_CHECK_LAUNCH("issue probe");
    return 0;
}
}  // namespace

// Runs `batches` batches of 8 products [128 x N x 16] (A from shared or tensor memory) on every SM and writes, for
// the first CTA, out[0] = clocks until the last product was issued and out[1] = clocks until all had finished
// (-1 if a wait ran out).  out: two 64-bit integers in device memory.  `after` other than 0 is built for 64-wide
// products from shared memory.
extern "C" int ttie_probe_mma_issue(int n, int a_in_tmem, int after, int batches, long long* out, void* stream) {
    if (after < 0 || after > 6 || batches <= 0) TTIE_FAIL("issue probe: after must be 0..6 and batches positive");
    if (after && (n != 64 || a_in_tmem)) TTIE_FAIL("issue probe: what follows a batch is varied only for 64-wide products from shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    if (a_in_tmem) {
        if (n == 64) return launch_probe<64, true, 0>(batches, out, s);
        if (n == 128) return launch_probe<128, true, 0>(batches, out, s);
    } else {
        if (n == 64) {
            switch (after) {
                case 0: return launch_probe<64, false, 0>(batches, out, s);
                case 1: return launch_probe<64, false, 1>(batches, out, s);
                case 2: return launch_probe<64, false, 2>(batches, out, s);
                case 3: return launch_probe<64, false, 3>(batches, out, s);
                case 4: return launch_probe<64, false, 4>(batches, out, s);
                case 5: return launch_probe<64, false, 5>(batches, out, s);
                default: return launch_probe<64, false, 6>(batches, out, s);
            }
        }
        if (n == 128) return launch_probe<128, false, 0>(batches, out, s);
        if (n == 256) return launch_probe<256, false, 0>(batches, out, s);
    }
    TTIE_FAIL("issue probe: products %d wide with A in %s memory are not built", n, a_in_tmem ? "tensor" : "shared");
}
