// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
// Plain FFMA with float32 accumulation - no tensor cores, no TF32 - so that the float32
// path shows faults that reduced precision would hide.  Any M, N, K.
// Two kernels: a 64 x 64 tile for prompt portions, and for up to 16 rows (decode steps) a form that streams the weight
// matrix once: a warp owns four weight rows at a time, its lanes walk K in 16-byte steps, and the activations - a few
// rows that every warp reads - come through the cache.
#include "common.cuh"
using namespace ttie;

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;      // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread; k is the fast index in memory
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
        }
    }
}
// ---- up to 16 activation rows.  acc[m][r]: lane-partial dot product of activation row m with weight row r of the warp's
// four; the lanes' partial sums are added by shuffles in a fixed order.  Rows of 4-element-aligned length and stride only.
constexpr int GV_WARPS = 8, GV_ROWS = 4;
template <int MT>
__global__ void __launch_bounds__(GV_WARPS * 32, MT <= 8 ? 3 : 1)     // (a long matrix streams best with many warps per SM)
gemv_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_ROWS;
    if (n0 >= N) return;
    const float* wrow[GV_ROWS];
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) wrow[r] = W + (size_t)min(n0 + r, N - 1) * ldw;       // (a row past the end repeats the last one; it is not stored)
    float acc[MT][GV_ROWS];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) acc[m][r] = 0.f;
    TTIE_PDL_ENTRY();
#pragma unroll(MT <= 4 ? 2 : 1)
    for (int k = lane * 4; k < K; k += 128) {
        float4 w[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) w[r] = __ldcs(reinterpret_cast<const float4*>(wrow[r] + k));   // streamed once
        // all activation loads of the step are asked for at once (a row past the last repeats it and is not stored): every
        // one of them is new to this SM's cache, and one after the other they would cost a trip to L2 each
        float4 x[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) x[m] = __ldg(reinterpret_cast<const float4*>(A + (size_t)min(m, M - 1) * lda + k));
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r)
                acc[m][r] = fmaf(x[m].w, w[r].w, fmaf(x[m].z, w[r].z, fmaf(x[m].y, w[r].y, fmaf(x[m].x, w[r].x, acc[m][r]))));
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            float v = acc[m][r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[m][r] = v;
        }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r)
                if (m < M && n0 + r < N) C[(size_t)m * ldc + n0 + r] = acc[m][r] + (bias ? bias[n0 + r] : 0.f);
    }
}

template <int MT>
int launch_gemv(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda, int ldw, int ldc, cudaStream_t s) {
    TTIE_LAUNCH(gemv_f32_kernel<MT>, ceil_div(N, GV_WARPS * GV_ROWS), GV_WARPS * 32, 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc);
    TTIE_CHECK_LAUNCH("gemm_f32 (few rows)");
    return 0;
}
}  // namespace

extern "C" int ttie_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                             int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) TTIE_FAIL("gemm_f32: K must be positive, got %d", K);
    if (M <= 32 && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0) {
        cudaStream_t s = (cudaStream_t)stream;
        if (M <= 2) return launch_gemv<2>(A, W, bias, C, M, N, K, lda, ldw, ldc, s);
        if (M <= 4) return launch_gemv<4>(A, W, bias, C, M, N, K, lda, ldw, ldc, s);
        if (M <= 8) return launch_gemv<8>(A, W, bias, C, M, N, K, lda, ldw, ldc, s);
        // 17 to 32 rows: twice 16 (measured against the tile kernel at 32 rows: 13 against 38 us on a [512, 512] matrix,
        // 137 against 170 on [50257, 512])
        for (int m0 = 0; m0 < M; m0 += 16) {
            const int rc = launch_gemv<16>(A + (size_t)m0 * lda, W, bias, C + (size_t)m0 * ldc, M - m0 < 16 ? M - m0 : 16, N, K, lda, ldw, ldc, s);
            if (rc) return rc;
        }
        return 0;
    }
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    if (grid.y > 65535) TTIE_FAIL("gemm_f32: M=%d too large for one launch", M);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
    TTIE_CHECK_LAUNCH("gemm_f32");
    return 0;
}
