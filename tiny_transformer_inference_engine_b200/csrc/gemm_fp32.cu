// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
// Plain FFMA with float32 accumulation - no tensor cores, no TF32 - so that the float32
// path shows faults that reduced precision would hide.  Any M, N, K.
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
}  // namespace

extern "C" int ttie_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                             int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) TTIE_FAIL("gemm_f32: K must be positive, got %d", K);
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    if (grid.y > 65535) TTIE_FAIL("gemm_f32: M=%d too large for one launch", M);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
    TTIE_CHECK_LAUNCH("gemm_f32");
    return 0;
}
