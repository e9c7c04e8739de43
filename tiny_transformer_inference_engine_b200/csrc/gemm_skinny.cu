// Weight-streaming matrix product for decode steps: out[M,N] = x[M,K] * W[N,K]^T with few rows
// (M <= 64), bfloat16 in, float32 accumulation.  Such a product is bound by reading W once from
// HBM; the library product launches too few CTAs for the narrow projections (N ~ 4096) to keep
// HBM busy.  Here the weight matrix takes the tensor core's M side (swap-AB): a CTA owns 16 rows
// of W, its four warps split the K range among themselves (and, optionally, CTAs split K further:
// blockIdx.y), every lane streams 16-byte pieces of its two weight rows straight from global
// memory into mma.sync A fragments, and the few activation rows ride as the B operand.
//
// Fragment trick: the sum over k does not care about order, so a lane's 16-byte load (8 consecutive
// k of one row) feeds two m16n8k16 steps; the activation fragment is cut from the same 8 k, so
// both operands agree on which k sits where and no shuffle or shared-memory staging is needed.
//
// Epilogues: (0) bfloat16 out (+bias); (1) float32 partial sums per K split, [S][M][N], for a
// consumer that adds them (add_rmsnorm, rope_store_partial) in a fixed order - so results do not
// depend on timing; (2) SwiGLU: the CTA streams gate rows n and up rows n+F together and writes
// silu(g)*u (models/mlp.py:24-32; silu in 32-bit as kernels/fused_swiglu/kernel.py:20-25);
// (3) float32 out (logits).
#include "common.cuh"
using namespace ttie;

namespace {
struct SkinnyParams {
    const __nv_bfloat16* x; long long ldx;
    const __nv_bfloat16* w; long long ldw;
    const __nv_bfloat16* bias;
    void* out; long long ldo;
    int M, N, K;
    int kslice;            // K range of one CTA (multiple of 128)
    int up_offset;         // SwiGLU: row offset of the up projection inside w (and bias)
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// SETS: sets of 16 weight rows per CTA for the plain epilogues.  Every set is multiplied with the same activation
// fragments, so the activations - which every CTA fetches for itself, through the caches - cost half as much per weight
// byte with two sets (SwiGLU has always had two: its gate rows and its up rows).
template <int MT, int EPI, int U, int SETS>
__global__ void __launch_bounds__(128)
skinny_gemm_kernel(const SkinnyParams p) {
    constexpr int NSET = EPI == 2 ? 2 : SETS;                    // SwiGLU streams two row sets: gate and up
    __shared__ float red[4][NSET][MT][32][4];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, q = lane & 3;
    const int n0 = blockIdx.x * 16 * (EPI == 2 ? 1 : SETS);
    const int set_stride = EPI == 2 ? p.up_offset : 16;           // rows from one set to the next
    const int split = blockIdx.y;
    const int kq = p.kslice / 4;
    const int k_begin = split * p.kslice + warp * kq;
    const int k_end = min(p.K, min((split + 1) * p.kslice, k_begin + kq));

    float acc[NSET][MT][4];
#pragma unroll
    for (int s = 0; s < NSET; ++s)
#pragma unroll
        for (int j = 0; j < MT; ++j) { acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f; }

    // (SwiGLU: N counts the gate rows, and an up row exists wherever its gate row does)
    bool row_a[NSET], row_b[NSET];
    const __nv_bfloat16* wrow[NSET][2];
#pragma unroll
    for (int s = 0; s < NSET; ++s) {
        const int in_n = n0 + r + (EPI == 2 ? 0 : s * 16);
        row_a[s] = in_n < p.N; row_b[s] = in_n + 8 < p.N;
        const long long base = (long long)(n0 + r + s * set_stride);
        wrow[s][0] = p.w + (row_a[s] ? base : 0) * p.ldw;
        wrow[s][1] = p.w + (row_b[s] ? base + 8 : 0) * p.ldw;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // Two register buffers: the loads of the next 32*U keys are in flight while the current ones
    // feed the tensor core, so every warp always has weight bytes on their way from HBM.  The weights
    // do not depend on the kernel before this one, so the first loads of both buffers are issued
    // before the wait for that kernel's results: the stream from HBM ramps up while it drains.
    uint4 wA[U][NSET][2], xA[U][MT], wB[U][NSET][2], xB[U][MT];
    auto load_w = [&](int k0, uint4 (&wv)[U][NSET][2]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k0 + 32 * u + 8 * q;
            const bool ok = kk < k_end;
#pragma unroll
            for (int s = 0; s < NSET; ++s) {
                wv[u][s][0] = (ok && row_a[s]) ? ld_stream(wrow[s][0] + kk) : zero;
                wv[u][s][1] = (ok && row_b[s]) ? ld_stream(wrow[s][1] + kk) : zero;
            }
        }
    };
    auto load_x = [&](int k0, uint4 (&xv)[U][MT]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k0 + 32 * u + 8 * q;
            const bool ok = kk < k_end;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const int m = 8 * j + r;
                xv[u][j] = (ok && m < p.M) ? __ldg(reinterpret_cast<const uint4*>(p.x + (long long)m * p.ldx + kk)) : zero;
            }
        }
    };
    auto compute = [&](const uint4 (&wv)[U][NSET][2], const uint4 (&xv)[U][MT]) {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int s = 0; s < NSET; ++s)
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    mma_bf16(acc[s][j], wv[u][s][0].x, wv[u][s][1].x, wv[u][s][0].y, wv[u][s][1].y, xv[u][j].x, xv[u][j].y);
                    mma_bf16(acc[s][j], wv[u][s][0].z, wv[u][s][1].z, wv[u][s][0].w, wv[u][s][1].w, xv[u][j].z, xv[u][j].w);
                }
    };
    load_w(k_begin, wA);                                       // (loads past k_end give zeros)
    load_w(k_begin + 32 * U, wB);
    TTIE_PDL_ENTRY();                                          // the activations are the predecessor's output
    load_x(k_begin, xA);
    load_x(k_begin + 32 * U, xB);
    for (int k0 = k_begin; k0 < k_end; k0 += 64 * U) {
        compute(wA, xA);
        if (k0 + 64 * U < k_end) { load_w(k0 + 64 * U, wA); load_x(k0 + 64 * U, xA); }
        if (k0 + 32 * U < k_end) {
            compute(wB, xB);
            if (k0 + 96 * U < k_end) { load_w(k0 + 96 * U, wB); load_x(k0 + 96 * U, xB); }
        }
    }

    // sum the four warps' K ranges in a fixed order
#pragma unroll
    for (int s = 0; s < NSET; ++s)
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) red[warp][s][j][lane][c] = acc[s][j][c];
    __syncthreads();
    const int c = warp;                                         // thread (lane, c) finishes accumulator element c of `lane`
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        const int m = 8 * j + 2 * q + (c & 1);
        float v[NSET];
#pragma unroll
        for (int s = 0; s < NSET; ++s)
            v[s] = ((red[0][s][j][lane][c] + red[1][s][j][lane][c]) + red[2][s][j][lane][c]) + red[3][s][j][lane][c];
        if (m >= p.M) continue;
        if (EPI == 2) {
            const int row = n0 + r + 8 * (c >> 1);
            if (row >= p.N) continue;
            const float g = v[0] + (p.bias ? __bfloat162float(p.bias[row]) : 0.f);
            const float u = v[NSET - 1] + (p.bias ? __bfloat162float(p.bias[row + p.up_offset]) : 0.f);
            reinterpret_cast<__nv_bfloat16*>(p.out)[(long long)m * p.ldo + row] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
            continue;
        }
#pragma unroll
        for (int s = 0; s < NSET; ++s) {
            const int row = n0 + 16 * s + r + 8 * (c >> 1);
            if (row >= p.N) continue;
            if (EPI == 0) {
                const float b = p.bias ? __bfloat162float(p.bias[row]) : 0.f;
                reinterpret_cast<__nv_bfloat16*>(p.out)[(long long)m * p.ldo + row] = __float2bfloat16_rn(v[s] + b);
            } else if (EPI == 1) {
                reinterpret_cast<float*>(p.out)[((long long)split * p.M + m) * p.ldo + row] = v[s];
            } else {
                const float b = p.bias ? __bfloat162float(p.bias[row]) : 0.f;
                reinterpret_cast<float*>(p.out)[(long long)m * p.ldo + row] = v[s] + b;
            }
        }
    }
}

template <int MT, int EPI, int U, int SETS>
int launch(const SkinnyParams& p, int splits, cudaStream_t s) {
    dim3 grid(ceil_div(p.N, 16 * (EPI == 2 ? 1 : SETS)), splits);
    TTIE_LAUNCH((skinny_gemm_kernel<MT, EPI, U, SETS>), grid, 128, 0, s, p);
    TTIE_CHECK_LAUNCH("skinny_gemm");
    return 0;
}

template <int EPI>
int dispatch(const SkinnyParams& p, int splits, int unroll, cudaStream_t s) {
    // unroll: low four bits 0 (chosen here), 2 or 4; + 16 asks for two row sets per CTA (plain epilogues)
    const bool two = EPI != 2 && (unroll & 16);
    unroll &= 15;
    const int mt = ceil_div(p.M, 8);
    // a product that is not split over CTAs streams best with deep unrolling, a split one with more CTAs per SM
    const bool deep = EPI != 2 && (unroll ? unroll >= 4 : splits == 1);
    if (two) {
        if (mt <= 1) return deep ? launch<1, EPI, 2, 2>(p, splits, s) : launch<1, EPI, 1, 2>(p, splits, s);
        if (mt <= 2) return launch<2, EPI, 1, 2>(p, splits, s);
        if (mt <= 4) return launch<4, EPI, 1, 2>(p, splits, s);
        return launch<8, EPI, 1, 1>(p, splits, s);
    }
    if (mt <= 1) return deep ? launch<1, EPI, 4, 1>(p, splits, s) : launch<1, EPI, (EPI == 2 ? 1 : 2), 1>(p, splits, s);
    if (mt <= 2) return launch<2, EPI, (EPI == 2 ? 1 : 2), 1>(p, splits, s);
    if (mt <= 4) return launch<4, EPI, (EPI == 2 ? 1 : 2), 1>(p, splits, s);
    return launch<8, EPI, 1, 1>(p, splits, s);
}
}  // namespace

extern "C" int ttie_skinny_max_rows() { return 64; }

// epilogue: 0 bfloat16 out, 1 float32 partial sums [splits][M][N], 2 SwiGLU (w holds gate rows then up
// rows, N = F), 3 float32 out.  kslice: K range per CTA, a multiple of 128; splits = ceil(K / kslice),
// which must be 1 unless epilogue is 1.
extern "C" int ttie_skinny_gemm_tuned(const void* x, long long ldx, const void* w, long long ldw, const void* bias, void* out,
                                      long long ldo, int M, int N, int K, int kslice, int epilogue, int up_offset, int unroll,
                                      void* stream);
extern "C" int ttie_skinny_gemm(const void* x, long long ldx, const void* w, long long ldw, const void* bias, void* out,
                                long long ldo, int M, int N, int K, int kslice, int epilogue, int up_offset, void* stream) {
    return ttie_skinny_gemm_tuned(x, ldx, w, ldw, bias, out, ldo, M, N, K, kslice, epilogue, up_offset, 0, stream);
}
// unroll: 0 = chosen from kslice; 2 or 4 = 32-key blocks per register buffer (rows <= 8 only); + 16 = two sets of 16
// weight rows per CTA (plain epilogues; halves the 32-key blocks per buffer).
extern "C" int ttie_skinny_gemm_tuned(const void* x, long long ldx, const void* w, long long ldw, const void* bias, void* out,
                                      long long ldo, int M, int N, int K, int kslice, int epilogue, int up_offset, int unroll,
                                      void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) TTIE_FAIL("skinny_gemm: %d rows; this kernel takes at most 64", M);
    if (K <= 0 || K % 8) TTIE_FAIL("skinny_gemm: K=%d must be a positive multiple of 8", K);
    if (ldx % 8 || ldw % 8) TTIE_FAIL("skinny_gemm: row strides must be multiples of 8 elements");
    if (((uintptr_t)x | (uintptr_t)w) & 15) TTIE_FAIL("skinny_gemm: pointers must be 16-byte aligned");
    if (kslice <= 0 || kslice % 128) TTIE_FAIL("skinny_gemm: kslice=%d must be a positive multiple of 128", kslice);
    const int splits = ceil_div(K, kslice);
    if (splits > 1 && epilogue != 1) TTIE_FAIL("skinny_gemm: K can be split over CTAs only with the partial-sum epilogue");
    if (splits > 65535) TTIE_FAIL("skinny_gemm: too many splits");
    SkinnyParams p;
    p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.w = (const __nv_bfloat16*)w; p.ldw = ldw;
    p.bias = (const __nv_bfloat16*)bias; p.out = out; p.ldo = ldo; p.M = M; p.N = N; p.K = K;
    p.kslice = kslice; p.up_offset = up_offset;
    cudaStream_t s = (cudaStream_t)stream;
    switch (epilogue) {
        case 0: return dispatch<0>(p, splits, unroll, s);
        case 1: return dispatch<1>(p, splits, unroll, s);
        case 2: return dispatch<2>(p, splits, unroll, s);
        case 3: return dispatch<3>(p, splits, unroll, s);
    }
    TTIE_FAIL("skinny_gemm: unknown epilogue %d", epilogue);
}
