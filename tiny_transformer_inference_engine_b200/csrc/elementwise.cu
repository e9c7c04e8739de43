// Memory-bound kernels of the step: embedding gather, residual add + RMSNorm, row gather +
// RMSNorm, SwiGLU activation, rotary position encoding fused with the key/value store.
//
// Formulas (reference files): RMSNorm models/rmsnorm.py:13-17 (x * rsqrt(mean(x^2) + eps) * w in
// 32-bit, eps inside the root); rotation models/rope.py:21-35 (interleaved pairs) or
// kernels/rope_kernel/rope_kernel.cu:133-157 (half-split pairs); page slot
// serving/kv_pool.py:40-55 (table[pos / page] * page + pos % page); SwiGLU
// kernels/fused_swiglu/kernel.py:20-25 (silu(g) * u in 32-bit).
#include "common.cuh"
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>

namespace ttie {
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_error, sizeof(g_error), fmt, ap); va_end(ap);
}
}  // namespace ttie
using namespace ttie;

namespace ttie {
static int g_pdl = -1;
bool pdl_enabled() {
    if (g_pdl < 0) { const char* e = getenv("TTIE_PDL"); g_pdl = (e && e[0] == '0') ? 0 : 1; }
    return g_pdl != 0;
}
}  // namespace ttie
extern "C" void ttie_set_pdl(int on) { ttie::g_pdl = on ? 1 : 0; }

namespace ttie {
int num_sms() {
    static int count[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!count[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        count[dev] = n;
    }
    return count[dev];
}
}  // namespace ttie
extern "C" int ttie_num_sms() { return ttie::num_sms(); }
extern "C" const char* ttie_last_error() { return ttie::g_error; }
extern "C" int ttie_abi_version() { return 4; }

// ------------------------------------------------------------------------------------------ embed
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                             int d, int vocab) {
    TTIE_PDL_ENTRY();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);          // ids are validated on the host; never read outside
    const T* row = table + (size_t)id * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

extern "C" int ttie_embed(const int* ids, const void* table, float* out, int T, int d, int vocab, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == kF32) TTIE_LAUNCH(embed_kernel<float>, T, threads, 0, s, ids, (const float*)table, out, d, vocab);
    else if (dtype == kBF16) TTIE_LAUNCH(embed_kernel<__nv_bfloat16>, T, threads, 0, s, ids, (const __nv_bfloat16*)table, out, d, vocab);
    else TTIE_FAIL("embed: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("embed");
    return 0;
}

// ------------------------------------------------------------------------------------------ rmsnorm
// One block per row.  resid (float32) += delta; out = rmsnorm(resid) * w.  `rows` (optional)
// gathers rows and then leaves resid untouched.
// `dpart` (optional, instead of delta): float32 partial sums [S][rows of resid][d] of a K-split matrix
// product; they are added in the order s = 0..S-1.
template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart,
                                   int S, long long part_stride, const int* __restrict__ rows,
                                   const W* __restrict__ weight, T* __restrict__ out, int d, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * d;
    float* x = resid + src;
    const T* dl = delta ? delta + src : nullptr;
    T* o = out + (size_t)r * d;
    extern __shared__ float row[];                                  // d floats: the summed row
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = x[i];
        if (dl) v += to_f32<T>(dl[i]);
        if (dpart) {
            float a = 0.f;
            for (int sp = 0; sp < S; ++sp) a += dpart[sp * part_stride + src + i];
            v += a;
        }
        row[i] = v;
        if (!rows && (dl || dpart)) x[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        o[i] = from_f32<T>(row[i] * inv * to_f32<W>(weight[i]));
}


// Vectorised form for widths that are a multiple of 4 and fit 8 float4 per thread: the row stays
// in registers between the sum of squares and the scaling, so memory is touched once.
template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u; u.x = *reinterpret_cast<unsigned*>(&a); u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename T, typename W, int NT, int MAXC>
__global__ void __launch_bounds__(NT)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart,
                       int S, long long part_stride, const int* __restrict__ rows,
                       const W* __restrict__ weight, T* __restrict__ out, int d, float eps) {
    __shared__ float scratch[32];
    TTIE_PDL_ENTRY();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * d;
    float4 v[MAXC];
    float ss = 0.f;
    const int nchunk = d >> 2;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int i = (threadIdx.x + c * NT) * 4;
        if (threadIdx.x + c * NT < nchunk) {
            float4 a = *reinterpret_cast<const float4*>(resid + src + i);
            if (delta) { const float4 b = Vec4<T>::load(delta + src + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            if (dpart) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < S; ++sp) {
                    const float4 b = *reinterpret_cast<const float4*>(dpart + sp * part_stride + src + i);
                    t.x += b.x; t.y += b.y; t.z += b.z; t.w += b.w;
                }
                a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
            }
            if (!rows && (delta || dpart)) *reinterpret_cast<float4*>(resid + src + i) = a;
            v[c] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int i = (threadIdx.x + c * NT) * 4;
        if (threadIdx.x + c * NT < nchunk) {
            const float4 w = Vec4<W>::load(weight + i);
            Vec4<T>::store(out + (size_t)r * d + i, make_float4(v[c].x * inv * w.x, v[c].y * inv * w.y, v[c].z * inv * w.z, v[c].w * inv * w.w));
        }
    }
}

// Few rows (a decode step): a row is shared by a cluster of C CTAs, so C times as many SMs pull the row
// and its partial sums, and each thread has all its loads in flight at once.  The CTAs exchange their
// shares of the sum of squares through distributed shared memory and add them in rank order, so every
// CTA of the cluster holds the same sum.  The norm weights do not depend on the kernel before this one
// and are loaded ahead of the wait for it.  Used up to 96 rows (64 rows of 4,096: 3.9 us against 4.4 for one CTA per row;
// at 128 rows the 512 CTAs lose, 6.8 us).
template <typename T, typename W, int NT, int MAXC, int C>
__global__ void __launch_bounds__(NT)
add_rmsnorm_cluster_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart,
                           int S, long long part_stride, const int* __restrict__ rows,
                           const W* __restrict__ weight, T* __restrict__ out, int d, float eps) {
    __shared__ float scratch[32];
    __shared__ float share;                                         // this CTA's part of the sum of squares
    const int r = blockIdx.x / C, rank = blockIdx.x - r * C;        // clusters are consecutive CTAs along x
    const int nchunk = d >> 2, per = (nchunk + C - 1) / C;
    const int c_begin = rank * per, c_end = min(nchunk, c_begin + per);
    float4 w[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int ch = c_begin + threadIdx.x + c * NT;
        if (ch < c_end) w[c] = Vec4<W>::load(weight + ch * 4);
    }
    TTIE_PDL_ENTRY();
    const size_t src = (size_t)(rows ? rows[r] : r) * d;
    float4 v[MAXC];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int ch = c_begin + threadIdx.x + c * NT;
        if (ch < c_end) {
            const int i = ch * 4;
            float4 a = *reinterpret_cast<const float4*>(resid + src + i);
            if (delta) { const float4 b = Vec4<T>::load(delta + src + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            if (dpart) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s0 = 0; s0 < S; s0 += 4) {                 // four loads in flight, added in the order s = 0..S-1
                    float4 b[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (s0 + k < S) b[k] = *reinterpret_cast<const float4*>(dpart + (s0 + k) * part_stride + src + i);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (s0 + k < S) { t.x += b[k].x; t.y += b[k].y; t.z += b[k].z; t.w += b[k].w; }
                }
                a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
            }
            if (!rows && (delta || dpart)) *reinterpret_cast<float4*>(resid + src + i) = a;
            v[c] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) share = ss;
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < C; ++k) {
        uint32_t remote;
        float part;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(&share)), "r"(k));
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part) : "r"(remote) : "memory");
        total += part;
    }
    const float inv = rsqrtf(total / (float)d + eps);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int ch = c_begin + threadIdx.x + c * NT;
        if (ch < c_end)
            Vec4<T>::store(out + (size_t)r * d + ch * 4, make_float4(v[c].x * inv * w[c].x, v[c].y * inv * w[c].y, v[c].z * inv * w[c].z, v[c].w * inv * w[c].w));
    }
    // no CTA may leave while another still reads its share
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
static int launch_rmsnorm(float* resid, const void* delta, const float* dpart, int S, long long part_stride,
                          const int* rows, const void* weight, int w_dtype, void* out,
                          int R, int d, float eps, cudaStream_t s) {
    const bool aligned = !(((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)dpart | (uintptr_t)weight | (uintptr_t)out) & 15)
                         && (part_stride % 4 == 0);
    if (d % 4 == 0 && d <= 8192 && d >= 1024 && aligned && R <= 96 && (w_dtype == kF32 || w_dtype == kBF16)) {
        constexpr int C = 4;                                        // (d / 4) chunks over 4 CTAs of 256 threads, 2 chunks each at most
        if (w_dtype == kF32) TTIE_LAUNCH_CLUSTER((add_rmsnorm_cluster_kernel<T, float, 256, 2, C>), R * C, 256, 0, s, C, resid, (const T*)delta, dpart, S, part_stride, rows, (const float*)weight, (T*)out, d, eps);
        else TTIE_LAUNCH_CLUSTER((add_rmsnorm_cluster_kernel<T, __nv_bfloat16, 256, 2, C>), R * C, 256, 0, s, C, resid, (const T*)delta, dpart, S, part_stride, rows, (const __nv_bfloat16*)weight, (T*)out, d, eps);
        TTIE_CHECK_LAUNCH("rmsnorm (cluster)");
        return 0;
    }
    if (d % 4 == 0 && d <= 8192 && aligned) {
        if (w_dtype == kF32) {
            if (d <= 2048) TTIE_LAUNCH((add_rmsnorm_vec_kernel<T, float, 128, 4>), R, 128, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows, (const float*)weight, (T*)out, d, eps);
            else TTIE_LAUNCH((add_rmsnorm_vec_kernel<T, float, 256, 8>), R, 256, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows, (const float*)weight, (T*)out, d, eps);
        } else if (w_dtype == kBF16) {
            if (d <= 2048) TTIE_LAUNCH((add_rmsnorm_vec_kernel<T, __nv_bfloat16, 128, 4>), R, 128, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows, (const __nv_bfloat16*)weight, (T*)out, d, eps);
            else TTIE_LAUNCH((add_rmsnorm_vec_kernel<T, __nv_bfloat16, 256, 8>), R, 256, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows, (const __nv_bfloat16*)weight, (T*)out, d, eps);
        } else TTIE_FAIL("rmsnorm: unknown weight dtype %d", w_dtype);
        TTIE_CHECK_LAUNCH("rmsnorm");
        return 0;
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) TTIE_FAIL("rmsnorm: width %d needs %zu bytes of shared memory (limit 204800)", d, smem);
    if (w_dtype == kF32) {
        auto k = add_rmsnorm_kernel<T, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<R, threads, smem, s>>>(resid, (const T*)delta, dpart, S, part_stride, rows, (const float*)weight, (T*)out, d, eps);
    } else if (w_dtype == kBF16) {
        auto k = add_rmsnorm_kernel<T, __nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<R, threads, smem, s>>>(resid, (const T*)delta, dpart, S, part_stride, rows, (const __nv_bfloat16*)weight, (T*)out, d, eps);
    } else TTIE_FAIL("rmsnorm: unknown weight dtype %d", w_dtype);
    TTIE_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// rows == nullptr: all R rows in place (resid updated).  rows != nullptr: gather R rows.
// delta: [rows of resid][d] in the compute dtype, or nullptr.  dpart: float32 partial sums
// [S][rows of resid][d] (part_stride = elements between two partial sums), or nullptr.
extern "C" int ttie_add_rmsnorm(float* resid, const void* delta, const float* dpart, int S, long long part_stride,
                                const int* rows, const void* weight, int w_dtype,
                                void* out, int R, int d, float eps, int dtype, void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kF32) return launch_rmsnorm<float>(resid, delta, dpart, S, part_stride, rows, weight, w_dtype, out, R, d, eps, s);
    if (dtype == kBF16) return launch_rmsnorm<__nv_bfloat16>(resid, delta, dpart, S, part_stride, rows, weight, w_dtype, out, R, d, eps, s);
    TTIE_FAIL("rmsnorm: unknown dtype %d", dtype);
}

// ------------------------------------------------------------------------------------------ swiglu
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F; const int f = (int)(i - t * F);
        const float g = to_f32<T>(gu[t * 2 * F + f]);
        const float u = to_f32<T>(gu[t * 2 * F + F + f]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// eight values per thread (bfloat16) when the width allows: 16-byte loads and stores
__global__ void swiglu_vec8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int F8, size_t total8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F8; const int f = (int)(i - t * F8);
        const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * F8 + f) * 8);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * F8 + F8 + f) * 8);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
            // the result is rounded to bfloat16 (2^-9): the fast exponential and division (about 2^-21) do not show
            o2[k] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + i * 8) = o4;
    }
}

extern "C" int ttie_swiglu(const void* gate_up, void* out, int T, int F, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * F;
    const int threads = 256;
    if (dtype == kBF16 && F % 8 == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15)) {
        const size_t total8 = total / 8;
        const int blocks = (int)((total8 + threads - 1) / threads < num_sms() * 16 ? (total8 + threads - 1) / threads : num_sms() * 16);
        swiglu_vec8_kernel<<<blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, F / 8, total8);
        TTIE_CHECK_LAUNCH("swiglu");
        return 0;
    }
    const int blocks = (int)((total + threads - 1) / threads < num_sms() * 16 ? (total + threads - 1) / threads : num_sms() * 16);
    if (dtype == kF32) swiglu_kernel<float><<<blocks, threads, 0, s>>>((const float*)gate_up, (float*)out, F, total);
    else if (dtype == kBF16) swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, F, total);
    else TTIE_FAIL("swiglu: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("swiglu");
    return 0;
}

// ------------------------------------------------------------------------------------------ rope + store
// One block per token.  qkv row: [Hq*D | Hkv*D | Hkv*D].  Rotates q and k in place (angles
// pos * inv_freq[j] in 32-bit, sine and cosine in 32-bit), then stores rotated k and raw v into
// the pages.  inv_freq == nullptr: no rotation.  write_kv == 0: store nothing.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, int row_stride, int Hq, int Hkv, int D,
                                  const int* __restrict__ positions, const int* __restrict__ token_seq,
                                  const float* __restrict__ inv_freq, int style,
                                  T* __restrict__ k_pages, T* __restrict__ v_pages,
                                  const int* __restrict__ block_table, int table_width, int page_size,
                                  int num_pages, int write_kv) {
    extern __shared__ float cs[];                                   // cos[D/2], sin[D/2]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = D >> 1;
    T* row = qkv + (size_t)t * row_stride;
    if (inv_freq) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float theta = (float)pos * inv_freq[j];
            float sn, c;
            sincosf(theta, &sn, &c);
            cs[j] = c; cs[half + j] = sn;
        }
        __syncthreads();
        const int n_rot = (Hq + Hkv) * half;
        for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
            const int h = i / half, j = i - h * half;
            T* x = row + h * D;
            const int a = style == 0 ? 2 * j : j, b = style == 0 ? 2 * j + 1 : j + half;
            const float xa = to_f32<T>(x[a]), xb = to_f32<T>(x[b]);
            const float c = cs[j], sn = cs[half + j];
            x[a] = from_f32<T>(xa * c - xb * sn);
            x[b] = from_f32<T>(xa * sn + xb * c);
        }
        __syncthreads();
    }
    if (write_kv && Hkv > 0) {
        const int seq = token_seq[t];
        int page = block_table[(size_t)seq * table_width + pos / page_size];
        if (page < 0 || page >= num_pages) page = 0;                 // validated on the host; never write outside
        const int off = pos % page_size;
        const T* k = row + Hq * D;
        const T* v = row + (Hq + Hkv) * D;
        for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
            const int h = i / D, dd = i - h * D;
            const size_t dst = (((size_t)page * Hkv + h) * page_size + off) * D + dd;
            k_pages[dst] = k[i];
            v_pages[dst] = v[i];
        }
    }
}

extern "C" int ttie_rope_store(void* qkv, int row_stride, int T, int Hq, int Hkv, int D, const int* positions,
                               const int* token_seq, const float* inv_freq, int style, void* k_pages, void* v_pages,
                               const int* block_table, int table_width, int page_size, int num_pages, int write_kv,
                               int dtype, void* stream) {
    if (T <= 0) return 0;
    if (D % 2) TTIE_FAIL("rope_store: head size %d must be even", D);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const size_t smem = (size_t)D * sizeof(float);
    if (dtype == kF32)
        rope_store_kernel<float><<<T, threads, smem, s>>>((float*)qkv, row_stride, Hq, Hkv, D, positions, token_seq, inv_freq,
            style, (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, num_pages, write_kv);
    else if (dtype == kBF16)
        rope_store_kernel<__nv_bfloat16><<<T, threads, smem, s>>>((__nv_bfloat16*)qkv, row_stride, Hq, Hkv, D, positions,
            token_seq, inv_freq, style, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_width,
            page_size, num_pages, write_kv);
    else TTIE_FAIL("rope_store: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("rope_store");
    return 0;
}

// ------------------------------------------------------------------------------------------ rope + store from partial sums
// The same as rope_store for a q/k/v row that arrives as float32 partial sums [S][T][width] of a
// K-split product: the row is summed (s = 0..S-1) into shared memory, rotated there in 32-bit, q is
// written to q_out [T][Hq*D] and k, v into the pages - the sum is rounded to the storage type once.
template <typename T>
__global__ void rope_store_partial_kernel(const float* __restrict__ part, int S, long long part_stride, int width,
                                          int Hq, int Hkv, int D, const int* __restrict__ positions,
                                          const int* __restrict__ token_seq, const float* __restrict__ inv_freq, int style,
                                          T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                          const int* __restrict__ block_table, int table_width, int page_size,
                                          int num_pages, int write_kv) {
    extern __shared__ float sm[];
    float* rowbuf = sm;                                             // [width]
    float* cs = sm + width;                                         // cos[D/2], sin[D/2]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = D >> 1;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float a = 0.f;
        for (int sp = 0; sp < S; ++sp) a += part[sp * part_stride + (long long)t * width + i];
        rowbuf[i] = a;
    }
    if (inv_freq)
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float sn, c;
            sincosf((float)pos * inv_freq[j], &sn, &c);
            cs[j] = c; cs[half + j] = sn;
        }
    __syncthreads();
    if (inv_freq) {
        const int n_rot = (Hq + Hkv) * half;
        for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
            const int h = i / half, j = i - h * half;
            float* x = rowbuf + h * D;
            const int a = style == 0 ? 2 * j : j, b = style == 0 ? 2 * j + 1 : j + half;
            const float xa = x[a], xb = x[b], c = cs[j], sn = cs[half + j];
            x[a] = xa * c - xb * sn;
            x[b] = xa * sn + xb * c;
        }
        __syncthreads();
    }
    T* qo = q_out + (size_t)t * Hq * D;
    for (int i = threadIdx.x; i < Hq * D; i += blockDim.x) qo[i] = from_f32<T>(rowbuf[i]);
    if (write_kv && Hkv > 0) {
        const int seq = token_seq[t];
        int page = block_table[(size_t)seq * table_width + pos / page_size];
        if (page < 0 || page >= num_pages) page = 0;
        const int off = pos % page_size;
        const float* k = rowbuf + Hq * D;
        const float* v = rowbuf + (Hq + Hkv) * D;
        for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
            const int h = i / D, dd = i - h * D;
            const size_t dst = (((size_t)page * Hkv + h) * page_size + off) * D + dd;
            k_pages[dst] = from_f32<T>(k[i]);
            v_pages[dst] = from_f32<T>(v[i]);
        }
    }
}

extern "C" int ttie_rope_store_partial(const float* part, int S, long long part_stride, int T, int Hq, int Hkv, int D,
                                       const int* positions, const int* token_seq, const float* inv_freq, int style,
                                       void* q_out, void* k_pages, void* v_pages, const int* block_table, int table_width,
                                       int page_size, int num_pages, int write_kv, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (D % 2) TTIE_FAIL("rope_store: head size %d must be even", D);
    cudaStream_t s = (cudaStream_t)stream;
    const int width = (Hq + 2 * Hkv) * D;
    const size_t smem = ((size_t)width + D) * sizeof(float);
    if (smem > 200 * 1024) TTIE_FAIL("rope_store_partial: row of %d values needs %zu bytes of shared memory", width, smem);
    const int threads = 256;
    if (dtype == kF32) {
        auto k = rope_store_partial_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<T, threads, smem, s>>>(part, S, part_stride, width, Hq, Hkv, D, positions, token_seq, inv_freq, style, (float*)q_out,
                                   (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, num_pages, write_kv);
    } else if (dtype == kBF16) {
        auto k = rope_store_partial_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<T, threads, smem, s>>>(part, S, part_stride, width, Hq, Hkv, D, positions, token_seq, inv_freq, style,
                                   (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
                                   table_width, page_size, num_pages, write_kv);
    } else TTIE_FAIL("rope_store_partial: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("rope_store_partial");
    return 0;
}

// ------------------------------------------------------------------------------------------ rope + store, vectorised
// Per step (not per layer): cos and sin of pos * inv_freq[j] for every token, [T][D/2] float2.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float2* __restrict__ cs,
                                  int half, int total) {
    TTIE_PDL_ENTRY();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int t = i / half, j = i - t * half;
    float sn, c;
    sincosf((float)positions[t] * inv_freq[j], &sn, &c);
    cs[i] = make_float2(c, sn);
}

extern "C" int ttie_rope_table(const int* positions, const float* inv_freq, void* cs, int T, int half, void* stream) {
    if (T <= 0) return 0;
    const int total = T * half;
    TTIE_LAUNCH(rope_table_kernel, ceil_div(total, 256), 256, 0, (cudaStream_t)stream, positions, inv_freq, (float2*)cs, half, total);
    TTIE_CHECK_LAUNCH("rope_table");
    return 0;
}

// Interleaved pairs, four values per thread (grid: tokens x pieces of 128 threads), no shared memory: the
// input row is either the packed q/k/v row in the compute dtype (then q and k are also written back in
// place) or float32 partial sums [S][T][width], of which a thread has up to four loads in flight.
// cos/sin come from the step's table.
template <typename T, bool PARTIAL>
__global__ void __launch_bounds__(256)
rope_store_vec_kernel(T* __restrict__ qkv, long long row_stride, const float* __restrict__ part, int S, long long part_stride,
                      int Hq, int Hkv, int D, const int* __restrict__ positions, const int* __restrict__ token_seq,
                      const float2* __restrict__ cs, T* __restrict__ q_out, long long q_stride,
                      T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                      int page_size, int num_pages, int write_kv) {
    TTIE_PDL_ENTRY();
    const int t = blockIdx.x;
    const int width = (Hq + 2 * Hkv) * D, half = D >> 1;
    // decode steps: one chunk per thread (grid y covers the row); prompt portions: one CTA walks the row
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < (width >> 2); c += gridDim.y * blockDim.x) {
    const int col = c << 2;
    const int h = col / D, i = col - h * D;
    float4 v;
    if (PARTIAL) {
        v = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = part + (long long)t * width + col;
        for (int s0 = 0; s0 < S; s0 += 4) {                         // added in the order s = 0..S-1
            float4 b[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (s0 + k < S) b[k] = *reinterpret_cast<const float4*>(src + (s0 + k) * part_stride);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (s0 + k < S) { v.x += b[k].x; v.y += b[k].y; v.z += b[k].z; v.w += b[k].w; }
        }
    } else {
        v = Vec4<T>::load(qkv + (long long)t * row_stride + col);
    }
    if (h < Hq + Hkv && cs) {
        const float4 t2 = *reinterpret_cast<const float4*>(cs + (size_t)t * half + (i >> 1));   // cos0 sin0 cos1 sin1
        v = make_float4(v.x * t2.x - v.y * t2.y, v.x * t2.y + v.y * t2.x, v.z * t2.z - v.w * t2.w, v.z * t2.w + v.w * t2.z);
    }
    if (h < Hq) {
        Vec4<T>::store(q_out + (long long)t * q_stride + col, v);
        continue;
    }
    if (!PARTIAL && h < Hq + Hkv) Vec4<T>::store(qkv + (long long)t * row_stride + col, v);
    if (write_kv) {
        const int pos = positions[t];
        int page = block_table[(size_t)token_seq[t] * table_width + pos / page_size];
        if (page < 0 || page >= num_pages) page = 0;
        const long long page_base = (long long)page * Hkv * page_size + pos % page_size;      // + h * page_size, all times D
        const int hk = h < Hq + Hkv ? h - Hq : h - Hq - Hkv;
        T* dst = (h < Hq + Hkv ? k_pages : v_pages) + (page_base + (long long)hk * page_size) * D + i;
        Vec4<T>::store(dst, v);
    }
    }
}

// qkv != nullptr: packed rows in the compute dtype, rotated in place (q_out may be qkv itself).
// part != nullptr: float32 partial sums; q goes to q_out [T][q_stride].  cs: table from ttie_rope_table or
// nullptr for no rotation.  Head size must be a multiple of 4.
extern "C" int ttie_rope_store_vec(void* qkv, long long row_stride, const float* part, int S, long long part_stride, int T,
                                   int Hq, int Hkv, int D, const int* positions, const int* token_seq, const void* cs,
                                   void* q_out, long long q_stride, void* k_pages, void* v_pages, const int* block_table,
                                   int table_width, int page_size, int num_pages, int write_kv, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (D % 4) TTIE_FAIL("rope_store_vec: head size %d must be a multiple of 4", D);
    if ((qkv == nullptr) == (part == nullptr)) TTIE_FAIL("rope_store_vec: give exactly one of qkv and part");
    if (((uintptr_t)qkv | (uintptr_t)part | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)cs) & 15)
        TTIE_FAIL("rope_store_vec: pointers must be 16-byte aligned");
    if (row_stride % 4 || q_stride % 4 || part_stride % 4) TTIE_FAIL("rope_store_vec: strides must be multiples of 4");
    cudaStream_t s = (cudaStream_t)stream;
    const bool few = T <= 64;                                       // a decode step: spread a row over CTAs of 128 threads
    const dim3 grid(T, few ? ceil_div((Hq + 2 * Hkv) * D / 4, 128) : 1);
    const int threads = few ? 128 : 256;
#define TTIE_ROPE_VEC(TT, P) TTIE_LAUNCH((rope_store_vec_kernel<TT, P>), grid, threads, 0, s, (TT*)qkv, row_stride, part, S, part_stride, Hq, Hkv, D, \
        positions, token_seq, (const float2*)cs, (TT*)q_out, q_stride, (TT*)k_pages, (TT*)v_pages, block_table, table_width, \
        page_size, num_pages, write_kv)
    if (dtype == kF32) { if (part) TTIE_ROPE_VEC(float, true); else TTIE_ROPE_VEC(float, false); }
    else if (dtype == kBF16) { if (part) TTIE_ROPE_VEC(__nv_bfloat16, true); else TTIE_ROPE_VEC(__nv_bfloat16, false); }
    else TTIE_FAIL("rope_store_vec: unknown dtype %d", dtype);
#undef TTIE_ROPE_VEC
    TTIE_CHECK_LAUNCH("rope_store_vec");
    return 0;
}
