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

namespace ttie {
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_error, sizeof(g_error), fmt, ap); va_end(ap);
}
}  // namespace ttie
using namespace ttie;

extern "C" const char* ttie_last_error() { return ttie::g_error; }
extern "C" int ttie_abi_version() { return 3; }

// ------------------------------------------------------------------------------------------ embed
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                             int d, int vocab) {
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
    if (dtype == kF32) embed_kernel<float><<<T, threads, 0, s>>>(ids, (const float*)table, out, d, vocab);
    else if (dtype == kBF16) embed_kernel<__nv_bfloat16><<<T, threads, 0, s>>>(ids, (const __nv_bfloat16*)table, out, d, vocab);
    else TTIE_FAIL("embed: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("embed");
    return 0;
}

// ------------------------------------------------------------------------------------------ rmsnorm
// One block per row.  resid (float32) += delta; out = rmsnorm(resid) * w.  `rows` (optional)
// gathers rows and then leaves resid untouched.
template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const int* __restrict__ rows,
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
        row[i] = v;
        if (!rows && dl) x[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        o[i] = from_f32<T>(row[i] * inv * to_f32<W>(weight[i]));
}

template <typename T>
static int launch_rmsnorm(float* resid, const void* delta, const int* rows, const void* weight, int w_dtype, void* out,
                          int R, int d, float eps, cudaStream_t s) {
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) TTIE_FAIL("rmsnorm: width %d needs %zu bytes of shared memory (limit 204800)", d, smem);
    if (w_dtype == kF32) {
        auto k = add_rmsnorm_kernel<T, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<R, threads, smem, s>>>(resid, (const T*)delta, rows, (const float*)weight, (T*)out, d, eps);
    } else if (w_dtype == kBF16) {
        auto k = add_rmsnorm_kernel<T, __nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<R, threads, smem, s>>>(resid, (const T*)delta, rows, (const __nv_bfloat16*)weight, (T*)out, d, eps);
    } else TTIE_FAIL("rmsnorm: unknown weight dtype %d", w_dtype);
    TTIE_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// rows == nullptr: all R rows in place (resid updated).  rows != nullptr: gather R rows.
extern "C" int ttie_add_rmsnorm(float* resid, const void* delta, const int* rows, const void* weight, int w_dtype,
                                void* out, int R, int d, float eps, int dtype, void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kF32) return launch_rmsnorm<float>(resid, delta, rows, weight, w_dtype, out, R, d, eps, s);
    if (dtype == kBF16) return launch_rmsnorm<__nv_bfloat16>(resid, delta, rows, weight, w_dtype, out, R, d, eps, s);
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

extern "C" int ttie_swiglu(const void* gate_up, void* out, int T, int F, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * F;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
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
