// Sampling on the device: one block per row of logits, per-request state in a table.
//
// Order and meaning as the reference's sample() (sampling.py:110-135): logits / temperature,
// top-k as a threshold (everything >= the k-th largest value stays, sampling.py:85-92), top-p
// over the sorted probabilities (a token stays iff the probability mass of the values above it
// is <= top_p, so the token that crosses top_p stays and the first always stays,
// sampling.py:51-59; equal values stay or go together), softmax, one draw.  Greedy
// (sampling.py:5-6) is argmax with the lowest index among equal maxima.
//
// The draw uses Philox-4x32-10 keyed by the request's seed with the request's draw counter
// as the counter, and inverse-CDF selection in index order.  Probability mass is held in
// 64-bit fixed point (exp(y - max) * 2^40), so all sums are exact integer sums: the result
// does not depend on the order in which threads add, and it is the same on every run.
//
// State row (int32 x 8): seed_lo, seed_hi, draws, top_k, temperature bits, top_p bits, greedy, -.
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {
constexpr int THREADS = 1024;
typedef unsigned long long u64;

__device__ __forceinline__ unsigned ordered_key(float x) {
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ u64 mass_of(float y, float ymax) {
    return (u64)(expf(y - ymax) * 1099511627776.0f);                 // 2^40
}

__device__ void philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0, unsigned k1, unsigned* out) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const unsigned n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ u64 block_sum_u64(u64 v, u64* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    u64 t = threadIdx.x < (THREADS / 32) ? scratch[threadIdx.x] : 0;
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    const u64 r = scratch[0];
    __syncthreads();
    return r;
}

// staged: the row (divided by the temperature) lives in shared memory after the first pass, so the later passes
// do not go back to global memory; a row too long for that is read from global memory every time.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int V, const int* __restrict__ slot_ids, int* __restrict__ state,
              int* __restrict__ out, float* __restrict__ probs_out, int staged) {
    extern __shared__ __align__(16) float s_row[];
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ u64 s_u64[32];
    __shared__ u64 s_hist[256];
    __shared__ unsigned s_prefix;
    __shared__ u64 s_acc;
    __shared__ int s_found;
    __shared__ u64 s_warp[THREADS / 32];

    TTIE_PDL_ENTRY();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * V;
    if (slot_ids[r] < 0) {                                            // a padding row of a fixed-size batch: no request, no draw
        if (tid == 0) out[r] = 0;
        return;
    }
    int* st = state + (size_t)slot_ids[r] * 8;
    const unsigned seed_lo = (unsigned)st[0], seed_hi = (unsigned)st[1], draws = (unsigned)st[2];
    const int top_k = st[3];
    const float temperature = __int_as_float(st[4]), top_p = __int_as_float(st[5]);
    const int greedy = st[6];

    // 1. maximum and the lowest index that holds it (and the row into shared memory)
    float best = -INFINITY; int best_i = 0x7fffffff;
    if (staged && (V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        for (int i = tid * 4; i < V; i += THREADS * 4) {
            const float4 x = *reinterpret_cast<const float4*>(row + i);
            *reinterpret_cast<float4*>(s_row + i) = x;
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (xs[k] > best || (xs[k] == best && i + k < best_i)) { best = xs[k]; best_i = i + k; }
        }
    } else {
        for (int i = tid; i < V; i += THREADS) {
            const float x = row[i];
            if (staged) s_row[i] = x;
            if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane]; best_i = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
    }
    __syncthreads();
    best = s_val[0]; best_i = s_idx[0];
    if (best_i == 0x7fffffff) best_i = 0;                            // a row of NaNs: report token 0
    if (greedy) {
        if (tid == 0) { out[r] = best_i; st[2] = (int)(draws + 1); }
        if (probs_out) for (int i = tid; i < V; i += THREADS) probs_out[(size_t)r * V + i] = (i == best_i) ? 1.f : 0.f;
        return;
    }
    const float ymax = best / temperature;
    if (staged) {
        for (int i = tid; i < V; i += THREADS) s_row[i] = s_row[i] / temperature;
        __syncthreads();
    }
    auto Y = [&](int i) -> float { return staged ? s_row[i] : row[i] / temperature; };

    // 2. top-k threshold: the k-th largest key, by radix select over 4 digits of 8 bits
    unsigned cut_key = 0;
    if (top_k > 0 && top_k < V) {
        unsigned prefix = 0; u64 remaining = (u64)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += THREADS) s_hist[b] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += THREADS) {
                const unsigned key = ordered_key(Y(i));
                if (shift == 24 || (key >> (shift + 8)) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], (u64)1);
            }
            __syncthreads();
            if (tid == 0) {
                u64 cum = 0; int digit = 0;
                for (int b = 255; b >= 0; --b) {
                    if (cum + s_hist[b] >= remaining) { digit = b; break; }
                    cum += s_hist[b];
                }
                s_prefix = (prefix << 8) | (unsigned)digit;
                s_acc = remaining - cum;
            }
            __syncthreads();
            prefix = s_prefix; remaining = s_acc;
            __syncthreads();
        }
        cut_key = prefix;
    }

    // 3. top-p threshold: the smallest key whose strictly-larger keys hold mass <= top_p * total
    if (top_p < 1.0f) {
        u64 z = 0;
        for (int i = tid; i < V; i += THREADS) {
            const float y = Y(i);
            if (ordered_key(y) >= cut_key) z += mass_of(y, ymax);
        }
        z = block_sum_u64(z, s_u64);
        const u64 limit = (u64)((double)top_p * (double)z);
        unsigned prefix = 0; u64 acc = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += THREADS) s_hist[b] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += THREADS) {
                const float y = Y(i);
                const unsigned key = ordered_key(y);
                if (key >= cut_key && (shift == 24 || (key >> (shift + 8)) == prefix))
                    atomicAdd(&s_hist[(key >> shift) & 255u], mass_of(y, ymax));
            }
            __syncthreads();
            if (tid == 0) {
                int digit = 0; u64 a = acc;
                for (int b = 255; b >= 0; --b) {
                    if (a + s_hist[b] > limit || b == 0) { digit = b; break; }   // the cut lies inside this digit
                    a += s_hist[b];                                              // (digit 0 if nothing is cut)
                }
                s_prefix = (prefix << 8) | (unsigned)digit;
                s_acc = a;
            }
            __syncthreads();
            prefix = s_prefix; acc = s_acc;
            __syncthreads();
        }
        if (prefix > cut_key) cut_key = prefix;
    }

    // 4. draw: inverse CDF in index order over the kept tokens.  A thread owns a run of consecutive tokens (an odd
    // number of them, so the threads of a warp read different banks of the staged row).
    const int chunk = ((V + THREADS - 1) / THREADS) | 1;
    const int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
    u64 local = 0;
    for (int i = i0; i < i1; ++i) {
        const float y = Y(i);
        if (ordered_key(y) >= cut_key) local += mass_of(y, ymax);
    }
    // inclusive scan of the threads' sums: inside each warp by shuffles, then over the warps' totals (integers: exact)
    u64 incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        u64 w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        s_warp[lane] = w;
    }
    __syncthreads();
    incl += warp ? s_warp[warp - 1] : 0;
    const u64 total = s_warp[THREADS / 32 - 1];
    unsigned rnd[4];
    philox4x32_10(draws, 0u, 0u, 0u, seed_lo, seed_hi, rnd);
    const double u = (double)(rnd[0] >> 8) * (1.0 / 16777216.0);
    u64 target = (u64)(u * (double)total);
    if (target >= total) target = total ? total - 1 : 0;
    if (tid == 0) s_found = best_i;                                   // total == 0 cannot happen (the maximum has mass 2^40)
    __syncthreads();
    const u64 before = incl - local;
    if (local > 0 && target >= before && target < before + local) {
        u64 c = before;
        for (int i = i0; i < i1; ++i) {
            const float y = Y(i);
            if (ordered_key(y) >= cut_key) {
                c += mass_of(y, ymax);
                if (target < c) { s_found = i; break; }
            }
        }
    }
    __syncthreads();
    if (tid == 0) { out[r] = s_found; st[2] = (int)(draws + 1); }
    if (probs_out) {
        const double inv = total ? 1.0 / (double)total : 0.0;
        for (int i = tid; i < V; i += THREADS) {
            const float y = Y(i);
            probs_out[(size_t)r * V + i] = ordered_key(y) >= cut_key ? (float)((double)mass_of(y, ymax) * inv) : 0.f;
        }
    }
}
}  // namespace

extern "C" int ttie_sample(const float* logits, int R, int V, const int* slot_ids, int* state, int* out,
                           float* probs_out, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0) TTIE_FAIL("sample: empty vocabulary");
    // the row in shared memory when it fits beside the kernel's own (200 KB: 51,200 tokens)
    const size_t smem = (size_t)V * sizeof(float);
    const int staged = smem <= 200 * 1024;
    if (staged && smem > 40 * 1024 &&
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        TTIE_FAIL("sample: 200 KB of shared memory refused");
    TTIE_LAUNCH(sample_kernel, R, THREADS, staged ? smem : 0, (cudaStream_t)stream, logits, V, slot_ids, state, out, probs_out, staged);
    TTIE_CHECK_LAUNCH("sample");
    return 0;
}
