// Sampling on the device: a row of logits is shared by up to 8 CTAs (a thread-block cluster), per-request state in a table.
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
#include <algorithm>
using namespace ttie;

namespace {
constexpr int THREADS = 1024;
constexpr int LIST_TOP_K = 256;                                      // largest top-k for which the short list is tried
constexpr int KEEP_CAP = 1024;                                       // tokens one CTA may hand in to the short list
constexpr float LIST_TOP_P = 1024.f;                                 // top-p alone: the list takes tokens of 1 / 1024 of the row's mass or more
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

// ---- histograms in shared memory.  The keys of a row crowd into a few bins of the leading digit, so one atomic per
// element would serialise; a warp first adds up the contributions of its lanes that fall into the same bin and one
// lane per bin adds the sum.  All 32 lanes call these together; a lane without an element passes bin = -1.
__device__ __forceinline__ void hist_add_count(u64* hist, int bin) {
    if (!__ballot_sync(0xffffffffu, bin >= 0)) return;               // (after the leading digit few lanes still take part)
    const unsigned peers = __match_any_sync(0xffffffffu, bin);
    if (bin >= 0 && (int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (u64)__popc(peers));
}
__device__ __forceinline__ void hist_add_mass(u64* hist, int bin, u64 mass) {
    unsigned todo = __ballot_sync(0xffffffffu, bin >= 0);
    while (todo) {                                                    // one round per distinct bin among the lanes
        const int leader = __ffs(todo) - 1;
        const int b = __shfl_sync(0xffffffffu, bin, leader);
        const bool mine = bin == b;
        u64 v = mine ? mass : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((int)(threadIdx.x & 31) == leader) atomicAdd(&hist[b], v);
        todo &= ~__ballot_sync(0xffffffffu, mine);
    }
}

// Walks the 256 bins from the highest down with a running sum that starts at `base`, and returns the first bin at
// which the sum, this bin included, reaches `limit` (strict: exceeds it); bin 0 if none does.  *above = base + the bins
// above the one returned.  One warp calls it: a lane owns 8 bins, the lanes' sums are scanned by shuffles.
__device__ __forceinline__ int pick_digit(const u64* hist, u64 base, u64 limit, bool strict, u64* above) {
    const int lane = threadIdx.x & 31;
    u64 h[8], t = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { h[j] = hist[255 - 8 * lane - j]; t += h[j]; }
    u64 incl = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    u64 cum = base + incl - t, at = 0;
    int hit = -1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const u64 next = cum + h[j];
        if (hit < 0 && (strict ? next > limit : next >= limit)) { hit = 255 - 8 * lane - j; at = cum; }
        cum = next;
    }
    const unsigned found = __ballot_sync(0xffffffffu, hit >= 0);
    const u64 total = __shfl_sync(0xffffffffu, incl, 31);
    if (!found) { *above = base + total - hist[0]; return 0; }
    const int src = __ffs(found) - 1;
    *above = __shfl_sync(0xffffffffu, at, src);
    return __shfl_sync(0xffffffffu, hit, src);
}

// ---- exchange between the CTAs that share a row (a thread-block cluster of C CTAs; C = 1: one CTA, no cluster)
__device__ __forceinline__ unsigned cluster_ctarank() { unsigned r; asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ void put_remote(T* local, unsigned rank, T v) {     // *local of CTA `rank` of the cluster = v
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    if (sizeof(T) == 8) asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote), "l"(*reinterpret_cast<u64*>(&v)) : "memory");
    else asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(*reinterpret_cast<unsigned*>(&v)) : "memory");
}
// Every CTA of the cluster hands in `n` values (thread t < n hands in v); afterwards buf[k * n + t] holds CTA k's
// value t in every CTA.  The caller alternates between two buffers from one exchange to the next: a CTA can be at
// most one exchange ahead of another, so a buffer is not written again while a slower CTA still reads it.
template <int C, typename T>
__device__ __forceinline__ void all_gather(T* buf, int n, T v, unsigned rank) {
    if (C == 1) {
        if ((int)threadIdx.x < n) buf[threadIdx.x] = v;
        __syncthreads();
    } else {
        if ((int)threadIdx.x < n) {
#pragma unroll
            for (int k = 0; k < C; ++k) put_remote(buf + (int)rank * n + threadIdx.x, (unsigned)k, v);
        }
        cluster_sync_all();
    }
}

// One row of logits is shared by C CTAs: CTA `rank` owns tokens [v0, v1) and keeps them (divided by the temperature)
// in its shared memory after the first pass, so the later passes do not go back to global memory; a slice too long
// for that (staged == 0) is read from global memory every time.  Maxima, histograms and sums of the slices are
// exchanged through distributed shared memory; every CTA then takes the same decisions from the same integers.
//
// With a top-k of a few hundred at most the row is left after two walks.  Every thread knows the largest value among its
// own tokens from the first walk; the k-th largest of a CTA's 1,024 such values is a bound that at least k tokens of the
// slice reach, so nothing below it can be among the row's k largest.  The tokens at or above the bound (a few more than k
// per CTA) are gathered in token order, handed to the first CTA of the cluster, and that CTA alone does the exact top-k
// cut, top-p and the draw on the list (`list_cap` entries fit the shared memory that held its slice).  If the list would
// overflow (thousands of equal values at the bound), every CTA goes on with its whole slice instead.
// Top-p without a top-k leaves the row the same way when the distribution is peaked: the (at most 1,024) tokens that hold
// 1 / 1,024 of the row's mass or more each are listed, and if together they hold more than top_p of the mass the cut lies
// among them.  A flat row (the listed tokens hold too little) is walked whole as before.
template <int C>
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int V, int slice, const int* __restrict__ slot_ids, int* __restrict__ state,
              int* __restrict__ out, float* __restrict__ probs_out, int staged, int list_cap) {
    extern __shared__ __align__(16) float s_row[];
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ u64 s_u64[32];
    __shared__ u64 s_hist[256];
    __shared__ u64 x_hist[2][C * 256];                               // exchange buffers, by exchange parity
    __shared__ u64 x_u64[2][C];
    __shared__ float x_val[C];
    __shared__ int x_idx[C];
    __shared__ int x_cnt[C];
    __shared__ float c_y[KEEP_CAP];                                   // this slice's tokens for the short list: value ...
    __shared__ int c_i[KEEP_CAP];                                     // ... and place in the slice
    __shared__ int s_scan[THREADS / 32];
    __shared__ unsigned s_prefix;
    __shared__ u64 s_acc;
    __shared__ int s_found;
    __shared__ u64 s_warp[THREADS / 32];

    TTIE_PDL_ENTRY();
    const unsigned rank = C == 1 ? 0u : cluster_ctarank();
    const int r = blockIdx.x / C, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v0 = min(V, (int)rank * slice), n = min(V, v0 + slice) - v0;     // this CTA's tokens: v0 .. v0 + n - 1
    const float* row = logits + (size_t)r * V + v0;
    const int slot = slot_ids[r];
    if (slot < 0) {                                                   // a padding row of a fixed-size batch: no request, no draw
        if (tid == 0 && rank == 0) out[r] = 0;
        return;                                                       // (the same for every CTA of the cluster)
    }
    // "I have started": nobody writes into a peer's shared memory before that peer is known to run (the wait stands
    // before the first exchange, with the first pass over the slice in between)
    if (C > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    int* st = state + (size_t)slot * 8;
    const unsigned seed_lo = (unsigned)st[0], seed_hi = (unsigned)st[1], draws = (unsigned)st[2];
    const int top_k = st[3];
    const float temperature = __int_as_float(st[4]), top_p = __int_as_float(st[5]);
    const int greedy = st[6];
    int xq = 0;                                                       // exchanges so far (their parity picks the buffer)

    // 1. maximum and the lowest index that holds it (and the slice into shared memory)
    float best = -INFINITY; int best_i = 0x7fffffff;
    if (staged && (n & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        for (int i = tid * 4; i < n; i += THREADS * 4) {
            const float4 x = *reinterpret_cast<const float4*>(row + i);
            *reinterpret_cast<float4*>(s_row + i) = x;
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (xs[k] > best || (xs[k] == best && i + k < best_i)) { best = xs[k]; best_i = i + k; }
        }
    } else {
        for (int i = tid; i < n; i += THREADS) {
            const float x = row[i];
            if (staged) s_row[i] = x;
            if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
        }
    }
    const float my_best = best;                                       // the largest among this thread's tokens (-inf: it has none)
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
        if (lane == 0) { s_val[0] = best; s_idx[0] = best_i == 0x7fffffff ? 0x7fffffff : best_i + v0; }
    }
    __syncthreads();
    if (C > 1) {                                                      // the slices' maxima, in rank order: lower tokens win ties
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        all_gather<C, float>(x_val, 1, s_val[0], rank);
        all_gather<C, int>(x_idx, 1, s_idx[0], rank);
        best = -INFINITY; best_i = 0x7fffffff;
#pragma unroll
        for (int k = 0; k < C; ++k)
            if (x_val[k] > best || (x_val[k] == best && x_idx[k] < best_i)) { best = x_val[k]; best_i = x_idx[k]; }
    } else {
        best = s_val[0]; best_i = s_idx[0];
    }
    if (best_i == 0x7fffffff) best_i = 0;                            // a row of NaNs: report token 0
    if (greedy) {
        if (tid == 0 && rank == 0) { out[r] = best_i; st[2] = (int)(draws + 1); }
        if (probs_out) for (int i = tid; i < n; i += THREADS) probs_out[(size_t)r * V + v0 + i] = (v0 + i == best_i) ? 1.f : 0.f;
        return;
    }
    const float ymax = best / temperature;
    if (staged) {
        for (int i = tid; i < n; i += THREADS) s_row[i] = s_row[i] / temperature;
        __syncthreads();
    }
    bool listed = false;                                              // the short list has replaced the row ...
    bool solo = C == 1;                                               // ... and this CTA goes on alone
    int n_cur = n;                                                    // tokens to walk: the slice, or the list
    float* u_y = s_row;                                               // the list (it takes the slice's place): values ...
    int* u_tok = reinterpret_cast<int*>(s_row + list_cap);            // ... and token ids, in token order
    auto Y0 = [&](int i) -> float { return staged ? s_row[i] : row[i] / temperature; };
    auto Y = [&](int i) -> float { return listed ? u_y[i] : Y0(i); };
    auto TOK = [&](int i) -> int { return listed ? u_tok[i] : v0 + i; };
    // the cluster's sum of a histogram of 256 bins that every CTA has filled in s_hist for its slice: into s_hist
    auto sum_hist = [&]() {
        if (C > 1 && !solo) {
            u64* buf = x_hist[xq & 1]; ++xq;
            all_gather<C, u64>(buf, 256, tid < 256 ? s_hist[tid] : 0, rank);
            if (tid < 256) {
                u64 t = 0;
#pragma unroll
                for (int k = 0; k < C; ++k) t += buf[k * 256 + tid];
                s_hist[tid] = t;
            }
        }
        __syncthreads();
    };
    u64 xs_parity = 0;                                                // exchanges of single values so far
    auto sum_u64 = [&](u64 v, u64* parts) -> u64 {                    // the cluster's sum of a per-CTA value; parts[k]: CTA k's
        if (solo) { if (parts) parts[0] = v; return v; }
        u64* buf = x_u64[xs_parity & 1]; ++xs_parity;
        all_gather<C, u64>(buf, 1, v, rank);
        u64 t = 0;
#pragma unroll
        for (int k = 0; k < C; ++k) { if (parts) parts[k] = buf[k]; t += buf[k]; }
        return t;
    };

    bool try_list = false, by_mass = false;
    unsigned low_key = 0;                                             // the list takes every token at or above this key
    u64 z_row = 0, limit_row = 0;                                     // top-p alone: the row's whole mass and top_p of it
    bool have_z = false;
    if (staged && list_cap > 0 && top_k > 0 && top_k < V && top_k <= LIST_TOP_K) {
        // (a) the bound: the top_k-th largest of the threads' own maxima (a radix select over one key per thread)
        const unsigned tkey = ordered_key(my_best / temperature);
        unsigned prefix = 0; u64 remaining = (u64)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += THREADS) s_hist[b] = 0;
            __syncthreads();
            hist_add_count(s_hist, (shift == 24 || (tkey >> (shift + 8)) == prefix) ? (int)((tkey >> shift) & 255u) : -1);
            __syncthreads();
            if (warp == 0) {
                u64 above;
                const int digit = pick_digit(s_hist, 0, remaining, false, &above);
                if (lane == 0) { s_prefix = (prefix << 8) | (unsigned)digit; s_acc = remaining - above; }
            }
            __syncthreads();
            prefix = s_prefix; remaining = s_acc;
            __syncthreads();
        }
        low_key = prefix; try_list = true;
    } else if (staged && list_cap > 0 && top_p < 1.0f && !(top_k > 0 && top_k < V)) {
        // (a') top-p without a top-k: at most LIST_TOP_P tokens hold 1 / LIST_TOP_P of the row's mass or more each.  If
        // together they hold more than top_p of it, the cut lies among them and the rest of the row is not needed.
        u64 zz = 0;
        for (int i = tid; i < n; i += THREADS) zz += mass_of(s_row[i], ymax);
        zz = block_sum_u64(zz, s_u64);
        z_row = sum_u64(zz, nullptr); have_z = true;
        limit_row = (u64)((double)top_p * (double)z_row);
        low_key = ordered_key(ymax + logf((float)((double)z_row * (1.0 / 1099511627776.0) / LIST_TOP_P)));
        try_list = true; by_mass = true;
    }
    if (try_list) {
        // (b) the tokens at or above the bound, in token order: a thread counts them in its run of consecutive tokens (an
        // odd run length: different banks), a scan over the block gives each run its place
        const int run = ((n + THREADS - 1) / THREADS) | 1;
        const int a = min(n, tid * run), b = min(n, a + run);
        int cnt = 0;
        u64 lm = 0;                                                   // (top-p alone) their mass
        for (int i = a; i < b; ++i) {
            const float y = s_row[i];
            if (ordered_key(y) >= low_key) { ++cnt; if (by_mass) lm += mass_of(y, ymax); }
        }
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) s_scan[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = s_scan[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += up;
            }
            s_scan[lane] = w;
        }
        __syncthreads();
        int at = incl - cnt + (warp ? s_scan[warp - 1] : 0);
        const int kept = s_scan[THREADS / 32 - 1];
        if (kept <= KEEP_CAP) {
            for (int i = a; i < b; ++i) {
                const float y = s_row[i];
                if (ordered_key(y) >= low_key) { c_y[at] = y; c_i[at] = i; ++at; }
            }
        }
        // (c) how many each CTA brings (this exchange also tells that every CTA is done reading its slice)
        int before = 0, total = 0;
        bool fits = true;
        if (C > 1) {
            all_gather<C, int>(x_cnt, 1, kept, rank);
#pragma unroll
            for (int k = 0; k < C; ++k) {
                fits = fits && x_cnt[k] <= KEEP_CAP;
                if (k < (int)rank) before += x_cnt[k];
                total += x_cnt[k];
            }
        } else {
            __syncthreads();
            fits = kept <= KEEP_CAP; total = kept;
        }
        fits = fits && total <= list_cap;
        if (by_mass) {                                                // the list must reach past the cut
            lm = block_sum_u64(lm, s_u64);
            fits = sum_u64(lm, nullptr) > limit_row && fits;
        }
        if (fits) {
            // (d) into the first CTA's list, slice after slice; the others are done
            for (int j = tid; j < kept; j += THREADS) {
                if (C > 1) { put_remote(u_y + before + j, 0u, c_y[j]); put_remote(u_tok + before + j, 0u, v0 + c_i[j]); }
                else { u_y[j] = c_y[j]; u_tok[j] = v0 + c_i[j]; }
            }
            if (C > 1) {
                cluster_sync_all();
                if (rank != 0) return;
            } else {
                __syncthreads();
            }
            listed = true; solo = true; n_cur = total;
        }
    }

    // The passes below visit every token of the slice several times.  A slice of up to 8 tokens per thread is kept in
    // registers as (key, probability mass) - the mass is computed once, not once per pass - ; a longer one is read from
    // shared (or global) memory and its masses recomputed on each visit.
    constexpr int EPT = 8;
    const int iters = (n_cur + THREADS - 1) / THREADS;             // visits per thread (the same for all: whole warps go round together)
    const bool cached = iters <= EPT && (top_k > 0 || top_p < 1.0f);
    unsigned ck[EPT];
    u64 cm[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        ck[e] = 0; cm[e] = 0;
        const int i = e * THREADS + tid;
        if (cached && i < n_cur) { const float y = Y(i); ck[e] = ordered_key(y); cm[e] = mass_of(y, ymax); }
    }
    auto for_all = [&](bool need_mass, auto&& body) {               // body(token present, key, mass)
        if (cached) {
#pragma unroll
            for (int e = 0; e < EPT; ++e)
                if (e < iters) body(e * THREADS + tid < n_cur, ck[e], cm[e]);
        } else {
            for (int i0 = 0; i0 < n_cur; i0 += THREADS) {
                const int i = i0 + tid;
                unsigned key = 0; u64 mass = 0;
                if (i < n_cur) { const float y = Y(i); key = ordered_key(y); if (need_mass) mass = mass_of(y, ymax); }
                body(i < n_cur, key, mass);
            }
        }
    };

    // 2. top-k threshold: the k-th largest key, by radix select over 4 digits of 8 bits
    unsigned cut_key = 0;
    if (top_k > 0 && top_k < V) {
        unsigned prefix = 0; u64 remaining = (u64)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += THREADS) s_hist[b] = 0;
            __syncthreads();
            for_all(false, [&](bool there, unsigned key, u64) {
                const int bin = there && (shift == 24 || (key >> (shift + 8)) == prefix) ? (int)((key >> shift) & 255u) : -1;
                hist_add_count(s_hist, bin);
            });
            __syncthreads();
            sum_hist();
            if (warp == 0) {
                u64 above;
                const int digit = pick_digit(s_hist, 0, remaining, false, &above);
                if (lane == 0) { s_prefix = (prefix << 8) | (unsigned)digit; s_acc = remaining - above; }
            }
            __syncthreads();
            prefix = s_prefix; remaining = s_acc;
            __syncthreads();
        }
        cut_key = prefix;
    }

    // 3. top-p threshold: the smallest key whose strictly-larger keys hold mass <= top_p * total
    if (top_p < 1.0f) {
        u64 z = z_row;                                                // (known already if the short list was tried for top-p alone)
        if (!have_z) {
            for_all(true, [&](bool there, unsigned key, u64 mass) { if (there && key >= cut_key) z += mass; });
            z = block_sum_u64(z, s_u64);
            if (C > 1 && !solo) z = sum_u64(z, nullptr);
        }
        const u64 limit = (u64)((double)top_p * (double)z);
        unsigned prefix = 0; u64 acc = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += THREADS) s_hist[b] = 0;
            __syncthreads();
            for_all(true, [&](bool there, unsigned key, u64 mass) {
                const bool in = there && key >= cut_key && (shift == 24 || (key >> (shift + 8)) == prefix);
                hist_add_mass(s_hist, in ? (int)((key >> shift) & 255u) : -1, in ? mass : 0);
            });
            __syncthreads();
            sum_hist();
            if (warp == 0) {                                                   // the cut lies inside the digit picked
                u64 a;                                                         // (digit 0 if nothing is cut)
                const int digit = pick_digit(s_hist, acc, limit, true, &a);
                if (lane == 0) { s_prefix = (prefix << 8) | (unsigned)digit; s_acc = a; }
            }
            __syncthreads();
            prefix = s_prefix; acc = s_acc;
            __syncthreads();
        }
        if (prefix > cut_key) cut_key = prefix;
    }

    // 4. draw: inverse CDF in index order over the kept tokens.  A thread owns a run of consecutive tokens of the
    // slice (an odd number of them, so the threads of a warp read different banks of the staged row); a slice that
    // is not staged is walked by warps instead, 32 consecutive tokens at a time, so its loads coalesce.
    const bool by_thread = staged != 0;
    const int chunk = by_thread ? (((n_cur + THREADS - 1) / THREADS) | 1) : ((((n_cur + THREADS / 32 - 1) / (THREADS / 32)) + 31) & ~31);
    const int i0 = min(n_cur, (by_thread ? tid : warp) * chunk), i1 = min(n_cur, i0 + chunk);
    u64 local = 0;
    if (by_thread) {
        for (int i = i0; i < i1; ++i) {
            const float y = Y(i);
            if (ordered_key(y) >= cut_key) local += mass_of(y, ymax);
        }
    } else {
        for (int i = i0 + lane; i < i1; i += 32) {
            const float y = Y(i);
            if (ordered_key(y) >= cut_key) local += mass_of(y, ymax);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);     // the warp's run: every lane holds its sum
    }
    // inclusive scan of the runs' sums: inside each warp by shuffles, then over the warps' totals (integers: exact)
    u64 incl = local;
    if (by_thread) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
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
    const u64 mine = s_warp[THREADS / 32 - 1];                        // kept mass of this CTA's slice
    u64 parts[C];
    const u64 total = (C > 1 && !solo) ? sum_u64(mine, parts) : mine;
    u64 below = 0;                                                    // kept mass of the slices before this one
#pragma unroll
    for (int k = 0; k < C; ++k) if (C > 1 && !solo && k < (int)rank) below += parts[k];
    unsigned rnd[4];
    philox4x32_10(draws, 0u, 0u, 0u, seed_lo, seed_hi, rnd);
    const double u = (double)(rnd[0] >> 8) * (1.0 / 16777216.0);
    u64 target = (u64)(u * (double)total);
    if (target >= total) target = total ? total - 1 : 0;             // total == 0 cannot happen (the maximum has mass 2^40)
    const bool here = target >= below && target < below + mine;       // exactly one CTA holds the target
    if (tid == 0) s_found = -1;
    __syncthreads();
    const u64 before = below + incl - local;
    if (here && local > 0 && target >= before && target < before + local) {
        if (by_thread) {
            u64 c = before;
            for (int i = i0; i < i1; ++i) {
                const float y = Y(i);
                if (ordered_key(y) >= cut_key) {
                    c += mass_of(y, ymax);
                    if (target < c) { s_found = TOK(i); break; }
                }
            }
        } else {
            // the warp walks its run again, 32 tokens at a time, with a scan over the lanes
            u64 c = before;
            for (int i = i0; i < i1; i += 32) {
                const int j = i + lane;
                u64 m = 0;
                if (j < i1) { const float y = Y(j); if (ordered_key(y) >= cut_key) m = mass_of(y, ymax); }
                u64 sc = m;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const u64 up = __shfl_up_sync(0xffffffffu, sc, o);
                    if (lane >= o) sc += up;
                }
                const bool hit = m > 0 && target >= c + sc - m && target < c + sc;
                const unsigned where = __ballot_sync(0xffffffffu, hit);
                if (where) { if (hit) s_found = TOK(j); break; }
                c += __shfl_sync(0xffffffffu, sc, 31);
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (here) out[r] = s_found >= 0 ? s_found : best_i;
        if (rank == 0) st[2] = (int)(draws + 1);
    }
    if (probs_out) {
        const double inv = total ? 1.0 / (double)total : 0.0;
        if (listed) {                                                 // this CTA is the only one left: the whole row is its to write
            for (int i = tid; i < V; i += THREADS) probs_out[(size_t)r * V + i] = 0.f;
            __syncthreads();
            for (int i = tid; i < n_cur; i += THREADS) {
                const float y = Y(i);
                if (ordered_key(y) >= cut_key) probs_out[(size_t)r * V + TOK(i)] = (float)((double)mass_of(y, ymax) * inv);
            }
        } else {
            for (int i = tid; i < n; i += THREADS) {
                const float y = Y0(i);
                probs_out[(size_t)r * V + v0 + i] = ordered_key(y) >= cut_key ? (float)((double)mass_of(y, ymax) * inv) : 0.f;
            }
        }
    }
}

constexpr int STAGE_FLOATS = 40 * 1024;                              // 160 KB of a slice in shared memory, beside the exchange buffers

template <int C>
int launch(const float* logits, int R, int V, const int* slot_ids, int* state, int* out, float* probs_out, cudaStream_t s) {
    int slice = (V + C - 1) / C;
    slice = (slice + 3) & ~3;                                         // slices start on 16-byte boundaries of a row that does
    const int staged = slice <= STAGE_FLOATS;
    // the staged slice, and room for the short list that may take its place (8 bytes an entry)
    const size_t smem = staged ? std::max((size_t)slice * sizeof(float), (size_t)32768) : 0;
    const int list_cap = (int)(smem / 8);
    auto k = sample_kernel<C>;
    static bool allowed = false;
    if (!allowed) {
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGE_FLOATS * 4) != cudaSuccess)
            TTIE_FAIL("sample: %d bytes of shared memory refused", STAGE_FLOATS * 4);
        allowed = true;
    }
    if (C == 1) TTIE_LAUNCH(k, R, THREADS, smem, s, logits, V, slice, slot_ids, state, out, probs_out, staged, list_cap);
    else TTIE_LAUNCH_CLUSTER(k, R * C, THREADS, smem, s, dim3(C, 1, 1), logits, V, slice, slot_ids, state, out, probs_out, staged, list_cap);
    TTIE_CHECK_LAUNCH("sample");
    return 0;
}
}  // namespace

// ctas_per_row: 0 = chosen from the vocabulary and the rows (measured: more CTAs per row are faster as long as all rows'
// clusters fit the GPU at once - 8 at batch 8, 2 at batch 64 - and a slice should fit the shared-memory staging), else
// 1, 2, 4 or 8.
extern "C" int ttie_sample_tuned(const float* logits, int R, int V, const int* slot_ids, int* state, int* out,
                                 float* probs_out, int ctas_per_row, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0) TTIE_FAIL("sample: empty vocabulary");
    int C = ctas_per_row;
    if (C == 0) {
        int need = 1;                                                 // fewest CTAs whose slices can be staged
        while (need < 8 && (V + need - 1) / need > STAGE_FLOATS) need *= 2;
        int fit = 8;                                                  // most CTAs per row with every cluster resident at once
        while (fit > 1 && (long long)R * fit > num_sms()) fit /= 2;
        C = fit > need ? fit : need;
        while (C > 1 && (V + C - 1) / C < 1024) C /= 2;               // (a tiny vocabulary needs no cluster)
    }
    cudaStream_t s = (cudaStream_t)stream;
    switch (C) {
        case 1: return launch<1>(logits, R, V, slot_ids, state, out, probs_out, s);
        case 2: return launch<2>(logits, R, V, slot_ids, state, out, probs_out, s);
        case 4: return launch<4>(logits, R, V, slot_ids, state, out, probs_out, s);
        case 8: return launch<8>(logits, R, V, slot_ids, state, out, probs_out, s);
    }
    TTIE_FAIL("sample: %d CTAs per row (1, 2, 4 or 8)", C);
}

extern "C" int ttie_sample(const float* logits, int R, int V, const int* slot_ids, int* state, int* out,
                           float* probs_out, void* stream) {
    return ttie_sample_tuned(logits, R, V, slot_ids, state, out, probs_out, 0, stream);
}
