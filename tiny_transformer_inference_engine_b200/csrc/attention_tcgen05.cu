// Causal paged attention on tcgen05 tensor cores (bfloat16, head size 64, 128 or 256).  Two kernels:
//   attn_tc_kernel     one 128-row query tile per CTA: decode steps with the key range cut over CTAs (partial
//                      results for the merge kernel), and any step with few query rows per request
//   attn_tc_pp_kernel  two 128-row query tiles per CTA (one at head size 256, where tensor memory holds one output
//                      tile): prompt portions, and every step at head size 256 (described where it stands, below)
// Query rows are (token, head of a kv head's group) pairs, so with multi-query attention 4 tokens x 32 heads
// share every key/value tile of a 128-row tile.
//
// attn_tc_kernel: a CTA owns 128 query rows and walks over 128-key tiles:
//   warp 0      TMA: key and value tiles straight from the pages (one box per page and 64-column
//               block, 128-byte swizzle) into a two-stage ring
//   warp 1      one thread issues  S = Q K^T  (tcgen05.mma, both operands K-major in shared memory,
//               S in tensor memory, two buffers) and  O_tile = P V  (P from tensor memory, where it
//               replaced the tile's scores; V as an MN-major operand from shared memory; O_tile in
//               tensor memory, two buffers)
//   warps 2-17  softmax, four threads per row (each one quarter of the columns): tcgen05.ld the row of S,
//               scale, mask, running maximum and sum in float32, P rounded to bfloat16 and stored back into
//               tensor memory over the scores (tcgen05.st; no trip through shared memory, no proxy fence);
//               one iteration later the same threads take O_tile out of tensor memory and add it to their
//               part of the output row, rescaled - the running output lives in registers, so nothing in
//               tensor memory is ever rescaled.
// Mask, scale and table lookup are those of kernels/pagedattn/pagedattn.cu:196-207,256 of the reference.
// Every mbarrier wait is bounded; a wait that runs out records a code and the CTA winds down.
#include "common.cuh"
#include <cuda.h>
#include <math.h>
using namespace ttie;

namespace {
constexpr int BM = 128, BN = 128;
constexpr long long WAIT_CYCLES = 2000000000LL;

__device__ int g_attn_tc_error = 0;
__device__ int* g_attn_tc_error_mirror = nullptr;                // the same word in pinned host memory, if the host gave one

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// limit: clocks after which the wait gives up (about a second by default)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code, long long limit = WAIT_CYCLES) {
    if (mbar_try(bar, parity)) return true;
    const long long deadline = clock64() + limit;
    while (!mbar_try(bar, parity)) {
        if (clock64() > deadline) {
            atomicCAS(&g_attn_tc_error, 0, code);
            if (g_attn_tc_error_mirror) { *reinterpret_cast<volatile int*>(g_attn_tc_error_mirror) = code; __threadfence_system(); }
            return false;
        }
    }
    return true;
}
// The same for a warp that runs ahead of the others (the copy producer): it sleeps between polls, so its polling
// does not take issue slots from the softmax warps of its SM sub-partition.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long deadline = clock64() + WAIT_CYCLES;
    while (!mbar_try(bar, parity)) {
        __nanosleep(64);
        if (clock64() > deadline) {
            atomicCAS(&g_attn_tc_error, 0, code);
            if (g_attn_tc_error_mirror) { *reinterpret_cast<volatile int*>(g_attn_tc_error_mirror) = code; __threadfence_system(); }
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }

__device__ __forceinline__ float ex2(float x) {                // 2^x, one instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory operand descriptors in two words.  The upper word is the same for every operand here: 8-row groups
// 1024 bytes apart, descriptor version of sm_100, 128-byte swizzle.  The lower word holds the address (in units of 16
// bytes) and the leading offset.  K-major operand (queries, keys): rows of 64 bfloat16 = 128 bytes, leading offset
// unused (1).  MN-major operand (the value tile as B: the head dimension is contiguous, the keys are the 128-byte
// rows): leading offset = distance between 64-column blocks.  An operand's next K step is 32 bytes (K-major) or 16
// rows = 2048 bytes (MN-major) further on: one addition to the lower word.
// The products' A operand comes from shared memory (umma_ss_lean) or from tensor memory (umma_ts_lean: lane = row,
// 32-bit columns hold two consecutive bfloat16 of K).
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) { return ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16); }
template <bool ACC>
__device__ __forceinline__ void umma_ss_lean(uint32_t tmem_c, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
                 ::"r"(tmem_c), "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_ts_lean(uint32_t tmem_c, uint32_t tmem_a, uint32_t b_lo, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
                 ::"r"(tmem_c), "r"(tmem_a), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}

struct AttnTcParams {
    const __nv_bfloat16* q; long long q_stride;
    const int* block_table; int table_width; int page_size;
    const int* qsl; const int* seq_lens;
    __nv_bfloat16* out;
    int num_seqs, Hq, Hkv;
    float scale_log2; int window;
    int row_tiles;
    int q_rows;                                                  // rows of the query tile that are staged (a multiple of 32 that covers every request's rows)
    int num_splits, split_len;                                   // keys per CTA along grid y (a multiple of 128); 1: no split
    float* ws_o; float* ws_ml;                                   // partial results [row][split][D] and [row][split][2] (max in natural log, sum)
};

constexpr int NP = 4;                                            // softmax threads per query row
constexpr int NTHREADS = 64 + NP * 128;

// AHEAD: the copy producer looks pages up one tile ahead (prompt portions); otherwise as it goes (decode steps).
// NST: stages of the key ring and of the value ring.  A decode step's CTA is bound by how many bytes it has in flight
// (it walks its keys once, each tile's copy is asked for when its stage comes free), and it has few query rows: only
// `q_rows` of the tile's 128 rows are staged, which leaves room for a third stage at head size 128 and a fourth at 64.
// The product still reads 128 rows; what it finds past `q_rows` belongs to the next block or to the ring, gives score
// rows that nobody reads, and costs nothing (rows of a product do not mix).
template <int D, bool AHEAD, int NST>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
    // barrier slots: key / value stages full and empty, score and output buffers full and empty, P written, exchanges.
    // Every barrier that counts thread arrivals exists twice, by tile parity: the softmax threads write P of tile j + 1
    // (into the other score buffer) before they wait for the product of tile j, so they can arrive for two tiles in a
    // row while the issuing thread still waits for a late value tile - on a single barrier two completed phases look
    // like none, and that wait ran out (seen once in several thousand launches of 600 CTAs).
    constexpr int KF = 0, KE = NST, VF = 2 * NST, VE = 3 * NST, SF = 4 * NST, SE = SF + 2, OF = SE + 2, OE = OF + 2, PF = OE + 2,
                  XB = PF + 2, XL = XB + 2, NBARS = XL + 1;
    constexpr int CB = D / 64;                                   // 64-column blocks of the head dimension
    constexpr uint32_t KVBLK = BN * 128;                         // bytes of one 64-column block of a key / value tile
    constexpr uint32_t KV_BYTES = CB * KVBLK;
    const uint32_t QBLK = (uint32_t)p.q_rows * 128;              // ... of the staged query rows
    const uint32_t Q_BYTES = CB * QBLK;
    constexpr uint32_t TMEM_COLS = 512;                          // 2 x 128 (S) + 2 x D (O_tile), rounded to a power of two
    constexpr uint32_t S_COL = 0, O_COL = 256;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = smem;
    unsigned char* Ks = Qs + Q_BYTES;                            // [NST stages]
    unsigned char* Vs = Ks + NST * KV_BYTES;                     // [NST stages]
    __shared__ __align__(8) unsigned long long bars[NBARS];
    __shared__ uint32_t tmem_slot;
    __shared__ float xch[2][NP][BM];                              // row maxima of the column parts, by tile parity

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.Hq / p.Hkv;
    int tile = blockIdx.x;
    const int rt = p.row_tiles - 1 - tile % p.row_tiles;         // long (late) tiles first
    tile /= p.row_tiles;
    const int kvh = tile % p.Hkv, seq = tile / p.Hkv;
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G, row0 = rt * BM;
    if (row0 >= nrows) return;                                   // uniform over the CTA, before anything is allocated
    const int ctx = kv_len - q_len;
    const int tok_lo = row0 / G, tok_hi = (min(nrows, row0 + BM) - 1) / G;
    int key_hi = ctx + tok_hi + 1;                               // exclusive
    int key_lo = p.window > 0 ? max(0, ctx + tok_lo - p.window + 1) : 0;
    const int split = blockIdx.y;
    if (p.num_splits > 1) {                                      // splits start on tile boundaries
        const int piece = piece_len(kv_len, p.num_splits, p.split_len, BN);
        key_lo = max(key_lo, split * piece);
        key_hi = min(key_hi, (split + 1) * piece);
    }
    const int t_begin = key_lo / BN, t_end = (key_hi + BN - 1) / BN;
    const int ntiles = t_end - t_begin;
    const int rows_here = min(BM, nrows - row0);
    if (ntiles <= 0) {
        // (only with splits) no key of this split is visible: an empty partial result, nothing allocated.  The scratch
        // memory may still be read by the merge kernel of the launch before this one: wait for it first.
        pdl_wait();
        for (int e = threadIdx.x; e < rows_here * D; e += blockDim.x) {
            const int r = e / D, row = row0 + r;
            const int tok = row / G, g = row - tok * G;
            const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
            p.ws_o[(grow * p.num_splits + split) * D + (e - r * D)] = 0.f;
            if (e - r * D == 0) { p.ws_ml[(grow * p.num_splits + split) * 2] = -INFINITY; p.ws_ml[(grow * p.num_splits + split) * 2 + 1] = 0.f; }
        }
        return;
    }
    // softmax warps whose 32 rows hold no query (a decode step fills the first quarter or two) take no part:
    // the barriers count the others only
    const int nquarters = (rows_here + 31) / 32;
    const uint32_t softmax_threads = 32u * NP * (uint32_t)nquarters;
    const uint32_t bar0 = smem_u32(&bars[0]);
#define BAR(i) (bar0 + 8u * (uint32_t)(i))

    // The start of a CTA, side by side (a decode step's CTA walks only a tile or two, so this counts): warp 1 sets up
    // the barriers, warp 0 allocates tensor memory and looks up the pages of the first two tiles (the small loads
    // only - their copies go out after the queries, or the queries would queue behind 128 KB of tiles), and the
    // softmax warps stage the queries.
    int y_first = 0;                                              // warp 0, lane = tile * boxes + box: first row of that box in the page matrix
    if (warp == 1) {
        if (lane == 0) {
            for (int i = 0; i < NBARS; ++i) {
                const bool many = (i >= OE && i < OE + 2) || (i >= PF && i < PF + 2) || i >= XB;      // arrivals of the softmax threads; the rest: one commit or copy
                mbar_init(BAR(i), many ? softmax_threads : 1u);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
    } else if (warp == 0) {
        if (!AHEAD) {
            const int ps = p.page_size;
            const int box_rows = ps < BN ? ps : BN, nboxes = BN / box_rows;            // at most 16 boxes per tile
            const int jt = lane / nboxes, bx = lane - jt * nboxes;
            if (jt < 2 && jt < ntiles) {
                const int key = (t_begin + jt) * BN + bx * box_rows;
                const int pg = key / ps;
                const int page = pg < p.table_width ? p.block_table[(size_t)seq * p.table_width + pg] : 0;
                y_first = (page * p.Hkv + kvh) * ps + (key - pg * ps);
            }
        }
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        pdl_wait();                                                // this warp asks for the pages the predecessor has just written
    } else {
        // queries of the tile -> shared memory in the K-major swizzled operand layout (they are the predecessor's output)
        pdl_wait();
        for (int c = threadIdx.x - 64; c < p.q_rows * (D / 8); c += blockDim.x - 64) {
            const int r = c / (D / 8), chunk = c - r * (D / 8);      // chunk: 8 bfloat16 = 16 bytes
            const int row = row0 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row < nrows) {
                const int tok = row / G, g = row - tok * G;
                v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + chunk * 8);
            }
            const int blk = chunk >> 3, cin = chunk & 7;
            *reinterpret_cast<uint4*>(Qs + blk * QBLK + r * 128 + ((cin ^ (r & 7)) << 4)) = v;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes of Q become visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    // (No griddepcontrol.launch_dependents here: with it the merge kernel's CTAs sit beside this kernel's from its start, and
    // a decode step of 8 requests at 4,096 tokens was measured at 3.00 ms instead of 2.74.  Asking for the successor only
    // when a CTA starts its last tile costs as well: 2.95 ms instead of 2.69, the kernel alone 10.4 instead of 9.0 us at
    // 2,048 keys.  The successor is scheduled as this grid's CTAs exit.)

    if (warp == 0 && AHEAD) {
        // Prompt portions.  The whole warp walks the tiles: lane b looks up the page of box b (a
        // tile is 128 / box_rows boxes) one tile ahead, so the table's latency hides behind the waits, and issues
        // that box's copies; lane 0 waits for the stages.
        const int ps = p.page_size;
        const int box_rows = ps < BN ? ps : BN, nboxes = BN / box_rows;
        const int* table = p.block_table + (size_t)seq * p.table_width;
        auto box_row = [&](int j) -> int {                      // first row of this lane's box of tile j in the page matrix
            int y = 0;
            if (lane < nboxes && j < ntiles) {
                const int key = (t_begin + j) * BN + lane * box_rows;
                const int pg = key / ps;
                const int page = pg < p.table_width ? table[pg] : 0;
                y = (page * p.Hkv + kvh) * ps + (key - pg * ps);
            }
            return y;
        };
        int y_cur = box_row(0);
        for (int j = 0; j < ntiles; ++j) {
            const int y_next = box_row(j + 1);
            const int st = j % NST;
            const uint32_t par = ((j / NST) & 1) ^ 1;
            int ok = 1;
            if (lane == 0) ok = mbar_wait_relaxed(BAR(KE + st), par, 1);
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            if (lane == 0) mbar_expect_tx(BAR(KF + st), KV_BYTES);
            __syncwarp();
            if (lane < nboxes) {
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(smem_u32(Ks + st * KV_BYTES + cb * KVBLK + lane * box_rows * 128), &tmK, BAR(KF + st), cb * 64, y_cur);
            }
            if (lane == 0) ok = mbar_wait_relaxed(BAR(VE + st), par, 2);
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            if (lane == 0) mbar_expect_tx(BAR(VF + st), KV_BYTES);
            __syncwarp();
            if (lane < nboxes) {
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(smem_u32(Vs + st * KV_BYTES + cb * KVBLK + lane * box_rows * 128), &tmV, BAR(VF + st), cb * 64, y_cur);
            }
            y_cur = y_next;
        }
    } else if (warp == 0 && !AHEAD) {
        // Few rows (decode steps).  Lane b owns box b of a tile (a tile is 128 / box_rows boxes, 16 of them with 8-key
        // pages): it looks the box's page up - one coalesced read of the table for the whole tile, ahead of the wait for
        // the stage - and issues the box's copies itself, for the keys and then, from the same look-up, for the values.
        // (One thread that looked up and issued box after box took 7,400 clocks per 128-key tile with 16-key pages.)
        const int ps = p.page_size;
        const int box_rows = ps < BN ? ps : BN, nboxes = BN / box_rows;
        const int* table = p.block_table + (size_t)seq * p.table_width;
        auto box_row = [&](int j) -> int {                      // first row of this lane's box of tile j in the page matrix
            int y = 0;
            if (lane < nboxes && j < ntiles) {
                const int key = (t_begin + j) * BN + lane * box_rows;
                const int pg = key / ps;
                const int page = pg < p.table_width ? table[pg] : 0;
                y = (page * p.Hkv + kvh) * ps + (key - pg * ps);
            }
            return y;
        };
        {
            // the first two tiles (both stages are free): their pages were looked up while the queries were staged
            // (lane = tile * boxes + box)
            const int jt = lane / nboxes, bx = lane - jt * nboxes;
            for (int j = 0; j < 2 && j < ntiles; ++j) {
                if (lane == 0) { mbar_expect_tx(BAR(KF + j), KV_BYTES); mbar_expect_tx(BAR(VF + j), KV_BYTES); }
                __syncwarp();
                if (jt == j) {
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb)
                        tma_load_2d(smem_u32(Ks + j * KV_BYTES + cb * KVBLK + bx * box_rows * 128), &tmK, BAR(KF + j), cb * 64, y_first);
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb)
                        tma_load_2d(smem_u32(Vs + j * KV_BYTES + cb * KVBLK + bx * box_rows * 128), &tmV, BAR(VF + j), cb * 64, y_first);
                }
            }
        }
        int y_cur = box_row(2);
        for (int j = 2; j < ntiles; ++j) {
            const int y_next = box_row(j + 1);
            const int st = j % NST;
            const uint32_t par = ((j / NST) & 1) ^ 1;
            int ok = 1;
            if (lane == 0) { ok = mbar_wait(BAR(KE + st), par, 1); if (ok) mbar_expect_tx(BAR(KF + st), KV_BYTES); }
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            if (lane < nboxes) {
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(smem_u32(Ks + st * KV_BYTES + cb * KVBLK + lane * box_rows * 128), &tmK, BAR(KF + st), cb * 64, y_cur);
            }
            if (lane == 0) { ok = mbar_wait(BAR(VE + st), par, 2); if (ok) mbar_expect_tx(BAR(VF + st), KV_BYTES); }
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            if (lane < nboxes) {
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(smem_u32(Vs + st * KV_BYTES + cb * KVBLK + lane * box_rows * 128), &tmV, BAR(VF + st), cb * 64, y_cur);
            }
            y_cur = y_next;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // S = Q K^T: D float32, A and B bfloat16 K-major, M = 128, N = 128
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // O_tile = P V: B (values) MN-major, N = D
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // the issuing thread's own instructions count (a product takes 64 clocks): descriptor words one addition away
            uint32_t q_lo[CB];
#pragma unroll
            for (int cb = 0; cb < CB; ++cb) q_lo[cb] = desc_lo(smem_u32(Qs + cb * QBLK), 16);
            const uint32_t ks_lo = desc_lo(smem_u32(Ks), 16), vs_lo = desc_lo(smem_u32(Vs), KVBLK);
            auto issue_s = [&](int j) -> bool {
                const int st = j % NST, sb = j & 1;
                if (!mbar_wait(BAR(KF + st), (j / NST) & 1, 3)) return false;
                if (!mbar_wait(BAR(SE + sb), ((j >> 1) & 1) ^ 1, 4)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_lo = ks_lo + (uint32_t)st * (KV_BYTES >> 4), d = tmem_base + S_COL + (uint32_t)sb * BN;
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (cb | k) umma_ss_lean<true>(d, q_lo[cb] + 2 * k, k_lo + cb * (KVBLK >> 4) + 2 * k, idesc_s);
                        else umma_ss_lean<false>(d, q_lo[cb] + 2 * k, k_lo + cb * (KVBLK >> 4) + 2 * k, idesc_s);
                    }
                umma_commit(BAR(SF + sb));
                umma_commit(BAR(KE + st));
                return true;
            };
            bool ok = ntiles > 0 ? issue_s(0) : true;
            for (int j = 0; j < ntiles && ok; ++j) {
                if (j + 1 < ntiles) { ok = issue_s(j + 1); if (!ok) break; }
                const int st = j % NST, ob = j & 1;
                if (!mbar_wait(BAR(VF + st), (j / NST) & 1, 5)) { ok = false; break; }
                if (!mbar_wait(BAR(OE + ob), ((j >> 1) & 1) ^ 1, 6)) { ok = false; break; }
                if (!mbar_wait(BAR(PF + (j & 1)), (j >> 1) & 1, 7)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_lo = vs_lo + (uint32_t)st * (KV_BYTES >> 4), o_tmem = tmem_base + O_COL + (uint32_t)ob * D;
                const uint32_t p_tmem = tmem_base + S_COL + (uint32_t)(j & 1) * BN;     // P sits where the tile's scores sat
                umma_ts_lean<false>(o_tmem, p_tmem, v_lo, idesc_o);
#pragma unroll
                for (int k = 1; k < BN / 16; ++k) umma_ts_lean<true>(o_tmem, p_tmem + (uint32_t)(k * 8), v_lo + k * 128, idesc_o);   // 16 keys = 2048 bytes on
                umma_commit(BAR(OF + ob));
                umma_commit(BAR(VE + st));
                umma_commit(BAR(SE + (j & 1)));                         // scores / P buffer of this tile is free again
            }
        }
    } else if ((warp & 3) < nquarters) {
        // softmax: NP threads per row (warps w, w+4, w+8, ... reach the same 32 lanes of tensor memory); each
        // owns one part of the tile's 128 score columns and one part of the output columns.  Only the row
        // maximum is exchanged per tile (shared memory + an mbarrier with a bounded wait); the row sums are
        // added at the end.  A thread reads its scores once and keeps them in registers across the exchange.
        const int quarter = warp & 3, part = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const int row = row0 + r;
        const bool valid = row < nrows;
        const int tok = valid ? row / G : 0, g = valid ? row - tok * G : 0;
        const int pos = valid ? ctx + tok : -1;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr int SC = BN / NP, OC = D / NP;                        // score and output columns of this thread
        static_assert(SC == 32 && (OC == 32 || OC == 16), "one tcgen05.ld per tile for the scores and one for the output");
        float o[OC];
#pragma unroll
        for (int i = 0; i < OC; ++i) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
        bool ok = true;
        for (int j = 0; j <= ntiles && ok; ++j) {
            if (j < ntiles) {
                const int sb = j & 1;
                ok = mbar_wait(BAR(SF + sb), (j >> 1) & 1, 8);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int key0 = (t_begin + j) * BN;
                // columns lo_col..hi_col of this tile are visible to the row; a tile that every row of the warp
                // sees whole takes the path without compares
                const int hi_col = valid ? pos - key0 : -1, lo_col = lo - key0;
                const bool tile_full = __all_sync(0xffffffffu, valid && hi_col >= BN - 1 && lo_col <= 0);
                uint32_t sv[SC];
                tmem_ld32(lane_addr + S_COL + sb * BN + part * SC, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (!tile_full) {
#pragma unroll
                    for (int i = 0; i < SC; ++i) {
                        const int col = part * SC + i;
                        if (!(col <= hi_col && col >= lo_col)) sv[i] = 0xff800000u;                   // -inf
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains instead of one
#pragma unroll
                for (int i = 0; i < SC; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // exchange with the threads that own the other parts of the row (a bounded wait, not bar.sync:
                // a warp that gave up elsewhere must not leave the others waiting for ever)
                xch[j & 1][part][r] = mx;
                mbar_arrive(BAR(XB + (j & 1)));
                ok = mbar_wait(BAR(XB + (j & 1)), (j >> 1) & 1, 11);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
#pragma unroll
                for (int k = 0; k < NP; ++k) mx = fmaxf(mx, xch[j & 1][k][r]);
                mx *= p.scale_log2;                                      // -inf stays -inf (the scale is positive)
                const float m_new = fmaxf(m_run, mx);
                const float msub = m_new == -INFINITY ? 0.f : m_new;
                const float alpha = m_new == -INFINITY ? 1.f : ex2(m_run - m_new);
                // probabilities, rounded to bfloat16 into the operand layout; their sum in float32
                float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t packed[SC / 2];
#pragma unroll
                for (int i = 0; i < SC; i += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(sv[i]), p.scale_log2, -msub));
                    const float p1 = ex2(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -msub));
                    ls4[(i >> 1) & 3] += p0 + p1;
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                }
                // P over the scores of this tile: every thread of the row has its scores in registers (the exchange
                // above came after the loads), so the columns can be overwritten; 32 keys = 16 packed columns
                tmem_st16(lane_addr + S_COL + sb * BN + part * (SC / 2), packed);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                l_run = l_run * alpha + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
                m_run = m_new;
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(BAR(PF + sb));                              // P is in tensor memory
                // rescale what has been summed so far to the new maximum
                if (alpha != 1.f) {
#pragma unroll
                    for (int i = 0; i < OC; ++i) o[i] *= alpha;
                }
                alpha_prev = alpha;
            }
            if (j > 0) {
                // take the previous tile's product out of tensor memory.  It was computed with the maximum of
                // tile j-1; the rescale for tile j (alpha above) must apply to it as well.
                const int ob = (j - 1) & 1;
                ok = mbar_wait(BAR(OF + ob), ((j - 1) >> 1) & 1, 10);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float f = j < ntiles ? alpha_prev : 1.f;
                uint32_t ov[OC];
                tmem_ld_cols(lane_addr + O_COL + ob * D + part * OC, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(BAR(OE + ob));
#pragma unroll
                for (int i = 0; i < OC; ++i) o[i] = fmaf(__uint_as_float(ov[i]), f, o[i]);
            }
        }
        // the parts of a row add their sums (in part order)
        float l_tot = 0.f;
        if (ok) {
            xch[ntiles & 1][part][r] = l_run;                            // the buffer the last tile did not use
            mbar_arrive(BAR(XL));
            ok = mbar_wait(BAR(XL), 0, 12);
#pragma unroll
            for (int k = 0; k < NP; ++k) l_tot += xch[ntiles & 1][k][r];
        }
        if (ok && valid && p.num_splits > 1) {
            const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
            float* dst = p.ws_o + (grow * p.num_splits + split) * D + part * OC;
#pragma unroll
            for (int i = 0; i < OC; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
            if (part == 0) {
                float* ml = p.ws_ml + (grow * p.num_splits + split) * 2;
                ml[0] = m_run * 0.6931471805599453f;                 // natural-log units for the merge
                ml[1] = l_tot;
            }
        } else if (ok && valid) {
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            __nv_bfloat16* dst = p.out + ((size_t)(q0 + tok) * p.Hq + kvh * G + g) * D + part * OC;
#pragma unroll
            for (int i = 0; i < OC; i += 8) {
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(o[i + 2 * k] * inv, o[i + 2 * k + 1] * inv);
                    w[k] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
#undef BAR
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA: the form for prompt portions.
//
// A CTA owns 256 query rows as two 128-row tiles that share every key/value tile, and walks the keys 64 at a time.
// Each query tile has TWO score buffers in tensor memory, so the scores of key step j+1 are computed while the
// softmax threads work on step j; and there are two query tiles, so the tensor core always has the other tile's
// products to do.  Tensor memory: 2 tiles x 2 buffers x 64 columns of scores, 2 x D columns of output.
//   warps 0-3    softmax of tile 0, ONE thread per row: the 64 scores of a key step come out of tensor memory into
//                registers, so row maximum and sum need no exchange between threads; P (bfloat16) goes back over
//                the scores and is the tensor-memory A operand of O += P V
//   warps 4-7    the same for tile 1
//   warps 8-11   correction: the running output stays in tensor memory (O += P V accumulates there); when a row's
//                maximum has grown by more than 2^8 since its output was last scaled, these warps scale the row of O
//                (tcgen05.ld / st).  Below that threshold the old maximum stays in use - P is then at most 2^8, which
//                costs bfloat16 nothing - so after the first steps O is rarely touched.  At the end they divide by
//                the row sum and store.
//   warp 12      TMA producer: key and value tiles through one ring, in the order the products need them
//                (K0 K1 V0 K2 V1 K3 ...)
//   warps 13-14  one thread each issues  O += P(j) V(j)  of one tile
//   warp 15      one thread issues the scores  S(j) = Q K(j)^T  of both tiles, as soon as K(j) is there and P(j-2) is used up
// Register budgets follow the roles (setmaxnreg).  Threads of one role run up to two steps apart, so every barrier
// that counts thread arrivals exists twice (by step parity).
namespace pp {
constexpr int BNK = 64;                                          // keys per step
constexpr int NS = 8;                                            // stages of the key/value ring (head size 256: 4 of them, of twice the size)
enum { PP_FULL = 0, PP_EMPTY = NS, PP_SF = 2 * NS, PP_PF = PP_SF + 4, PP_SC = PP_PF + 4, PP_OC = PP_SC + 4, PP_OF = PP_OC + 4,
       PP_LF = PP_OF + 4, PP_NBARS = PP_LF + 2 };                // SF, PF, SC, OC, OF: [tile][step parity]
constexpr int PP_NTHREADS = 512;
constexpr float RESCALE_LOG2 = 8.f;                              // a row's output is rescaled when its maximum grew by more
}

// Two float32 operations in one instruction (fma.rn.f32x2 / add.rn.f32x2 of sm_100): the softmax threads are short of
// issue slots, not of arithmetic.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}" : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {      // (d0, d1) += (a0, a1)
    asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}

// NT: query tiles per CTA.  Tensor memory holds 2 x 2 x 64 score columns and NT x D output columns: two tiles up to
// head size 128, one tile (its scores at columns 0..127, its output at 256..511) at head size 256.
template <int D, int NT>
__global__ void __launch_bounds__(pp::PP_NTHREADS, 1)
attn_tc_pp_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
    using namespace pp;
    static_assert(256 + NT * D <= 512, "tensor memory: scores of two tiles, then the output tiles");
    constexpr int NSD = D > 128 ? 4 : NS;                        // ring stages in use (a stage is D x 64 x 2 bytes)
    constexpr int CB = D / 64;
    constexpr uint32_t QBLK = BM * 128, KVBLK = BNK * 128;       // bytes of one 64-column block of a query / key tile
    constexpr uint32_t QT_BYTES = CB * QBLK, KV_BYTES = CB * KVBLK;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t S_COL = 0, O_COL = 256;                   // scores of (tile t, buffer b) at t * 128 + b * 64; output of tile t at 256 + t * D
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = smem;                                    // [NT tiles]
    unsigned char* ring = Qs + NT * QT_BYTES;                    // [NSD stages]
    __shared__ __align__(8) unsigned long long bars[PP_NBARS];
    __shared__ uint32_t tmem_slot;
    __shared__ float alpha_s[2][2][BM];                          // [step parity][tile]: factor for a row of O before the step's product is added
    __shared__ float lsum_s[2][BM], mrun_s[2][BM];               // a row's sum and the maximum it is relative to, at the end

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.Hq / p.Hkv;
    int tile = blockIdx.x;
    const int rt = p.row_tiles - 1 - tile % p.row_tiles;         // long (late) tiles first
    tile /= p.row_tiles;
    const int kvh = tile % p.Hkv, seq = tile / p.Hkv;
    const int q0 = p.qsl[seq], q_len = p.qsl[seq + 1] - q0, kv_len = p.seq_lens[seq];
    const int nrows = q_len * G, row0 = rt * (NT * BM);
    if (row0 >= nrows) return;                                   // uniform over the CTA, before anything is allocated
    const int ctx = kv_len - q_len;
    const int rows_here = min(NT * BM, nrows - row0);
    const int tok_lo = row0 / G, tok_hi = (row0 + rows_here - 1) / G;
    int key_hi = ctx + tok_hi + 1;                               // exclusive
    int key_lo = p.window > 0 ? max(0, ctx + tok_lo - p.window + 1) : 0;
    const int split = blockIdx.y;
    if (p.num_splits > 1) {
        const int piece = piece_len(kv_len, p.num_splits, p.split_len, BN);
        key_lo = max(key_lo, split * piece);
        key_hi = min(key_hi, (split + 1) * piece);
    }
    const int t_begin = key_lo / BNK, t_end = (key_hi + BNK - 1) / BNK;
    const int nsteps = t_end - t_begin;
    if (nsteps <= 0) {
        // (only with splits) no key of this split is visible: an empty partial result, nothing allocated.  The scratch
        // memory may still be read by the merge kernel of the launch before this one: wait for it first.
        pdl_wait();
        for (int e = threadIdx.x; e < rows_here * D; e += blockDim.x) {
            const int r = e / D, row = row0 + r;
            const int tok = row / G, g = row - tok * G;
            const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
            p.ws_o[(grow * p.num_splits + split) * D + (e - r * D)] = 0.f;
            if (e - r * D == 0) { p.ws_ml[(grow * p.num_splits + split) * 2] = -INFINITY; p.ws_ml[(grow * p.num_splits + split) * 2 + 1] = 0.f; }
        }
        return;
    }
    const int ntq = rows_here > BM ? 2 : 1;                      // query tiles in use
    const uint32_t bar0 = smem_u32(&bars[0]);
#define BAR(i) (bar0 + 8u * (uint32_t)(i))

    if (warp == 13 && lane == 0) {
        for (int i = 0; i < PP_NBARS; ++i)                       // PF, SC, OC, LF count thread arrivals, EMPTY the issuers; the rest one commit or copy
            mbar_init(BAR(i), (i >= PP_PF && i < PP_OF) || i >= PP_LF ? 128u : (i >= PP_EMPTY && i < PP_SF) ? (uint32_t)ntq : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // queries of both tiles -> shared memory in the K-major swizzled operand layout (rows past the end: zeros).  They and
    // the newest pages are the predecessor's output: what stands above ran while that kernel was finishing.
    pdl_wait();
    for (int c = threadIdx.x; c < ntq * BM * (D / 8); c += PP_NTHREADS) {
        const int r = c / (D / 8), chunk = c - r * (D / 8);      // chunk: 8 bfloat16 = 16 bytes
        const int row = row0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < nrows) {
            const int tok = row / G, g = row - tok * G;
            v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)(kvh * G + g) * D + chunk * 8);
        }
        const int qt = r >> 7, rr = r & 127, blk = chunk >> 3, cin = chunk & 7;
        *reinterpret_cast<uint4*>(Qs + qt * QT_BYTES + blk * QBLK + rr * 128 + ((cin ^ (rr & 7)) << 4)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes of Q become visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp < 8) {
        // ---------------------------------------------------------------- softmax of tile t, one thread per row
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;" ::: "memory");
        const int t = warp >> 2;
        if (t < ntq) {
            const int quarter = warp & 3, r = quarter * 32 + lane;
            const int row = row0 + t * BM + r;
            const bool valid = row < nrows;
            const int tok = valid ? row / G : 0;
            const int pos = valid ? ctx + tok : -1;
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const uint32_t s_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + S_COL + (uint32_t)t * 128;
            const float sl2 = p.scale_log2;
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < nsteps; ++j) {
                const int b = j & 1;
                const uint32_t par = (j >> 1) & 1;
                const uint32_t s_addr = s_base + (uint32_t)b * BNK;
                ok = mbar_wait(BAR(PP_SF + 2 * t + b), par, 8);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t sv[BNK];
#pragma unroll
                for (int c = 0; c < BNK / 32; ++c) tmem_ld32(s_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int key0 = (t_begin + j) * BNK;
                const int hi_col = valid ? pos - key0 : -1, lo_col = lo - key0;
                const bool tile_full = __all_sync(0xffffffffu, valid && hi_col >= BNK - 1 && lo_col <= 0);
                if (!tile_full) {
#pragma unroll
                    for (int i = 0; i < BNK; ++i)
                        if (!(i <= hi_col && i >= lo_col)) sv[i] = 0xff800000u;                   // -inf
                }
                float mx8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(__uint_as_float(sv[i]), __uint_as_float(sv[i + 8]));
#pragma unroll
                for (int i = 16; i < BNK; i += 16)
#pragma unroll
                    for (int k = 0; k < 8; ++k) mx8[k] = fmaxf(mx8[k], fmaxf(__uint_as_float(sv[i + k]), __uint_as_float(sv[i + 8 + k])));
                const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                                       fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * sl2;   // -inf stays -inf (the scale is positive)
                // The maximum in use moves only when it has grown by more than the threshold (or was -inf): then the
                // row of O is scaled by alpha before this step's product is added.
                const float m_cand = fmaxf(m_run, mx);
                const bool up = (m_cand - m_run) > RESCALE_LOG2;             // false for -inf - -inf (NaN)
                const float alpha = up ? ex2(m_run - m_cand) : 1.f;
                m_run = up ? m_cand : m_run;
                alpha_s[b][t][r] = j > 0 ? alpha : 1.f;                      // nothing to scale before the first product
                mbar_arrive(BAR(PP_SC + 2 * t + b));
                const float msub = m_run == -INFINITY ? 0.f : m_run;
                float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                const float nmsub = -msub;
#pragma unroll
                for (int c = 0; c < BNK / 32; ++c) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float x0, x1;
                        fma2(x0, x1, __uint_as_float(sv[c * 32 + i]), __uint_as_float(sv[c * 32 + i + 1]), sl2, nmsub);
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        add2(ls4[(i >> 1) & 1], ls4[2 + ((i >> 1) & 1)], p0, p1);
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    tmem_st16(s_addr + c * 16, packed);                  // P over the scores: 32 keys = 16 packed columns
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(BAR(PP_PF + 2 * t + b));                     // P is in tensor memory
                l_run = l_run * alpha + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
            }
            if (ok) {
                lsum_s[t][r] = l_run;
                mrun_s[t][r] = m_run;
                mbar_arrive(BAR(PP_LF + t));
            }
        }
    } else if (warp < 12) {
        // ---------------------------------------------------------------- correction and epilogue
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;" ::: "memory");
        const int quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        // A parity wait tells "phase k is over" from "phase k is running" only.  The softmax - hence this warp - may be
        // two steps ahead of the products, and this warp does not look at every product, so the products of a tile
        // signal two barriers in turn (by step parity): whoever waits for product j is then at most one phase of
        // that barrier away from it.
        auto product_done = [&](int t, int j) -> bool {         // waits until product j of tile t has landed
            return __all_sync(0xffffffffu, mbar_wait(BAR(PP_OF + 2 * t + (j & 1)), (j >> 1) & 1, 10));
        };
        for (int j = 0; j < nsteps && ok; ++j) {
            const int b = j & 1;
            const uint32_t par = (j >> 1) & 1;
            for (int t = 0; t < ntq; ++t) {
                ok = mbar_wait(BAR(PP_SC + 2 * t + b), par, 9);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const float a = alpha_s[b][t][r];
                if (__any_sync(0xffffffffu, a != 1.f)) {                // never in step 0
                    ok = product_done(t, j - 1);                        // the product of the step before has landed
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t ov[32];
                        tmem_ld32(lane_addr + O_COL + t * D + c * 32, ov);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * a);
                        tmem_st32(lane_addr + O_COL + t * D + c * 32, ov);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(BAR(PP_OC + 2 * t + b));
            }
        }
        for (int t = 0; t < ntq && ok; ++t) {
            ok = mbar_wait(BAR(PP_LF + t), 0, 12);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) ok = product_done(t, nsteps - 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = row0 + t * BM + r;
            const bool valid = row < nrows;
            const int tok = valid ? row / G : 0, g = valid ? row - tok * G : 0;
            const size_t grow = (size_t)(q0 + tok) * p.Hq + kvh * G + g;
            const float l_tot = lsum_s[t][r];
            const bool partial = p.num_splits > 1;
            const float inv = partial ? 1.f : (l_tot > 0.f ? 1.f / l_tot : 0.f);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t ov[32];
                tmem_ld32(lane_addr + O_COL + t * D + c * 32, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!valid) continue;
                if (partial) {
                    float* dst = p.ws_o + (grow * p.num_splits + split) * D + c * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(ov[i]), __uint_as_float(ov[i + 1]),
                                                                          __uint_as_float(ov[i + 2]), __uint_as_float(ov[i + 3]));
                } else {
                    __nv_bfloat16* dst = p.out + grow * D + c * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * k]) * inv, __uint_as_float(ov[i + 2 * k + 1]) * inv);
                            w[k] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            if (valid && partial) {
                float* ml = p.ws_ml + (grow * p.num_splits + split) * 2;
                ml[0] = mrun_s[t][r] * 0.6931471805599453f;          // natural-log units for the merge
                ml[1] = l_tot;
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 48;" ::: "memory");
        if (warp == 12) {
            // ------------------------------------------------------------ copy producer: K0 K1 V0 K2 V1 K3 ... through the ring.
            // Lane x looks up the page of box x of a tile (a tile is 64 / box_rows boxes) ahead of its use and issues that
            // box's copies; lane 0 waits for the stage.
            const int ps = p.page_size;
            const int box_rows = ps < BNK ? ps : BNK, nboxes = BNK / box_rows;
            const int* table = p.block_table + (size_t)seq * p.table_width;
            auto box_row = [&](int j) -> int {                  // first row of this lane's box of tile j in the page matrix
                int y = 0;
                if (lane < nboxes && j < nsteps) {
                    const int key = (t_begin + j) * BNK + lane * box_rows;
                    const int pg = key / ps;
                    const int page = pg < p.table_width ? table[pg] : 0;
                    y = (page * p.Hkv + kvh) * ps + (key - pg * ps);
                }
                return y;
            };
            int it = 0;                                         // tiles copied so far
            auto emit = [&](const CUtensorMap* map, int y_lane, int code) -> bool {
                const int st = it % NSD;
                int ok = 1;
                if (lane == 0) ok = mbar_wait_relaxed(BAR(PP_EMPTY + st), ((it / NSD) & 1) ^ 1, code);
                if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
                if (lane == 0) mbar_expect_tx(BAR(PP_FULL + st), KV_BYTES);
                __syncwarp();
                if (lane < nboxes) {                                // every lane issues the copies of its own box
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb)
                        tma_load_2d(smem_u32(ring + st * KV_BYTES + cb * KVBLK + lane * box_rows * 128), map, BAR(PP_FULL + st), cb * 64, y_lane);
                }
                ++it;
                return true;
            };
            int y0 = box_row(0), y1 = box_row(1), y2 = box_row(2);   // tiles j, j+1, j+2
            bool go = emit(&tmK, y0, 1);
            if (go && nsteps > 1) go = emit(&tmK, y1, 1);
            for (int j = 0; j < nsteps && go; ++j) {
                const int y3 = box_row(j + 3);
                go = emit(&tmV, y0, 2);
                if (go && j + 2 < nsteps) go = emit(&tmK, y2, 1);
                y0 = y1; y1 = y2; y2 = y3;
            }
        } else if (lane == 0) {
            // ------------------------------------------------------------ product issuers
            // Measured on this part: after a thread has issued tcgen05.mma, its next instruction that touches memory
            // or a barrier - an mbarrier wait, a flag poll, a named barrier; tcgen05.commit itself costs 46 clocks -
            // does not complete until those products have finished, 160-260 clocks after the tensor core is done with
            // them.  One issuing thread therefore leaves the tensor core idle for that long between batches.  Three
            // threads issue here, each blocked only behind its own batch: warp 15 the scores of both tiles, warps 13
            // and 14 the P V products of one tile each.  Between threads nothing is ordered by issue: S(j+2) goes over
            // P(j) only after the barrier of O += P(j) V(j) has completed.
            // A product of 48-64 clocks leaves its thread a dozen instructions: the descriptors' upper words are
            // constants, the lower words are one addition away from values kept in registers.
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNK >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // position of a tile in the ring's order K0 K1 V0 K2 V1 K3 ... V(n-2) V(n-1)
            auto k_index = [&](int j) { return j < 2 ? j : 2 * j - 1; };
            auto v_index = [&](int j) { return j == nsteps - 1 ? 2 * nsteps - 1 : 2 * j + 2; };
            if (warp == 15) {
                uint32_t q_lo[NT][CB];                          // lower descriptor words of the query blocks
#pragma unroll
                for (int t = 0; t < NT; ++t)
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb) q_lo[t][cb] = desc_lo(smem_u32(Qs + t * QT_BYTES + cb * QBLK), 16);
                const uint32_t ring_k_lo = desc_lo(smem_u32(ring), 16);
                for (int j = 0; j < nsteps; ++j) {
                    const int b = j & 1, idx = k_index(j), st = idx % NSD;
                    if (!mbar_wait(BAR(PP_FULL + st), (idx / NSD) & 1, 3)) break;
                    const uint32_t k_lo = ring_k_lo + (uint32_t)st * (KV_BYTES >> 4);
                    bool ok = true;
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        if (t < ntq) {
                            // the buffer holds P(j-2) until its product with V has finished
                            if (j >= 2 && !mbar_wait(BAR(PP_OF + 2 * t + b), ((j - 2) >> 1) & 1, 4)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            const uint32_t d = tmem_base + S_COL + (uint32_t)t * 128 + (uint32_t)b * BNK;
#pragma unroll
                            for (int cb = 0; cb < CB; ++cb)
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    if (cb | k) umma_ss_lean<true>(d, q_lo[t][cb] + 2 * k, k_lo + cb * (KVBLK >> 4) + 2 * k, idesc_s);
                                    else umma_ss_lean<false>(d, q_lo[t][cb] + 2 * k, k_lo + cb * (KVBLK >> 4) + 2 * k, idesc_s);
                                }
                            umma_commit(BAR(PP_SF + 2 * t + b));
                            umma_commit(BAR(PP_EMPTY + st));           // one arrival per tile in use
                        }
                    }
                    if (!ok) break;
                }
            } else if (warp - 13 < ntq) {
                const int t = warp - 13;
                const uint32_t ring_v_lo = desc_lo(smem_u32(ring), KVBLK);
                const uint32_t s_tmem = tmem_base + S_COL + (uint32_t)t * 128, o_tmem = tmem_base + O_COL + (uint32_t)t * D;
                for (int j = 0; j < nsteps; ++j) {
                    const int b = j & 1, idx = v_index(j), st = idx % NSD;
                    const uint32_t par = (j >> 1) & 1;
                    if (!mbar_wait(BAR(PP_FULL + st), (idx / NSD) & 1, 5)) break;
                    if (!mbar_wait(BAR(PP_PF + 2 * t + b), par, 7)) break;
                    if (!mbar_wait(BAR(PP_OC + 2 * t + b), par, 6)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t v_lo = ring_v_lo + (uint32_t)st * (KV_BYTES >> 4);
                    const uint32_t p_tmem = s_tmem + (uint32_t)b * BNK;      // P sits where the step's scores sat
                    if (j) umma_ts_lean<true>(o_tmem, p_tmem, v_lo, idesc_o);
                    else umma_ts_lean<false>(o_tmem, p_tmem, v_lo, idesc_o);
#pragma unroll
                    for (int k = 1; k < BNK / 16; ++k) umma_ts_lean<true>(o_tmem, p_tmem + (uint32_t)(k * 8), v_lo + k * 128, idesc_o);   // 16 keys = 2048 bytes on
                    umma_commit(BAR(PP_OF + 2 * t + b));
                    umma_commit(BAR(PP_EMPTY + st));
                }
            }
        }
    }
#undef BAR
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 12) {
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
// pages [num_pages][Hkv][page][D] seen as a matrix [num_pages*Hkv*page][D]; box = 64 columns x box_rows keys.
// A pool keeps its address for the life of an engine and every layer of every step asks for the same few maps, so the
// last ones made are kept (per host thread) and an encode is paid once per pool, layer and kernel form.
int encode_page_map(CUtensorMap* map, const void* base, long long rows, int D, int box_rows);
int make_page_map(CUtensorMap* map, const void* base, long long rows, int D, int box_rows) {
    struct Kept { const void* base; long long rows; int D, box_rows; CUtensorMap map; };
    constexpr int KEEP = 256;
    thread_local Kept kept[KEEP];
    thread_local int used = 0, next = 0;
    for (int i = 0; i < used; ++i)
        if (kept[i].base == base && kept[i].rows == rows && kept[i].D == D && kept[i].box_rows == box_rows) { *map = kept[i].map; return 0; }
    if (encode_page_map(map, base, rows, D, box_rows)) return -1;
    Kept& k = kept[next];
    k.base = base; k.rows = rows; k.D = D; k.box_rows = box_rows; k.map = *map;
    next = (next + 1) % KEEP;
    if (used < KEEP) ++used;
    return 0;
}
int encode_page_map(CUtensorMap* map, const void* base, long long rows, int D, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) TTIE_FAIL("attention_tc: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TTIE_FAIL("attention_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int D, bool AHEAD, int NST>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, cudaStream_t s) {
    const size_t smem = (size_t)(D / 64) * p.q_rows * 128 + 2 * NST * (size_t)(D / 64) * BN * 128 + 1024;
    const size_t most = (size_t)(D / 64) * (NST > 2 && D > 64 ? 64 : BM) * 128 + 2 * NST * (size_t)(D / 64) * BN * 128 + 1024;
    auto k = attn_tc_kernel<D, AHEAD, NST>;
    static bool allowed[64] = {false};                           // the attribute is set once per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!allowed[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) TTIE_FAIL("attention_tc: %zu bytes of shared memory refused: %s", most, cudaGetErrorString(e));
        allowed[dev] = true;
    }
    if (smem > most) TTIE_FAIL("attention_tc: %d staged query rows with %d stages do not fit", p.q_rows, NST);
    // a programmatic dependent of the kernel before it: its set-up (tensor memory, barriers, page look-ups) runs while
    // that kernel finishes; griddepcontrol.wait stands before the first read of queries and pages
    TTIE_LAUNCH(k, dim3(p.num_seqs * p.Hkv * p.row_tiles, p.num_splits), NTHREADS, smem, s, mk, mv, p);
    TTIE_CHECK_LAUNCH("attention_tc");
    return 0;
}
template <int D>
int launch_pp(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, cudaStream_t s) {
    constexpr int NT = D > 128 ? 1 : 2, NSD = D > 128 ? 4 : pp::NS;
    const size_t smem = NT * (size_t)(D / 64) * BM * 128 + NSD * (size_t)(D / 64) * pp::BNK * 128 + 1024;
    auto k = attn_tc_pp_kernel<D, NT>;
    static bool allowed[64] = {false};                           // the attribute is set once per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!allowed[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) TTIE_FAIL("attention_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        allowed[dev] = true;
    }
    TTIE_LAUNCH(k, dim3(p.num_seqs * p.Hkv * p.row_tiles, p.num_splits), pp::PP_NTHREADS, smem, s, mk, mv, p);
    TTIE_CHECK_LAUNCH("attention_tc (two query tiles)");
    return 0;
}
}  // namespace

// The path a kernel takes when a barrier never completes, run on purpose and briefly: one thread waits with the
// kernels' own bounded wait, and a limit of the caller's choosing, on a barrier at which nobody arrives.  The wait runs
// out, records `code` in the error word and its host mirror as it would in an attention kernel, and the kernel returns.
__global__ void wait_selftest_kernel(long long limit_cycles, int code, int* gave_up) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) *gave_up = mbar_wait(smem_u32(&bar), 0, code, limit_cycles) ? 0 : 1;
}
extern "C" int ttie_attn_tc_wait_selftest(long long limit_cycles, int code, int* gave_up, void* stream) {
    if (limit_cycles <= 0 || limit_cycles > 200000000LL) TTIE_FAIL("wait self-test: limit of %lld clocks (1 .. 200,000,000)", limit_cycles);
    if (!gave_up) TTIE_FAIL("wait self-test: no result word");
    wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_cycles, code, gave_up);
    TTIE_CHECK_LAUNCH("wait self-test");
    return 0;
}

// A word of pinned host memory (device-accessible) that also receives the failure code, so the host can look at it
// after every step without a call into the runtime.  nullptr: none.
extern "C" int ttie_attn_tc_set_mirror(int* host_word) {
    return cudaMemcpyToSymbol(g_attn_tc_error_mirror, &host_word, sizeof(int*)) == cudaSuccess ? 0 : 1;
}

extern "C" int ttie_attn_tc_error() {
    int v = 0, zero = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}

// Head size 64, 128 or 256 (256: the two-tile kernel's form only, with one tile); page size a multiple of 8 that
// divides 128 or is a multiple of 128.
extern "C" int ttie_attn_tc_supported(int D, int page_size) {
    return (D == 64 || D == 128 || D == 256) && page_size >= 8 && page_size % 8 == 0 && (128 % page_size == 0 || page_size % 128 == 0) && page_size <= 256;
}

// two_tiles: 0 = a CTA owns one 128-row query tile (any number of rows; decode steps; head size 64 or 128), 1 = the
// kernel for prompt portions: a CTA owns 256 rows as two tiles taken in turns (128 rows as one tile at head size 256).
// num_splits > 1: the key range is cut into pieces of split_len keys (a multiple of 128) over grid y; the partial
// results go to `scratch` (ttie_attn_scratch_floats) and a merge kernel writes `out`.
extern "C" int ttie_paged_attention_tc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                       int num_pages, const int* block_table, int table_width, int page_size, const int* qsl,
                                       const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                       int max_q_len, float scale, int window, int num_splits, int split_len, float* scratch,
                                       int two_tiles, void* stream) {
    if (T <= 0 || num_seqs <= 0) return 0;
    if (!ttie_attn_tc_supported(D, page_size)) TTIE_FAIL("attention_tc: head size %d with pages of %d keys is not supported", D, page_size);
    if (Hkv <= 0 || Hq % Hkv) TTIE_FAIL("attention_tc: %d heads are not a multiple of %d kv heads", Hq, Hkv);
    if (q_stride % 8 || ((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out | (uintptr_t)scratch) & 15)
        TTIE_FAIL("attention_tc: pointers must be 16-byte aligned and the query stride a multiple of 8");
    if (D > 128 && !two_tiles) TTIE_FAIL("attention_tc: head size %d runs in the prompt-portion form only", D);
    if (num_splits < 1) num_splits = 1;
    if (num_splits > 1 && (split_len <= 0 || split_len % BN || !scratch))
        TTIE_FAIL("attention_tc: splits need scratch and a split length that is a multiple of %d", BN);
    if (num_splits > 65535) TTIE_FAIL("attention_tc: too many splits (%d)", num_splits);
    CUtensorMap mk, mv;
    const long long rows = (long long)num_pages * Hkv * page_size;
    const int tile_keys = two_tiles ? pp::BNK : BN;              // keys per copy tile of the kernel
    const int box_rows = page_size < tile_keys ? page_size : tile_keys;
    if (make_page_map(&mk, k_pages, rows, D, box_rows)) return -1;
    if (make_page_map(&mv, v_pages, rows, D, box_rows)) return -1;
    AttnTcParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.block_table = block_table; p.table_width = table_width;
    p.page_size = page_size; p.qsl = qsl; p.seq_lens = seq_lens; p.out = (__nv_bfloat16*)out;
    p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
    p.row_tiles = ceil_div(max_q_len * (Hq / Hkv), two_tiles && D <= 128 ? 2 * BM : BM);
    p.num_splits = num_splits; p.split_len = split_len;
    p.ws_o = scratch; p.ws_ml = scratch ? scratch + (size_t)T * Hq * num_splits * D : nullptr;
    if ((long long)num_seqs * Hkv * p.row_tiles > 2147483647LL) TTIE_FAIL("attention_tc: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    const int rows_most = max_q_len * (Hq / Hkv);
    const bool ahead = rows_most >= BM;                          // full row tiles: a prompt portion
    p.q_rows = ahead ? BM : 32 * ceil_div(rows_most, 32);
    const int rc = two_tiles ? (D == 64 ? launch_pp<64>(mk, mv, p, s) : D == 128 ? launch_pp<128>(mk, mv, p, s) : launch_pp<256>(mk, mv, p, s))
                 : D == 64 ? (ahead ? launch<64, true, 2>(mk, mv, p, s) : launch<64, false, 4>(mk, mv, p, s))
                           : (ahead ? launch<128, true, 2>(mk, mv, p, s)
                                    : p.q_rows <= 64 ? launch<128, false, 3>(mk, mv, p, s) : launch<128, false, 2>(mk, mv, p, s));
    if (rc) return rc;
    if (num_splits > 1) return attn_merge_bf16(p.ws_o, p.ws_ml, out, T * Hq, num_splits, D, s);
    return 0;
}
