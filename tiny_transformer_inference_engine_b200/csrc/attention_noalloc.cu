// The allocation-free variant of split-key paged attention (see attention_noalloc.h).
#include "attention_noalloc.h"
#include "common.cuh"
#include <mutex>
using namespace ttie;

// Scratch for split-key partial results, owned by the library, one copy per GPU that loads it.
// In host code this name is only a handle for cudaGetSymbolAddress - it is not a device address
// and must never be handed to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[TTIE_NOALLOC_SCRATCH_FLOATS];

extern "C" int ttie_paged_attention_mma(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_width, int page_size, const int* qsl,
                                        const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                        int max_q_len, float scale, int window, int num_splits, int split_len,
                                        float* scratch, void* stream);

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_addr[kMaxDevices] = {};            // device address of the array on each GPU, looked up once

// Device address of the scratch array on the current device; nullptr and an error message on failure.
float* scratch_on_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("noalloc attention: cudaGetDevice failed: %s", cudaGetErrorString(e)); return nullptr; }
    if (dev < 0 || dev >= kMaxDevices) { set_error("noalloc attention: device index %d out of range", dev); return nullptr; }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_addr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);      // with this device current
        if (e != cudaSuccess || !p) {
            set_error("noalloc attention: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        g_scratch_addr[dev] = p;
    }
    return g_scratch_addr[dev];
}
}  // namespace

extern "C" int ttie_paged_attention_mma_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                                const int* block_table, int table_width, int page_size, const int* qsl,
                                                const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                                int max_q_len, float scale, int window, int num_splits, int split_len,
                                                void* stream) {
    if (T <= 0 || num_seqs <= 0) return 0;
    if (num_splits < 1) num_splits = 1;
    float* scratch = nullptr;
    if (num_splits > 1) {
        const long long need = (long long)T * Hq * num_splits * (D + 2);
        if (need > (long long)TTIE_NOALLOC_SCRATCH_FLOATS)
            TTIE_FAIL("noalloc attention: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of scratch exceed the "
                      "library's %d; use fewer splits or the entry point that takes scratch from the caller",
                      T, Hq, num_splits, D, need, (int)TTIE_NOALLOC_SCRATCH_FLOATS);
        scratch = scratch_on_current_device();
        if (!scratch) return -3;
    }
    return ttie_paged_attention_mma(q, q_stride, k_pages, v_pages, block_table, table_width, page_size, qsl, seq_lens, out,
                                    T, num_seqs, Hq, Hkv, D, max_q_len, scale, window, num_splits, split_len, scratch, stream);
}
