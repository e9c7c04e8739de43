// Shared helpers of the sm_100a kernels: element types, conversions, reductions, error reporting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <cstdlib>

namespace ttie {

enum DType : int { kF32 = 0, kBF16 = 1 };

// Every exported function returns 0 or a negative code and leaves a message for ttie_last_error().
void set_error(const char* fmt, ...);
#define TTIE_FAIL(...) do { ::ttie::set_error(__VA_ARGS__); return -1; } while (0)
#define TTIE_CHECK_LAUNCH(what) do { cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) { ::ttie::set_error("%s: launch failed: %s", what, cudaGetErrorString(e_)); return -2; } } while (0)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// first statement of a kernel: wait for the predecessor's results, then let the successor be scheduled
#define TTIE_PDL_ENTRY() do { ::ttie::pdl_wait(); ::ttie::pdl_launch_dependents(); } while (0)

// Keys per piece for a request of kv_len keys, in a step that was planned as num_splits pieces of split_len keys for its
// longest request (or for the longest a captured graph may meet): an even share of the request's own keys, rounded up
// to the kernel's tile, never more than planned.  So every request spreads over all the CTAs it was given, whatever its
// length, and a graph planned for 8,192 keys does not walk a 4,096-key request with half of its CTAs.
__device__ __forceinline__ int piece_len(int kv_len, int num_splits, int split_len, int granule) {
    const int share = ((kv_len + num_splits - 1) / num_splits + granule - 1) / granule * granule;
    return min(split_len, max(share, granule));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block in a fixed order (warp shuffles, then the warp sums by warp 0): the
// result does not depend on timing.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.f;
    if (warp == 0) { t = warp_sum(t); if (lane == 0) scratch[0] = t; }
    __syncthreads();
    return scratch[0];
}

// merges split-KV partial results (attention_simt.cu)
int attn_merge_bf16(const float* ws_o, const float* ws_ml, void* out, int rows, int num_splits, int D, cudaStream_t s);

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// multiprocessors of the current device (asked once per device)
int num_sms();

// Programmatic dependent launch: a kernel launched this way may be scheduled while its predecessor in
// the stream drains; it must call pdl_wait() before it touches anything the predecessor wrote (the
// kernels here call it first thing, so only launch latency and CTA scheduling overlap).  Works inside
// captured graphs.  ttie_set_pdl(0) turns it off.
bool pdl_enabled();
// cluster: CTAs per thread-block cluster along x, y, z (the grid must be a multiple); dim3(1) for none.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, dim3 cluster,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    // (a cluster launch does not take the attribute: as a programmatic dependent it was measured to start late)
    const bool clustered = cluster.x * cluster.y * cluster.z > 1;
    if (pdl_enabled() && !clustered) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (clustered) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x; attr[n].val.clusterDim.y = cluster.y; attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define TTIE_LAUNCH(kernel, grid, block, smem, stream, ...) \
    ::ttie::launch_kernel(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, dim3(1), __VA_ARGS__)
#define TTIE_LAUNCH_CLUSTER(kernel, grid, block, smem, stream, cluster, ...) \
    ::ttie::launch_kernel(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, dim3(cluster), __VA_ARGS__)


}  // namespace ttie
