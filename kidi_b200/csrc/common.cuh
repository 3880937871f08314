// Shared helpers of the kernels: element types, conversions, reductions and the
// integer tables of a step. Every launcher is an extern "C" function that takes raw
// device pointers and a stream, validates what it can on the host, launches, and
// returns the CUDA error code of the launch (0 = success; a negative value means the
// arguments were refused and nothing was launched).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#define KIDI_API extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { KIDI_F32 = 0, KIDI_BF16 = 1, KIDI_NONE = -1 };

// Refusal codes (negative so they cannot collide with cudaError_t).
enum : int { KIDI_REFUSED_DTYPE = -2, KIDI_REFUSED_SIZE = -3 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_float(T value);
template <> __device__ __forceinline__ float to_float<float>(float value) { return value; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 value) { return __bfloat162float(value); }

template <typename T> __device__ __forceinline__ T from_float(float value);
template <> __device__ __forceinline__ float from_float<float>(float value) { return value; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float value) { return __float2bfloat16_rn(value); }

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
    return value;
}

// Sum over a block of THREADS threads (a multiple of 32, at most 1024). Every thread
// gets the result. The order of additions depends only on THREADS.
template <int THREADS> __device__ __forceinline__ float block_sum(float value, float* scratch /* [32] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    value = warp_sum(value);
    __syncthreads();
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int index = 0; index < THREADS / 32; ++index) total += scratch[index];
    return total;
}

// Where the keys and values of a cached token live. A sequence's pages are found
// through its row of the block table; a windowed group keeps a ring of `ring_pages`
// pages. Storage of one schedule entry: [pages, kv_heads, page_size, head_dim].
struct CacheGeometry {
    const int* table;   // [slots, pages_per_seq]
    int pages_per_seq;
    int page_shift;     // log2(page_size)
    int ring_pages;     // 0: every page of the sequence is kept
    int kv_heads;
    int head_dim;
};

__device__ __forceinline__ long long cache_row_offset(const CacheGeometry& g, int slot, int position, int kv_head) {
    int page_index = position >> g.page_shift;
    if (g.ring_pages) page_index %= g.ring_pages;
    const int page = g.table[(long long)slot * g.pages_per_seq + page_index];
    const int within = position & ((1 << g.page_shift) - 1);
    return ((((long long)page * g.kv_heads + kv_head) << g.page_shift) + within) * g.head_dim;
}

static inline int kidi_launch_status() { return (int)cudaGetLastError(); }

__device__ __forceinline__ void prefetch_l2(const void* pointer) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(pointer));
}

template <typename... Expected, typename... Actual>
static inline int kidi_launch(void (*kernel)(Expected...), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                              Actual&&... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, static_cast<Expected>(arguments)...);
    return status != cudaSuccess ? (int)status : (int)cudaGetLastError();
}

// The same with the blocks along x grouped into thread-block clusters of `cluster_x`
// (the grid's x extent must be a multiple of it; at most 8).
template <typename... Expected, typename... Actual>
static inline int kidi_launch_clusters(void (*kernel)(Expected...), dim3 grid, dim3 block, size_t shared,
                                       cudaStream_t stream, unsigned cluster_x, Actual&&... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster_x;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, static_cast<Expected>(arguments)...);
    return status != cudaSuccess ? (int)status : (int)cudaGetLastError();
}
