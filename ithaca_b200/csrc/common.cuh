// Shared declarations of the kernel library: storage types, loads and stores
// that convert to and from float, and the status codes the entry points return.
//
// Every entry point is extern "C", takes raw device pointers and a stream, checks
// its arguments on the host, launches, and returns 0 or a negative status / a
// positive cudaError_t.  Nothing here allocates device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IK_OK 0
#define IK_BAD_ARGUMENT (-1)
#define IK_UNSUPPORTED (-2)

#define IK_F32 0
#define IK_BF16 1

#define IK_EXPORT extern "C" __attribute__((visibility("default")))

#define IK_LAUNCH_STATUS()                         \
    do {                                           \
        cudaError_t e__ = cudaGetLastError();      \
        return e__ == cudaSuccess ? IK_OK : (int)e__; \
    } while (0)

__device__ __forceinline__ float ik_ld(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ik_ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void ik_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void ik_st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Value a float would have after a round trip through the storage type.
template <typename T> __device__ __forceinline__ float ik_round_to(float v);
template <> __device__ __forceinline__ float ik_round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float ik_round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Block-wide sum / max with a fixed order: lanes by shuffle, warps in index order.
// Every thread of the block must call; the result is returned to all threads.
template <int THREADS>
__device__ __forceinline__ float ik_block_sum(float v, float* scratch /* >= 32 floats */) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    #pragma unroll
    for (int w = 0; w < THREADS / 32; w++) t += scratch[w];
    return t;
}

template <int THREADS>
__device__ __forceinline__ float ik_block_max(float v, float* scratch) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = scratch[0];
    #pragma unroll
    for (int w = 1; w < THREADS / 32; w++) t = fmaxf(t, scratch[w]);
    return t;
}
