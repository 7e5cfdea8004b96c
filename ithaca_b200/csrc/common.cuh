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
#include <stdlib.h>
#include <utility>

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

// Four consecutive values (16-byte aligned source, 8- or 16-byte aligned destination).
__device__ __forceinline__ void ik_st4(float* p, size_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void ik_st4(__nv_bfloat16* p, size_t i, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p + i) = w;
}

// silu(g) * u with silu(x) = x / (1 + exp(-x)).
__device__ __forceinline__ float ik_swiglu(float g, float u) { return g / (1.0f + expf(-g)) * u; }
// The same with the hardware's approximate exp and reciprocal (relative error ~1e-6), for results that are
// rounded to bfloat16 anyway.
__device__ __forceinline__ float ik_swiglu_fast(float g, float u) { return g * __frcp_rn(1.0f + __expf(-g)) * u; }

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

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the attribute may start before its predecessor in the stream has finished.  The rules
// every kernel of this library keeps:
//   * ik_pdl_wait() returns when every earlier kernel has completed and its writes are visible.  Before it a
//     kernel touches nothing that another kernel writes: only index arithmetic, barrier and TMEM set-up, and, in
//     the bandwidth-bound products, the first batch of WEIGHTS, which no kernel writes.  So a product launched
//     early has its first 128 KB per SM on the way while the kernel before it is still finishing.
//   * ik_pdl_launch_dependents() comes AFTER the kernel's own wait (so at most two kernels are ever on the
//     device: this one and the one after it) and as late as is useful: small kernels call it right after the
//     wait (the product behind a norm starts at once and loads weights while the norm runs); the products and
//     decode attention call it after their main loop (their successor takes the SM slots that their finishing
//     blocks free, and does not compete with blocks that have not started yet).
//   * what the kernel before has written is read with ordinary loads AFTER the wait.  A read-only load
//     (__ldg, or a plain load through a `const __restrict__` pointer) is not enough: the compiler takes it for a
//     read of constant memory and may move it to before the wait.  The skinny product, the one family that is
//     launched early by default, reads its tokens with an explicit ld.global for that reason (with __ldg its
//     results were wrong under graph replay); the element-wise kernels pass their input pointers through
//     IK_AFTER_WAIT.
// IK_PDL=<mask of kernel families> chooses which launches get the attribute (0 = none: kernels start strictly
// one after another and the device-side calls are no-ops).  Default: the products (skinny and tcgen05) and the
// element-wise kernels.  Measured on the graph-replayed decode step of the 8B shape: skinny products 1.1 % faster,
// with the element-wise kernels another 0.5 %, with decode attention 8 % slower (its blocks take SM slots while
// they wait for the queries): attention and sampling stay off.
__device__ __forceinline__ void ik_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void ik_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// After the wait: makes a pointer to what the kernel before wrote opaque to the compiler, so that no load through
// it (not even a read-only one through `const __restrict__`) can be moved to before the wait.
#define IK_AFTER_WAIT(ptr) asm volatile("" : "+l"(ptr))

// The status word: kernels that meet something they refuse to do (an index out of range, a wait that ran out)
// skip the access and set one bit per kind of event, so no cause hides another; the host reads and clears it.
#define IK_STATUS_BAD_TOKEN 1            // a token id outside the vocabulary
#define IK_STATUS_WRITE_NO_PAGE 2        // a cache write without a page
#define IK_STATUS_READ_NO_PAGE 3         // a cache read without a page
#define IK_STATUS_GEMM_TIMEOUT 4         // a tensor-core block that gave up waiting for its data
#define IK_STATUS_SMEM_ALIGN 5           // shared memory not aligned for the tensor-core tiles
#define IK_STATUS_BIT(code) (1 << ((code) - 1))
__device__ __forceinline__ void ik_set_status(int* status, int code) { if (status) atomicOr(status, IK_STATUS_BIT(code)); }
__device__ __forceinline__ bool ik_status_has(const int* status, int code) {
    return status && (*(const volatile int*)status & IK_STATUS_BIT(code)) != 0;
}

// Streaming multiprocessors of the current device (asked once per device).  Grids of persistent kernels, split
// choices and scratch sizes follow it.
static inline int ik_sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

// Kernel families, for IK_PDL=<bit mask>: which launches get the attribute.
#define IK_FAMILY_ELEMENTWISE 1
#define IK_FAMILY_SKINNY 2
#define IK_FAMILY_ATTENTION 4
#define IK_FAMILY_TCGEN05 8
#define IK_FAMILY_SAMPLING 16
#define IK_FAMILY_ATTENTION_MERGE 32     // the kernel that merges the chunks of decode attention
#ifndef IK_FAMILY
#define IK_FAMILY IK_FAMILY_ELEMENTWISE
#endif

static inline int ik_pdl_mask() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("IK_PDL"); v = e ? atoi(e) : (IK_FAMILY_ELEMENTWISE | IK_FAMILY_SKINNY | IK_FAMILY_TCGEN05); }
    return v;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t ik_launch_family(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ik_pdl_mask() & family) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define ik_launch(...) ik_launch_family(IK_FAMILY, __VA_ARGS__)

#define IK_RETURN_IF_ERROR(...)                         \
    do {                                                \
        cudaError_t e__ = (__VA_ARGS__);                \
        if (e__ != cudaSuccess) return (int)e__;        \
    } while (0)
