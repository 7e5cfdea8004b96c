// Inline-PTX helpers of the kernels that use the fifth-generation tensor cores: mbarriers with bounded
// waits, TMA tile loads, shared-memory and instruction descriptors, tcgen05.mma / commit / ld / st, and
// the host-side encoder of TMA tensor maps.
#pragma once
#include <cuda.h>
#include "common.cuh"


namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity to complete.  Gives up after `limit_ns` (about a second unless the
// caller says otherwise), or as soon as another thread of the block has given up, and returns false; the thread
// that gives up first raises the block's abort flag and records the event in the status word.
// The limit is counted in cycles of this SM's own clock (two per nanosecond asked for: at the clocks this part
// runs at, between 1x and 2x the time asked for).  %globaltimer is not used for it: that counter is kept in step
// with the host's clock from outside and may move by more than it ran.
constexpr unsigned long long IK_WAIT_LIMIT_NS = 1000000000ull;
__device__ __forceinline__ long long wait_clock() { return clock64(); }
__device__ __forceinline__ bool wait_ran_out(long long c0, unsigned long long limit_ns) {
    return (unsigned long long)(clock64() - c0) > 2ull * limit_ns;
}

// Where the first wait of this module gave up: [0] the wait's site number (0 = none yet), [1] the block's linear
// index, [2] a number the site chose (a loop count), [3] the parity it waited for.  The host reads and clears it
// when the status word says that a wait ran out.
__device__ int ik_wait_record[4];
__device__ __forceinline__ void note_wait_gave_up(int site, int info, int parity) {
    if (atomicCAS(&ik_wait_record[0], 0, site) == 0) {
        ik_wait_record[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        ik_wait_record[2] = info;
        ik_wait_record[3] = parity;
    }
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          unsigned long long limit_ns = IK_WAIT_LIMIT_NS, int site = 99, int info = 0) {
    if (mbar_test(bar, parity)) return true;
    const long long c0 = wait_clock();
    for (int spin = 0;; spin++) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 63) == 63) {
            if (*abort_flag) return false;
            if (wait_ran_out(c0, limit_ns)) {
                note_wait_gave_up(site, info, (int)parity);
                *abort_flag = 1;
                ik_set_status(status, IK_STATUS_GEMM_TIMEOUT);
                return false;
            }
        }
    }
}

// Distributed shared memory: the address of `local` (an address in this block's shared memory) in the block of
// rank `rank` of the cluster; stores and barrier arrivals there.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {        // releases this thread's earlier stores to the cluster
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(addr) : "memory");
}
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, uint32_t parity) {   // acquires what other blocks released
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor: rows of 128 bytes under the 128-byte swizzle (version 1 = sm_100).
// K-major tile (K contiguous): groups of 8 rows 1024 bytes apart (stride offset); the leading offset is unused.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused under swizzle) = 1
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// MN-major tile (the M or N index contiguous: a row of shared memory is one k with 64 consecutive n): blocks of
// 64 n lie `lead_bytes` apart (leading offset), groups of 8 k lie 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lead_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lead_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: D float, A and B bfloat16, A K-major, M = 128, N = n; B K-major, or MN-major
// (its N index contiguous in shared memory) when b_mn_major is set.
__device__ __forceinline__ uint32_t umma_idesc(int n, int b_mn_major = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(b_mn_major & 1) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same from descriptor halves: every descriptor of a kernel has the same upper word (umma_desc_hi), and the lower
// word is the start address in 16-byte units beside a constant (umma_desc_lo), so stepping through a stage or from
// stage to stage is one 32-bit addition for the thread that issues.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t umma_desc_hi() { return (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ void umma_halves(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        :: "r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory: row i of A in lane i, two bfloat16 per 32-bit cell (k even in the
// low half), so the 16 k of one instruction are 8 consecutive cells from `tmem_a`.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :: "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
// 16 consecutive columns of this thread's TMEM lane, written from registers.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        :: "r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
           "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
           "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
           "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
           "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tmem_st16_bits(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
           "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The same load without the wait: several may be issued back to back, then tmem_ld_wait() once.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    #pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ik_ex2(float x) {            // 2^x, hardware approximation; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {     // one instruction on sm_100
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Two floats per instruction (sm_100): (d0, d1) = (a0, a1) * b + c, and (d0, d1) += (a0, a1).
__device__ __forceinline__ void fma_f32x2(float& d0, float& d1, float a0, float a1, float b, float c) {
    uint64_t a, bb, cc, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bb) : "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(bb), "l"(cc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
__device__ __forceinline__ void add_f32x2(float& d0, float& d1, float a0, float a1) {
    uint64_t a, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(d0), "f"(d1));
    asm("add.rn.f32x2 %0, %0, %1;" : "+l"(d) : "l"(a));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}


typedef CUresult (*IkEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Copies the record of the first wait that gave up to the host and clears it on the device.
inline int ik_take_wait_record(int* out4) {
    int zero[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpyFromSymbol(out4, ik_wait_record, sizeof(zero));
    if (e != cudaSuccess) return (int)e;
    e = cudaMemcpyToSymbol(ik_wait_record, zero, sizeof(zero));
    return e == cudaSuccess ? IK_OK : (int)e;
}

inline IkEncodeTiled ik_encode_fn() {
    static IkEncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (IkEncodeTiled)p;
    }
    return fn;
}

// rows x cols bfloat16 matrix, cols contiguous, row stride ld elements; box = 64 x box_rows, 128-byte swizzle,
// zero fill outside.
inline int ik_make_map(CUtensorMap* map, const void* base, unsigned long long rows, int cols, unsigned long long ld,
                       int box_rows) {
    IkEncodeTiled enc = ik_encode_fn();
    if (!enc) return IK_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IK_OK : IK_BAD_ARGUMENT;
}

}  // namespace
