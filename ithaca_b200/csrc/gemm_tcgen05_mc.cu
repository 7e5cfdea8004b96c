// The pair mode of the tcgen05 product: the two instructions that make two blocks share one copy of a token tile.
//
// gemm_tcgen05.cu holds the whole kernel and says where a paired copy and a paired commit go; this file gives it the
// two instructions and includes it.  It is a library of its own (built on demand, see gemm_pairs.py): the kernel
// library proper is built without it, and everything runs without it, a little slower at prefill.
//
//   tma_load_2d_pair   a TMA tile copy whose destination is the same shared-memory offset in both blocks of the
//                      cluster, and which counts its bytes on the barrier at the same offset in both;
//   umma_commit_pair   a tcgen05.commit that arrives on the barrier at the same offset in both blocks once the
//                      products issued so far have read their operands.
//
// Both blocks of a pair run on this GPU and the copy reads this GPU's own memory.
#define IK_TCGEN05_PAIRS 1
#define IK_FAMILY 8
#include "tc_common.cuh"

namespace {
constexpr uint16_t BOTH_BLOCKS = 3;       // ranks 0 and 1 of the cluster

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster [%0], [%1, {%3, %4}], [%2], %5;"
        :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "h"(BOTH_BLOCKS) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"(BOTH_BLOCKS) : "memory");
}
}  // namespace

#include "gemm_tcgen05.cu"
