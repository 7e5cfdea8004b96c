// bfloat16 product on the fifth-generation tensor cores of sm_100a:
//   Y[M, N] (+)= X[M, K] * W[N, K]^T,  X and W bfloat16 with K contiguous, float accumulation in TMEM.
//
// The weight matrix is the 128-row operand (one TMEM lane per output feature) and the tokens
// are the N-operand (one TMEM column per token, BN = 32 .. 256 of them per block), for prefill
// and decode alike: the epilogue then writes, for each token, 32 consecutive features per warp
// instruction (coalesced), and a handful of decode tokens wastes no tensor work.
//
// A block computes 128 x BN tiles (optionally one slice of K each), one after another:
//   warp 0      one lane issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//               128 x 64 weight tile and the BN x 64 token tile of each K step into a ring of
//               shared-memory stages; completion is counted on the stage's "full" mbarrier.
//   warp 1      allocates TMEM (two accumulators); one lane issues four tcgen05.mma (K = 16 each)
//               per stage and commits them to the stage's "empty" mbarrier; after a tile's last
//               stage it commits to that accumulator's "full" mbarrier.  Frees TMEM at the end.
//   warps 2..5  read a full accumulator with tcgen05.ld (each warp its 32 lanes), store it, and
//               hand it back ("empty") while the MMA warp is already filling the other one.
// Tails in M, N and K are zero-filled by TMA and masked in the epilogue.  No multicast, no
// clusters.
//
// How the work is shared out.  Data-parallel: the items (K slice, weight tile, token tile) are dealt round
// robin; with K slices a second kernel adds the slices.  Stream-K: all (tile, K step) units are laid end to
// end and every block takes an equal contiguous share, so that all SMs stream the same number of bytes
// whatever the number of tiles.  A block whose share begins in the middle of a tile computes that piece
// FIRST and hands the raw sums to the block that holds the tile's first K step (a scratch slot of its own,
// then a flag); that block computes its own piece LAST, adds the others' pieces in ascending K order and
// runs the epilogue.  A block thus only ever waits for blocks with a higher index that produced their piece
// at the very start of their run, so the wait is short, cannot be circular, and the result does not depend on
// timing.  The wait is bounded like the mbarrier waits.  Flags are cleared by their reader.
//
// Few tiles (a small matrix and few tokens): a cluster of 2 to 4 blocks shares one tile, each block taking a slice
// of K.  The blocks of ranks 1.. write their raw sums into the shared memory of the block of rank 0 (distributed
// shared memory) and arrive on a barrier there; rank 0 adds them to its own in rank order and runs the epilogue.
// No partial sums go through global memory and no second kernel runs.
//
// Many tiles (prefill): pairs of blocks (clusters of 2) can take two weight tiles that meet the same token tile and
// load that token tile once between them: each block fetches half of its rows and the copy lands in both blocks'
// shared memory.  A stage may then be refilled only when both blocks' products have read it, so the "empty" barriers
// count two arrivals and each block's commit arrives on both.  This file only says where the paired copy and the
// paired commit go; the two instructions live in gemm_tcgen05_mc.cu, which includes this file, and without that
// file the library is built and runs without the mode.
//
// Every wait on an mbarrier is bounded: after about a second without progress the waiting
// thread sets the status word to IK_STATUS_GEMM_TIMEOUT, raises the block's abort flag and
// every role leaves its loop; TMEM is freed and the block returns.  Blocks that start after
// the status word is set return at once.  Needs K % 8 == 0 and 16-byte aligned rows (TMA
// strides); the host entry returns IK_UNSUPPORTED otherwise.
#ifndef IK_FAMILY
#define IK_FAMILY 8
#endif
#include "tc_common.cuh"
#include "rope_store.cuh"

#ifndef IK_TCGEN05_PAIRS
namespace {
// Stand-ins of the two paired instructions for the build without them (the pair mode is then never launched).
__device__ __forceinline__ void tma_load_2d_pair(void*, const CUtensorMap*, int, int, uint64_t*) {}
__device__ __forceinline__ void umma_commit_pair(uint64_t*) {}
}  // namespace
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 128;              // weight rows per tile = TMEM lanes
constexpr int BK = 64;               // 64 bf16 = 128 bytes = one swizzle row
constexpr int THREADS = 192;

template <int BN> struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE) > 8 ? 8 : (200 * 1024 / STAGE);
    static constexpr int STAGES2 = 200 * 1024 / (2 * STAGE);    // stages that hold two K blocks each (MODE 3)
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;           // TMEM columns of one accumulator
    static constexpr int TMEM_COLS = 2 * ACC_COLS;               // two accumulators: one is drained while the other fills
    static constexpr int SMEM = STAGES * STAGE + 1024 /* alignment slack */ + 256 /* barriers */;
    // cluster mode: room for the other ranks' sums ([rank - 1][BN][128] floats) beside a shorter ring of stages
    static constexpr int RED_SLOTS = BN <= 64 ? 3 : (BN <= 128 ? 1 : 0);
    static constexpr int RED_BYTES = RED_SLOTS * BN * BM * 4;
    static constexpr int CL_ROOM = 232448 - 1024 - 256 - 4 * BN * 4 /* static */ - RED_BYTES;
    static constexpr int CL_STAGES = CL_ROOM / STAGE > 8 ? 8 : CL_ROOM / STAGE;
    static constexpr int CL_SMEM = CL_STAGES * STAGE + RED_BYTES + 1024 + 256;
};

// Persistent: one block per SM of the device.  Stream-K scratch: a flag per block and epilogue warp (room for 1024
// blocks), then a [256][128] piece of raw sums per block.
constexpr int SK_MAX_BLOCKS = 1024;
constexpr size_t SK_FLAG_INTS = (size_t)SK_MAX_BLOCKS * 4;
inline int max_blocks() { const int n = ik_sm_count(); return n < SK_MAX_BLOCKS ? n : SK_MAX_BLOCKS; }
inline size_t stream_k_bytes() { return SK_FLAG_INTS * 4 + (size_t)max_blocks() * 256 * BM * 4; }

// One accumulator's worth of work: K steps [kb0, kb0 + nkb) of output tile (nt, mt).
struct Work {
    int tile, mt, nt, z, kb0, nkb;
    bool first, last;                 // holds the tile's first / last K step
};

// The sequence of Work of one block.  Every role of the block walks it on its own.
struct Walk {
    bool sk, cl = false, cl_done = false;   // cl: one piece of work per block: tile blockIdx.x / n_splits, K slice = rank in the cluster
    bool pairs = false;                     // pairs: block 2c + r takes weight tile 2 * (item / tiles_m) + r of the items c, c + grid / 2, ...
    int tiles_m, tiles_n, nkb_total, kb_per_split;
    int item, n_items;                // data-parallel: items blockIdx.x, + gridDim.x, ...; item -> (K slice, weight tile, token tile)
    long long u, u_end, n_units;      // stream-K: this block's share [u, u_end) of all (tile, K step) units, token tile fastest
    __device__ Walk(bool sk_, int tm, int tn, int nkb, int per, int n_splits)
        : sk(sk_), tiles_m(tm), tiles_n(tn), nkb_total(nkb), kb_per_split(per), item(blockIdx.x), n_items(tm * tn * n_splits),
          n_units((long long)tm * tn * nkb) {
        u = share_begin(blockIdx.x);
        u_end = share_begin(blockIdx.x + 1);
    }
    __device__ long long share_begin(int block) const { return n_units * block / gridDim.x; }
    __device__ bool next(Work& w) {
        if (pairs) {
            if (item >= (tiles_n + 1) / 2 * tiles_m) return false;
            w.mt = item % tiles_m;
            w.nt = 2 * (item / tiles_m) + (int)(blockIdx.x & 1);     // may lie past the last weight tile: all zeros, nothing stored
            w.tile = w.nt * tiles_m + w.mt;
            w.z = 0; w.kb0 = 0; w.nkb = nkb_total;
            w.first = w.last = true;
            item += gridDim.x / 2;
            return true;
        }
        if (cl) {
            if (cl_done) return false;
            cl_done = true;
            const int n_splits = n_items / (tiles_m * tiles_n);
            w.tile = blockIdx.x / n_splits;
            w.z = blockIdx.x % n_splits;
            w.kb0 = w.z * kb_per_split;
            w.nkb = min(kb_per_split, nkb_total - w.kb0);
        } else if (sk) {
            if (u >= u_end) return false;
            w.tile = (int)(u / nkb_total);
            w.kb0 = (int)(u - (long long)w.tile * nkb_total);
            const long long left = u_end - u;
            w.nkb = left < nkb_total - w.kb0 ? (int)left : nkb_total - w.kb0;
            w.z = 0;
            u += w.nkb;
        } else {
            if (item >= n_items) return false;
            w.tile = item % (tiles_m * tiles_n);
            w.z = item / (tiles_m * tiles_n);
            w.kb0 = w.z * kb_per_split;
            w.nkb = min(kb_per_split, nkb_total - w.kb0);
            item += gridDim.x;
        }
        w.mt = w.tile % tiles_m;
        w.nt = w.tile / tiles_m;
        w.first = w.kb0 == 0;
        w.last = w.kb0 + w.nkb == nkb_total;
        return true;
    }
};

// The rotary table can be the result of the kernel right before this one.  A volatile asm keeps its place after the
// wait for that kernel; a read-only load (__ldg) is one the compiler may move.
__device__ __forceinline__ float2 ld_cos_sin(const float2* p) {
    float2 v;
    asm volatile("ld.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}

// Waits until *flag is set by another block (acquire).  Bounded like mbar_wait.
__device__ __forceinline__ bool flag_wait(const int* flag, volatile int* abort_flag, int* status,
                                          unsigned long long limit_ns = IK_WAIT_LIMIT_NS) {
    const long long c0 = wait_clock();
    for (int spin = 0;; spin++) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v) return true;
        if ((spin & 63) == 63) {
            if (*abort_flag) return false;
            if (wait_ran_out(c0, limit_ns)) {
                note_wait_gave_up(5, (int)(flag - (const int*)nullptr) & 0xFFFF, 0);
                *abort_flag = 1;
                ik_set_status(status, IK_STATUS_GEMM_TIMEOUT);
                return false;
            }
        }
    }
}

// Built with -DIK_TIMELINE, the product stamps the nanosecond clock at the stations of a block's life (for the first
// 1024 blocks of the launch): 0 entry, 1 barriers and TMEM set up, 2 the kernel before has finished, 3 the first
// stage has landed, 4 the last product is issued, 5 the block's last accumulator is complete, 6 its epilogue is done,
// 7 the block leaves.  ik_gemm_tcgen05_timeline copies the stamps out.  Not compiled otherwise.
#ifdef IK_TIMELINE
__device__ unsigned long long ik_timeline[1024][8];
#define IK_STAMP(i) do { if (blockIdx.x < 1024) ik_timeline[blockIdx.x][i] = globaltimer(); } while (0)
#else
#define IK_STAMP(i) do { } while (0)
#endif

// map_w: [N rows, K] box {64, 128};  map_x: [M rows, K] box {64, BN}.
// out: Y (float or bf16) when partial == nullptr, else partial sums [splits][M][N] float.
//
// Persistent: the grid has at most one block per SM and every block walks the tiles
// t = blockIdx.x, blockIdx.x + gridDim.x, ...  Tiles that share a weight tile are neighbours in
// that order, so they run at the same time on different SMs and the weight tile is fetched from
// HBM once.  The accumulator is double-buffered in TMEM: while the epilogue warps drain tile i,
// the MMA warp already fills the other buffer with tile i + 1.
// MODE 1 (CL): the cluster mode described at the top (n_splits blocks per tile, partial == nullptr, one piece of work
// per block).  MODE 2 (PAIRS): pairs of blocks share the token tile's copy (whole tiles only; map_x's box is half a tile).
// MODE 3: as MODE 0 with two K blocks (128 k) per stage, for token tiles up to 128 wide.  Measured with one thread issuing
// back to back in a kernel that does nothing else (ik_gemm_tcgen05_issue_rate below): a product instruction costs the
// issuing thread about 75 cycles and a commit about 190, whatever the tile's width, while the tensor core needs 32 / 64 /
// 128 cycles for 64 / 128 / 256 tokens.  At 256 tokens four products and a commit per K block just keep up (about 490
// against 512 cycles); below that the issuing thread would be the bound, and eight products per commit make it cheaper.  (Two issuing threads, each with an accumulator of its own,
// issue twice as fast in that kernel, but did not speed up this one: with stages this large only three or four are in
// flight, and what a block can take in, 192 KB per load latency, is the bound that is left.)
// A stage holds [W block 0][W block 1][X block 0][X block 1].
template <int BN, typename TY, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    TY* __restrict__ Y, float* __restrict__ partial, int M, int N, int K, int ldy, int accumulate,
                    int swiglu, int kb_per_split, int n_splits, int stream_k, int* status, const IkRopeStore rope, int bn) {
    // bn <= BN: the width of a token tile in use (a multiple of 16): tiles lie bn tokens apart, bn rows of tokens are
    // loaded per stage and the products are bn columns wide; BN is the room a stage and an accumulator have.
    typedef Cfg<BN> C;
    constexpr bool CL = MODE == 1, PAIRS = MODE == 2;
    constexpr int KSUB = MODE == 3 ? 2 : 1;            // K blocks of 64 per stage
    extern __shared__ unsigned char smem_raw[];
    __shared__ int rope_rows[4][BN];                   // per epilogue warp: the cache row of each of the tile's tokens
    if (threadIdx.x == 0) IK_STAMP(0);
    // (in cluster mode every block goes on to the cluster's barrier below; its waits are bounded all the same)
    if (!CL && !PAIRS && ik_status_has(status, IK_STATUS_GEMM_TIMEOUT)) return;     // an earlier block gave up
    constexpr int NST = CL ? C::CL_STAGES : KSUB == 2 ? C::STAGES2 : C::STAGES;
    constexpr int STAGE = KSUB * C::STAGE;             // bytes from one stage to the next
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* const red = (float*)(tiles + NST * STAGE);                     // cluster mode: [rank - 1][BN][128] sums of the other ranks
    uint64_t* full = (uint64_t*)(tiles + NST * STAGE + (CL ? C::RED_BYTES : 0));
    uint64_t* empty = full + NST;
    uint64_t* acc_full = empty + NST;                  // [2] accumulator written, ready to be drained
    uint64_t* acc_empty = acc_full + 2;                // [2] accumulator drained, free to be overwritten
    uint64_t* red_full = acc_empty + 2;                // cluster mode, rank 0: the other ranks' sums have arrived
    uint32_t* tmem_slot = (uint32_t*)(red_full + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BM - 1) / BM, tiles_m = (M + bn - 1) / bn;
    const int block_bytes = C::A_BYTES + bn * BK * 2;  // what one K block brings: 128 weight rows and bn token rows of 64 k
    const int nkb_total = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full + s, 1); mbar_init(empty + s, PAIRS ? 2 : 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 128); }
        mbar_init(red_full, CL ? (n_splits - 1) * 128 : 1);         // one arrival per epilogue thread of every other rank
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (CL || PAIRS) cluster_sync();                   // every block's barriers exist before another block arrives on them
    Walk walk_first(stream_k != 0, tiles_m, tiles_n, nkb_total, kb_per_split, n_splits);
    walk_first.cl = CL;
    walk_first.pairs = PAIRS;
    if (PAIRS) walk_first.item = blockIdx.x / 2;
    const Walk walk_init = walk_first;
    // Weights are written by no kernel: the first stages' weight tiles are asked for before the wait for the kernel
    // before this one (whose results are the tokens), so a product launched early has them on the way by then.
    int pre_issued = 0;
    if (threadIdx.x == 0) {
        Walk walk = walk_init;
        for (Work w; pre_issued < NST && walk.next(w);)
            for (int i = 0; i < w.nkb && pre_issued < NST; i += KSUB, pre_issued++) {
                const int n_sub = min(KSUB, w.nkb - i);
                mbar_expect_tx(full + pre_issued, n_sub * block_bytes);
                for (int sub = 0; sub < n_sub; sub++)
                    tma_load_2d(tiles + pre_issued * STAGE + sub * C::A_BYTES, &map_w, (w.kb0 + i + sub) * BK, w.nt * BM, full + pre_issued);
            }
    }
    if (threadIdx.x == 0) IK_STAMP(1);
    ik_pdl_wait();                                     // barriers, TMEM and the first weights are under way while the kernel before finishes
    ik_pdl_launch_dependents();
    if (threadIdx.x == 0) IK_STAMP(2);

    float* const slice_sums = stream_k ? nullptr : partial;           // data-parallel K slices: [slice][M][N]
    int* const piece_flags = stream_k ? reinterpret_cast<int*>(partial) : nullptr;                        // [block][4]
    float* const pieces = stream_k ? partial + SK_FLAG_INTS : nullptr;  // stream-K: [block][BN][128] raw sums of a piece

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, armed = 0;
            bool ok = true;
            Walk walk = walk_init;
            for (Work w; ok && walk.next(w);) {
                const int n0 = w.nt * BM, m0 = w.mt * bn, kb0 = w.kb0, nkb = w.nkb;
                for (int i = 0; i < nkb; i += KSUB, it++) {
                    const int s = it % NST, n_sub = min(KSUB, nkb - i);
                    unsigned char* a = tiles + s * STAGE;
                    if (it >= pre_issued) {             // the first stages are armed and their weights asked for already
                        if (!mbar_wait(empty + s, ((it / NST) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 1, it)) { ok = false; break; }
                        mbar_expect_tx(full + s, n_sub * block_bytes);
                        for (int sub = 0; sub < n_sub; sub++)
                            tma_load_2d(a + sub * C::A_BYTES, &map_w, (kb0 + i + sub) * BK, n0, full + s);
                    }
                    if (PAIRS) {
                        // this block's half of the token tile's rows, into both blocks of the pair
                        const int half = bn / 2, r = (int)(blockIdx.x & 1);
                        tma_load_2d_pair(a + C::A_BYTES + r * half * (BK * 2), &map_x, (kb0 + i) * BK, m0 + r * half, full + s);
                    } else {
                        for (int sub = 0; sub < n_sub; sub++)
                            tma_load_2d(a + KSUB * C::A_BYTES + sub * C::B_BYTES, &map_x, (kb0 + i + sub) * BK, m0, full + s);
                    }
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // leave no copy of this block in flight: wait (bounded) for the stages that were armed last
                for (int i = max(0, armed - NST); i < armed; i++) {
                    const long long c0 = wait_clock();
                    while (!mbar_test(full + i % NST, (i / NST) & 1) && !wait_ran_out(c0, 2000000ull)) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // With the loads compiled out, a K block of four products and a commit takes this thread 0.27-0.3 us whether
            // the token tile is 64, 128 or 256 wide (see MODE 3 above), so what it does besides is kept short: stage and
            // phase are counted, not divided, and the descriptors are one addition away.
            const uint32_t idesc = umma_idesc(bn), desc_hi = umma_desc_hi(), a_lo0 = umma_desc_lo(smem_u32(tiles));
            int it = 0, lt = 0, s = 0;                     // s = it % NST, phase = (it / NST) & 1
            uint32_t phase = 0;
            bool ok = true;
            Walk walk = walk_init;
            for (Work w; ok && walk.next(w); lt++) {
                const int nkb = w.nkb;
                const int buf = lt & 1;
                ok = mbar_wait(acc_empty + buf, ((lt >> 1) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 2, lt);   // drained by the epilogue
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * C::ACC_COLS;
                for (int i = 0; i < nkb; i += KSUB, it++, s = s + 1 == NST ? 0 : s + 1, phase ^= (uint32_t)(s == 0)) {
                    ok = mbar_wait(full + s, phase, abort_flag, status, IK_WAIT_LIMIT_NS, 3, it);
                    if (!ok) break;
                    if (it == 0) IK_STAMP(3);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * (STAGE >> 4), b_lo = a_lo + ((KSUB * C::A_BYTES) >> 4);
                    #pragma unroll
                    for (int sub = 0; sub < KSUB; sub++) {
                        if (sub > 0 && i + sub >= nkb) break;      // an odd number of K blocks: the last stage holds one
                        #pragma unroll
                        for (int j = 0; j < BK / 16; j++)          // 16 k = 32 bytes = 2 units of the descriptor's address
                            umma_halves(acc, a_lo + sub * (C::A_BYTES >> 4) + 2 * j, b_lo + sub * (C::B_BYTES >> 4) + 2 * j, desc_hi,
                                        idesc, (i | sub | j) != 0);
                    }
                    if (PAIRS) umma_commit_pair(empty + s);    // ... in both blocks, whose copies fill each other's stages
                    else umma_commit(empty + s);             // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full + buf);
                IK_STAMP(4);
            }
        }
    } else {
        // epilogue: warp w owns TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const bool fused_rope = rope.q_out && !slice_sums;
        int lt = 0;
        Walk walk = walk_init;
        for (Work w; walk.next(w); lt++) {
            const int n0 = w.nt * BM, m0 = w.mt * bn, z = w.z;
            const int buf = lt & 1;
            // stream-K: a piece that does not hold the tile's first K step is handed over raw; the piece that does
            // hold it gathers the pieces of the blocks after this one, [c_lo, c_hi)
            const bool hand_over = stream_k && !w.first;
            int c_lo = 0, c_hi = 0;
            if (stream_k && w.first && !w.last) {
                const long long tile_end = (long long)(w.tile + 1) * nkb_total;
                c_lo = c_hi = blockIdx.x + 1;
                while (c_hi < (int)gridDim.x && walk.share_begin(c_hi) < tile_end) c_hi++;
            }
            const int feature = n0 + quarter * 32 + lane;
            if (fused_rope) {
                // each warp keeps its own list of the tile's cache rows (no barrier between warps is needed); the
                // lookups run while the accumulator is still being filled
                __syncwarp();
                for (int i = lane; i < bn; i += 32) rope_rows[quarter][i] = ik_rope_cache_row(rope, m0 + i, M);
                __syncwarp();
            }
            const int row = quarter * 32 + lane;
            // the other blocks' pieces of this tile: waited for first (they were computed at the very start of those
            // blocks' runs), and the first two are fetched one 16-column chunk ahead of their use
            bool gathered = true;
            for (int c = c_lo; c < c_hi && gathered; c++) gathered = flag_wait(piece_flags + c * 4 + quarter, abort_flag, status);
            if (!gathered) break;
            float ahead[2][16];
            auto fetch_piece = [&](int c, int c0, float (&p)[16]) {
                const float* theirs = pieces + ((size_t)c * BN + c0) * BM + row;
                #pragma unroll
                for (int i = 0; i < 16; i++) p[i] = c < c_hi && m0 + c0 + i < M ? __ldcg(theirs + (size_t)i * BM) : 0.f;
            };
            if (c_hi > c_lo) {
                fetch_piece(c_lo, 0, ahead[0]);
                fetch_piece(c_lo + 1, 0, ahead[1]);
            }
            // Adding into Y: what Y holds was written by earlier kernels, so the first 16 columns of it are asked for
            // before the accumulator is waited for, and each further 16 while the 16 before them are being added.
            const bool adds_to_y = accumulate && !slice_sums && !swiglu && !fused_rope && !hand_over && !(CL && z > 0);
            float y_ahead[16];
            auto load_y = [&](int c0) {
                #pragma unroll
                for (int c = 0; c < 16; c++)
                    y_ahead[c] = (feature < N && m0 + c0 + c < M) ? ik_ld(Y, (size_t)(m0 + c0 + c) * ldy + feature) : 0.f;
            };
            if (adds_to_y) load_y(0);
            if (!mbar_wait(acc_full + buf, (lt >> 1) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 4, lt)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * C::ACC_COLS;
            if (threadIdx.x == 64) IK_STAMP(5);
            if (CL && z > 0) {
                // cluster mode, not rank 0: this lane's row of raw sums goes into rank 0's shared memory, then this
                // thread's arrival on rank 0's barrier releases what it stored
                const uint32_t theirs = cluster_addr(smem_u32(red + ((size_t)(z - 1) * BN) * BM + row), 0);
                #pragma unroll 1
                for (int c0 = 0; c0 < bn && m0 + c0 < M; c0 += 16) {
                    float v[16];
                    tmem_ld16(acc + c0, v);
                    #pragma unroll
                    for (int c = 0; c < 16; c++) st_cluster_f32(theirs + (uint32_t)(c0 + c) * BM * 4, v[c]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(acc_empty + buf);
                mbar_arrive_cluster(cluster_addr(smem_u32(red_full), 0));
                continue;
            }
            if (CL && n_splits > 1) {
                // rank 0: the other ranks' sums (waited for with the same bound as everything else)
                const long long c0 = wait_clock();
                bool there = mbar_test_cluster(red_full, 0);
                for (int spin = 0; !there; spin++) {
                    there = mbar_test_cluster(red_full, 0);
                    if (!there && (spin & 63) == 63) {
                        if (*abort_flag) break;
                        if (wait_ran_out(c0, IK_WAIT_LIMIT_NS)) {
                            note_wait_gave_up(6, lt, 0);
                            *abort_flag = 1;
                            ik_set_status(status, IK_STATUS_GEMM_TIMEOUT);
                            break;
                        }
                    }
                }
                if (!there) break;
            }
            if (hand_over) {
                float* mine = pieces + (size_t)blockIdx.x * BN * BM + row;
                #pragma unroll 1
                for (int c0 = 0; c0 < bn && m0 + c0 < M; c0 += 16) {
                    float v[16];
                    tmem_ld16(acc + c0, v);
                    #pragma unroll
                    for (int c = 0; c < 16; c++)
                        if (m0 + c0 + c < M) mine[(size_t)(c0 + c) * BM] = v[c];
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(acc_empty + buf);
                __threadfence();                         // this lane's sums are visible before the flag is
                __syncwarp();
                if (lane == 0)
                    asm volatile("st.release.gpu.global.s32 [%0], %1;" :: "l"(piece_flags + blockIdx.x * 4 + quarter), "r"(1) : "memory");
                continue;
            }
            // the accumulator's columns c0 .. c0 + 15 of this lane's row, with the other blocks' pieces added in K order
            auto read_sums = [&](int c0, float (&v)[16]) {
                tmem_ld16(acc + c0, v);
                if (CL) {                                // the other ranks' sums of these columns, added in rank order
                    for (int r = 0; r + 1 < n_splits; r++) {
                        const float* p = red + ((size_t)r * BN + c0) * BM + row;
                        #pragma unroll
                        for (int i = 0; i < 16; i++) v[i] += p[(size_t)i * BM];
                    }
                    return;
                }
                if (c_hi == c_lo) return;
                float p[16], q[16];
                #pragma unroll
                for (int i = 0; i < 16; i++) { p[i] = ahead[0][i]; q[i] = ahead[1][i]; }
                if (c0 + 16 < bn && m0 + c0 + 16 < M) {
                    fetch_piece(c_lo, c0 + 16, ahead[0]);
                    fetch_piece(c_lo + 1, c0 + 16, ahead[1]);
                }
                #pragma unroll
                for (int i = 0; i < 16; i++) v[i] = (v[i] + p[i]) + q[i];
                for (int c = c_lo + 2; c < c_hi; c += 2) {
                    fetch_piece(c, c0, p);
                    fetch_piece(c + 1, c0, q);
                    #pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = (v[i] + p[i]) + q[i];
                }
            };
            // what the rotary epilogue needs of this lane's feature pair: fixed for the whole tile
            const int f0 = feature & ~1;
            const int head = fused_rope ? f0 / rope.hd : 0, r0 = fused_rope ? f0 - head * rope.hd : 0;
            const bool is_q = head < rope.nh, rotated = head < rope.nh + rope.nkv;
            bf16* const kv_base = (rotated ? rope.k_pages : rope.v_pages) +
                                  (size_t)(head - rope.nh - (rotated ? 0 : rope.nkv)) * rope.page_size * rope.hd + r0;
            const float2* const cs_base = reinterpret_cast<const float2*>(rope.cos_sin) + (r0 >> 1);
            // The plain epilogue (whole sums of this block, to Y or added to Y): 32 columns a turn, both halves of the
            // accumulator asked for before either is waited for.
            if (!fused_rope && !swiglu && !slice_sums && !CL && c_hi == c_lo) {
                #pragma unroll 1
                for (int c0 = 0; c0 < bn && m0 + c0 < M; c0 += 32) {
                    float v[32];
                    const bool second = c0 + 16 < bn && m0 + c0 + 16 < M;
                    tmem_ld16_issue(acc + c0, v);
                    if (second) tmem_ld16_issue(acc + c0 + 16, v + 16);
                    tmem_ld_wait();
                    if (feature < N) {
                        #pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (h == 1 && !second) break;
                            if (accumulate) {
                                #pragma unroll
                                for (int c = 0; c < 16; c++) v[16 * h + c] += y_ahead[c];
                                if (c0 + 16 * h + 16 < bn && m0 + c0 + 16 * h + 16 < M) load_y(c0 + 16 * h + 16);
                            }
                            #pragma unroll
                            for (int c = 0; c < 16; c++)
                                if (m0 + c0 + 16 * h + c < M) ik_st(Y, (size_t)(m0 + c0 + 16 * h + c) * ldy + feature, v[16 * h + c]);
                        }
                    }
                }
            } else
            #pragma unroll 1
            for (int c0 = 0; c0 < bn; c0 += 16) {
                if (m0 + c0 >= M) break;
                float v[16];
                if (fused_rope) {
                    // lanes (2j, 2j + 1) hold a rotary pair (or two neighbouring values of a v head).  The pair shares
                    // the work: the even lane takes columns 0..7, the odd lane columns 8..15.  All cosines and sines
                    // are fetched before the accumulator is read and before any store, so that they are in flight
                    // together (a store could alias them as far as the compiler knows).
                    const bool odd = lane & 1;
                    const int col0 = c0 + (odd ? 8 : 0);
                    float2 cs[8];
                    #pragma unroll
                    for (int c = 0; c < 8; c++)
                        cs[c] = rotated && feature < N && m0 + col0 + c < M
                                    ? ld_cos_sin(cs_base + (size_t)(m0 + col0 + c) * (rope.hd >> 1)) : make_float2(1.f, 0.f);
                    read_sums(c0, v);
                    __nv_bfloat162 packed[8];
                    #pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const float other = __shfl_xor_sync(0xffffffffu, odd ? v[c] : v[c + 8], 1);
                        const float a = odd ? other : v[c], b = odd ? v[c + 8] : other;
                        packed[c] = __floats2bfloat162_rn(a * cs[c].x - b * cs[c].y, a * cs[c].y + b * cs[c].x);
                    }
                    if (feature < N) {
                        if (is_q) {
                            #pragma unroll
                            for (int c = 0; c < 8; c++)
                                if (m0 + col0 + c < M)
                                    *reinterpret_cast<__nv_bfloat162*>(rope.q_out + (size_t)(m0 + col0 + c) * rope.nh * rope.hd + f0) = packed[c];
                        } else {
                            int rows[8];
                            #pragma unroll
                            for (int c = 0; c < 8; c++) rows[c] = rope_rows[quarter][col0 + c];
                            #pragma unroll
                            for (int c = 0; c < 8; c++)
                                if (rows[c] >= 0) *reinterpret_cast<__nv_bfloat162*>(kv_base + (size_t)rows[c] * rope.hd) = packed[c];
                        }
                    }
                    continue;
                }
                read_sums(c0, v);
                if (feature < N || (swiglu && !slice_sums)) {     // N is even under swiglu: a pair is in or out together
                    if (slice_sums) {
                        #pragma unroll
                        for (int c = 0; c < 16; c++)
                            if (m0 + c0 + c < M) slice_sums[((size_t)z * M + m0 + c0 + c) * N + feature] = v[c];
                    } else if (swiglu) {
                        // lanes (2j, 2j + 1) hold gate j and up j.  The pair shares the work: the even lane takes
                        // columns 0..7 (it gets the up values from its neighbour), the odd lane columns 8..15.
                        const bool odd = lane & 1;
                        #pragma unroll
                        for (int c = 0; c < 8; c++) {
                            const float other = __shfl_xor_sync(0xffffffffu, odd ? v[c] : v[c + 8], 1);
                            const float gte = odd ? other : v[c], up = odd ? v[c + 8] : other;
                            const int m = m0 + c0 + c + (odd ? 8 : 0);
                            if (feature < N && m < M) ik_st(Y, (size_t)m * ldy + (feature >> 1), ik_swiglu_fast(gte, up));
                        }
                    } else {
                        if (accumulate) {
                            #pragma unroll
                            for (int c = 0; c < 16; c++) v[c] += y_ahead[c];
                            if (c0 + 16 < bn && m0 + c0 + 16 < M) load_y(c0 + 16);
                        }
                        #pragma unroll
                        for (int c = 0; c < 16; c++)
                            if (m0 + c0 + c < M) ik_st(Y, (size_t)(m0 + c0 + c) * ldy + feature, v[c]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty + buf);               // 128 arrivals: this accumulator may be overwritten
            if (c_hi > c_lo) {                          // the pieces are used up: their flags go back to zero for the next launch
                __syncwarp();
                if (lane == 0)
                    for (int c = c_lo; c < c_hi; c++) piece_flags[c * 4 + quarter] = 0;
            }
        }
    }
    if (threadIdx.x == 64) IK_STAMP(6);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0) IK_STAMP(7);
    // no block of a cluster leaves while another may still store into its shared memory or arrive on its barrier
    if (CL || PAIRS) cluster_sync();
}

// Adds the K slices in slice order and writes Y.
template <typename TY>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TY* __restrict__ Y, int M, int N, int ldy,
                                     int splits, int accumulate, int swiglu, const IkRopeStore rope) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    asm volatile("" : "+l"(partial));      // the slices are the kernel before's results: no read of them may move above the wait
    const size_t total = (size_t)M * N;
    if (rope.q_out) {                   // columns (2j, 2j + 1) are rotary pairs: rotate and store to q_out and the cache
        const size_t half = (size_t)M * (N / 2);
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < half; idx += (size_t)gridDim.x * blockDim.x) {
            const size_t m = idx / (N / 2), j = idx - m * (N / 2);
            float a = 0.f, b = 0.f;
            for (int z = 0; z < splits; z++) {
                a += partial[(size_t)z * total + m * N + 2 * j];
                b += partial[(size_t)z * total + m * N + 2 * j + 1];
            }
            ik_rope_store_pair(rope, (int)m, (int)(2 * j), a, b);
        }
        return;
    }
    if (swiglu) {                       // columns (2j, 2j + 1) are gate j and up j; Y is [M, N / 2]
        const size_t half = (size_t)M * (N / 2);
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < half; idx += (size_t)gridDim.x * blockDim.x) {
            const size_t m = idx / (N / 2), j = idx - m * (N / 2);
            float g = 0.f, u = 0.f;
            for (int z = 0; z < splits; z++) {
                g += partial[(size_t)z * total + m * N + 2 * j];
                u += partial[(size_t)z * total + m * N + 2 * j + 1];
            }
            ik_st(Y, m * ldy + j, ik_swiglu(g, u));
        }
        return;
    }
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += partial[(size_t)z * total + idx];
        const size_t m = idx / N, n = idx - m * N;
        const size_t o = m * ldy + n;
        if (accumulate) s += ik_ld(Y, o);
        ik_st(Y, o, s);
    }
}

// Cluster mode: n_cl blocks per tile, each a slice of K, summed in rank 0's shared memory.
template <int BN, typename TY>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, int M, int N, int K, int ldy, int accumulate,
                   int swiglu, int n_cl, int* status, const IkRopeStore& rope, int bn, cudaStream_t stream) {
    typedef Cfg<BN> C;
    if (C::RED_SLOTS == 0) return IK_UNSUPPORTED;
    const int nkb = (K + BK - 1) / BK;
    const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    const int per = (nkb + n_cl - 1) / n_cl;
    if (n_cl < 2 || n_cl > C::RED_SLOTS + 1 || (long long)(n_cl - 1) * per >= nkb || tiles * n_cl > max_blocks()) return IK_UNSUPPORTED;
    auto kern = gemm_tcgen05_kernel<BN, TY, 1>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::CL_SMEM);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * n_cl));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::CL_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = n_cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ik_pdl_mask() & IK_FAMILY) ? 2 : 1;
    IK_RETURN_IF_ERROR(cudaLaunchKernelEx(&cfg, kern, mw, mx, (TY*)Y, (float*)nullptr, M, N, K, ldy, accumulate, swiglu, per, n_cl, 0,
                                          status, rope, bn));
    return (int)cudaGetLastError();
}

template <int BN, typename TY>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, float* partial, int M, int N, int K, int ldy,
           int accumulate, int swiglu, int splits, int* status, const IkRopeStore& rope, int bn, cudaStream_t stream) {
    typedef Cfg<BN> C;
    if (splits < 0) return launch_cluster<BN, TY>(mw, mx, Y, M, N, K, ldy, accumulate, swiglu, -splits, status, rope, bn, stream);
    auto kern = gemm_tcgen05_kernel<BN, TY, 0>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    const int nkb = (K + BK - 1) / BK;
    const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    if (splits == 0) {                  // stream-K: equal shares of all (tile, K step) units, at least four K steps a block
        const long long units = tiles * nkb;
        const int blocks = (int)(units / 4 < 1 ? 1 : units / 4 < max_blocks() ? units / 4 : max_blocks());
        IK_RETURN_IF_ERROR(ik_launch(kern, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, partial, M, N, K, ldy, accumulate,
                                     swiglu, nkb, 1, 1, status, rope, bn));
        return (int)cudaGetLastError();
    }
    const int per = (nkb + splits - 1) / splits;
    const int n_splits = (nkb + per - 1) / per;
    const long long total = tiles * n_splits;
    const int blocks = (int)(total < max_blocks() ? total : max_blocks());
    if (n_splits == 1 && BN <= 128 && M > 128) {
        // whole narrow tiles of a product with several token tiles (compute-bound, few weight tiles): two K blocks a stage
        auto kern2 = gemm_tcgen05_kernel<BN <= 128 ? BN : 128, TY, 3>;
        e = cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        IK_RETURN_IF_ERROR(ik_launch(kern2, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, (float*)nullptr, M, N, K, ldy, accumulate,
                                     swiglu, per, 1, 0, status, rope, bn));
        return (int)cudaGetLastError();
    }
    IK_RETURN_IF_ERROR(ik_launch(kern, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, n_splits > 1 ? partial : nullptr, M,
                                 N, K, ldy, accumulate, swiglu, per, n_splits, 0, status, rope, bn));
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        const size_t elems = (size_t)M * N;
        const size_t rcap = (size_t)ik_sm_count() * 8;
        const int rblocks = (int)((elems + 255) / 256 < rcap ? (elems + 255) / 256 : rcap);
        IK_RETURN_IF_ERROR(ik_launch(splitk_reduce_kernel<TY>, rblocks, 256, 0, stream, partial, (TY*)Y, M, N, ldy, n_splits, accumulate, swiglu, rope));
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return IK_OK;
}

}  // namespace

// The room a token tile of that width has (the kernel's variant): 32, 64, 128 or 256 tokens.
IK_EXPORT int ik_gemm_tcgen05_tile(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// The width of token tile in use for M tokens and N output features: a multiple of 16.  Up to 128 tokens: the tokens
// rounded up (one token tile; few tiles fill the SMs by slicing K).  Beyond: of the widths from 64 to 256, the one whose
// tiles need the fewest rounds of the persistent grid, a tile costing nearly the same whatever its width (the tensor
// core is busy for a K step's four instructions just as long with 64 tokens as with 256; loads and epilogue grow
// with the width): 512 tokens and 4,096 features are 64 tiles of 256, which leave more than half of the SMs idle, or
// 128 tiles of 128, in one round either way; 2,048 tokens are 256 tiles of 256 or 288 of 240, two rounds either way.
IK_EXPORT int ik_gemm_tcgen05_tile_width(int M, int N) {
    if (M <= 128) return M <= 16 ? 16 : (M + 15) / 16 * 16;
    const long long tiles_n = (N + BM - 1) / BM, sms = max_blocks();
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 64; bn -= 16) {
        const long long rounds = (tiles_n * ((M + bn - 1) / bn) + sms - 1) / sms;
        const long long cost = rounds * (1024 + bn);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

#ifdef IK_TCGEN05_PAIRS
// ------------------------------------------------------------------------------------------
// The pair mode (this build only): whole tiles, more than 256 tokens, two blocks to a token tile's copy.
namespace {
template <typename TY>
int launch_pairs(const CUtensorMap& mw, const CUtensorMap& mx_half, void* Y, int M, int N, int K, int ldy, int accumulate,
                 int swiglu, int* status, const IkRopeStore& rope, int bn, cudaStream_t stream) {
    typedef Cfg<256> C;
    auto kern = gemm_tcgen05_kernel<256, TY, 2>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    const int nkb = (K + BK - 1) / BK;
    const long long items = (long long)(((N + BM - 1) / BM + 1) / 2) * ((M + bn - 1) / bn);
    const long long clusters = items < max_blocks() / 2 ? items : max_blocks() / 2;
    if (clusters < 1) return IK_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ik_pdl_mask() & IK_FAMILY) ? 2 : 1;
    IK_RETURN_IF_ERROR(cudaLaunchKernelEx(&cfg, kern, mw, mx_half, (TY*)Y, (float*)nullptr, M, N, K, ldy, accumulate, swiglu, nkb, 1, 0,
                                          status, rope, bn));
    return (int)cudaGetLastError();
}

int pairs_impl(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int ldx, int ldw, int ldy,
               int accumulate, int swiglu, int* status, const IkRopeStore& rope, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || (!rope.q_out && ldy < (swiglu ? N / 2 : N))) return IK_BAD_ARGUMENT;
    if (swiglu && ((N & 1) || accumulate)) return IK_BAD_ARGUMENT;
    if (y_dtype != IK_F32 && y_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return IK_UNSUPPORTED;
    if (M <= 256) return IK_UNSUPPORTED;                 // fewer tokens are bound by the weights' bytes: nothing to share
    const int bn = ik_gemm_tcgen05_tile_width(M, N);
    if (bn <= 128) return IK_UNSUPPORTED;                // narrow tiles (few weight tiles to fill the SMs with): the variant with their room
    CUtensorMap mw, mx;
    int st = ik_make_map(&mw, W, N, K, ldw, BM);
    if (st != IK_OK) return st;
    st = ik_make_map(&mx, X, M, K, ldx, bn / 2);         // a block copies half of a token tile's rows
    if (st != IK_OK) return st;
    return y_dtype == IK_F32 ? launch_pairs<float>(mw, mx, Y, M, N, K, ldy, accumulate, swiglu, status, rope, bn, stream)
                             : launch_pairs<bf16>(mw, mx, Y, M, N, K, ldy, accumulate, swiglu, status, rope, bn, stream);
}
}  // namespace

// Arguments as ik_gemm_tcgen05 without the scratch and the way of sharing out; IK_UNSUPPORTED up to 256 tokens.
IK_EXPORT int ik_gemm_tcgen05_pairs(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int ldx, int ldw,
                                    int ldy, int accumulate, int swiglu, int* status, cudaStream_t stream) {
    IkRopeStore none = {};
    return pairs_impl(X, W, Y, y_dtype, M, N, K, ldx, ldw, ldy, accumulate, swiglu, status, none, stream);
}

IK_EXPORT int ik_gemm_qkv_rope_tcgen05_pairs(const void* X, const void* W, int M, int N, int K, int ldx, int ldw, int* status,
                                             const IkRopeStore* rope, cudaStream_t stream) {
    if (!rope || !rope->q_out || (rope->hd & 1) || N != (rope->nh + 2 * rope->nkv) * rope->hd) return IK_BAD_ARGUMENT;
    return pairs_impl(X, W, nullptr, IK_F32, M, N, K, ldx, ldw, N, 0, 0, status, *rope, stream);
}
#else
// Scratch of the stream-K mode, in bytes: zeroed once by the caller, then left to the kernels (one stream at a time).
IK_EXPORT int ik_gemm_tcgen05_stream_k_bytes() { return (int)stream_k_bytes(); }

// splits > 1 needs `partial`: splits * M * N floats of scratch owned by the caller.
// splits == 0 is the stream-K mode; `partial` is then the scratch described above.
// splits < 0 is the cluster mode with -splits blocks per tile (2 to 4 for up to 64 tokens, 2 for up to 128); it needs
// no scratch, and returns IK_UNSUPPORTED where it does not apply (more tokens, more tiles than SMs, too few K steps).
// status: device int; set to 4 if a block gave up waiting (the result is then not to be used).
// swiglu: W holds (gate j, up j) in rows (2j, 2j + 1); Y is [M, N / 2] = silu(gate) * up.
static int gemm_tcgen05_impl(const void* X, const void* W, void* Y, int y_dtype, float* partial, int M, int N, int K,
                             int ldx, int ldw, int ldy, int accumulate, int swiglu, int splits, int* status,
                             const IkRopeStore& rope, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || (!rope.q_out && ldy < (swiglu ? N / 2 : N)))
        return IK_BAD_ARGUMENT;
    if (swiglu && ((N & 1) || accumulate)) return IK_BAD_ARGUMENT;
    if (y_dtype != IK_F32 && y_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return IK_UNSUPPORTED;
    if (splits != 1 && splits >= 0 && !partial) return IK_BAD_ARGUMENT;
    if (M == 0) return IK_OK;
    if (splits < 0 && M > 128) return IK_UNSUPPORTED;     // the cluster mode is for one token tile of at most 128 tokens
    const int bn = ik_gemm_tcgen05_tile_width(M, N), room = ik_gemm_tcgen05_tile(bn);
    CUtensorMap mw, mx;
    int st = ik_make_map(&mw, W, N, K, ldw, BM);
    if (st != IK_OK) return st;
    st = ik_make_map(&mx, X, M, K, ldx, bn);
    if (st != IK_OK) return st;
#define IK_TC(BN_)                                                                                                       \
    return y_dtype == IK_F32 ? launch<BN_, float>(mw, mx, Y, partial, M, N, K, ldy, accumulate, swiglu, splits, status, rope, bn, stream) \
                             : launch<BN_, bf16>(mw, mx, Y, partial, M, N, K, ldy, accumulate, swiglu, splits, status, rope, bn, stream)
    switch (room) {
        case 32: IK_TC(32);
        case 64: IK_TC(64);
        case 128: IK_TC(128);
        default: IK_TC(256);
    }
#undef IK_TC
}

IK_EXPORT int ik_gemm_tcgen05(const void* X, const void* W, void* Y, int y_dtype, float* partial, int M, int N, int K,
                              int ldx, int ldw, int ldy, int accumulate, int swiglu, int splits, int* status,
                              cudaStream_t stream) {
    IkRopeStore none = {};
    return gemm_tcgen05_impl(X, W, Y, y_dtype, partial, M, N, K, ldx, ldw, ldy, accumulate, swiglu, splits, status, none, stream);
}

// The fused q/k/v product with the rotary / cache epilogue (rope_store.cuh).  N must be (nh + 2 nkv) * hd, hd even.
IK_EXPORT int ik_gemm_qkv_rope_tcgen05(const void* X, const void* W, float* partial, int M, int N, int K, int ldx, int ldw,
                                       int splits, int* status, const IkRopeStore* rope, cudaStream_t stream) {
    if (!rope || !rope->q_out || (rope->hd & 1) || N != (rope->nh + 2 * rope->nkv) * rope->hd) return IK_BAD_ARGUMENT;
    return gemm_tcgen05_impl(X, W, nullptr, IK_F32, partial, M, N, K, ldx, ldw, N, 0, 0, splits, status, *rope, stream);
}

// ------------------------------------------------------------------------------------------
// Self-test of the bounded waits: a wait that nothing will ever satisfy must give up after its limit, record
// the event, raise the block's abort flag and let the kernel return; other waiting threads of the block must
// then leave at once.  One block; thread 0 waits on an mbarrier nobody arrives at, thread 32 (after it) on the
// same barrier with a long limit, thread 64 on a global flag that stays zero.
// result: [0] thread 0's wait returned true?  [1] abort flag afterwards  [2] microseconds thread 0 waited
//         [3] thread 32's wait returned true?  [4] microseconds it waited  [5] the flag wait returned true?
namespace {
__global__ void wait_expiry_kernel(int* status, int* result, const int* never_set, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = globaltimer();
        result[0] = mbar_wait(&bar, 0, &abort_flag, status, limit_ns) ? 1 : 0;
        result[2] = (int)((globaltimer() - t0) / 1000);
        result[1] = abort_flag;
    }
    __syncthreads();
    if (threadIdx.x == 32) {
        const unsigned long long t0 = globaltimer();
        result[3] = mbar_wait(&bar, 0, &abort_flag, status, 200 * limit_ns) ? 1 : 0;
        result[4] = (int)((globaltimer() - t0) / 1000);
    }
    if (threadIdx.x == 64) {
        volatile int own_abort = 0;
        result[5] = flag_wait(never_set, &own_abort, nullptr, limit_ns) ? 1 : 0;
    }
}
}  // namespace

// ------------------------------------------------------------------------------------------
// What issuing costs: `issuers` threads (1 or 2, in warps of their own) each issue `rounds` x `per_commit` product
// instructions (128 rows, 16 k, n tokens) back to back into an accumulator of their own, with a commit to a barrier of
// its own after every `per_commit`, over shared memory that holds ones; nothing is loaded meanwhile.
// out[0] = cycles of this SM's clock until the slowest thread's last commit has completed, out[1] = 1 if all waits ended.
namespace {
constexpr int RATE_ROUNDS = 64;
__global__ void __launch_bounds__(128, 1) issue_rate_kernel(int n, int per_commit, int issuers, long long* out, int* status) {
    extern __shared__ __align__(1024) unsigned char rate_smem[];
    __shared__ uint64_t bars[2 * RATE_ROUNDS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ long long cycles[2];
    __shared__ int fine[2];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)rate_smem + 1023) & ~(uintptr_t)1023);
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) ((uint32_t*)tiles)[i] = 0x3f803f80u;      // bfloat16 ones
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * RATE_ROUNDS; i++) mbar_init(bars + i, 1);
        abort_flag = 0; cycles[0] = cycles[1] = 0; fine[0] = fine[1] = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the ones above are read by the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    if ((threadIdx.x & 31) == 0 && (int)(threadIdx.x >> 5) < issuers) {
        const int me = threadIdx.x >> 5;
        const uint32_t idesc = umma_idesc(n), a0 = smem_u32(tiles), b0 = a0 + 64 * 1024;
        const long long t0 = clock64();
        for (int r = 0; r < RATE_ROUNDS; r++) {
            for (int u = 0; u < per_commit; u++) {
                const uint32_t off = (uint32_t)((u & 3) * 32 + ((u >> 2) & 3) * 16384);       // other k, other K block
                umma(tmem + me * 256, umma_desc(a0 + off), umma_desc(b0 + off), idesc, 1);
            }
            umma_commit(bars + me * RATE_ROUNDS + r);       // each barrier is used once
        }
        fine[me] = mbar_wait(bars + me * RATE_ROUNDS + RATE_ROUNDS - 1, 0, &abort_flag, status, 100000000ull) ? 1 : 0;   // commits complete in order
        cycles[me] = clock64() - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) { out[0] = cycles[0] > cycles[1] ? cycles[0] : cycles[1]; out[1] = fine[0] && fine[1]; }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512u) : "memory");
    }
}
}  // namespace

// Cycles per product instruction of one issuing thread (and, with two, of both together: divide by two) for token
// tiles n wide; see issue_rate_kernel.  n: a multiple of 16 up to 256; per_commit 1..16; issuers 1 or 2.
IK_EXPORT int ik_gemm_tcgen05_issue_rate(int n, int per_commit, int issuers, long long* out2, int* status, cudaStream_t stream) {
    if (n < 16 || n > 256 || n % 16 || per_commit < 1 || per_commit > 16 || issuers < 1 || issuers > 2 || !out2) return IK_BAD_ARGUMENT;
    cudaError_t e = cudaFuncSetAttribute(issue_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    issue_rate_kernel<<<1, 128, 200 * 1024, stream>>>(n, per_commit, issuers, out2, status);
    IK_LAUNCH_STATUS();
}

// Sites of the product's waits: 1 = loader for a free stage, 2 = MMA issuer for a drained accumulator, 3 = MMA issuer
// for a loaded stage, 4 = epilogue for a finished accumulator, 5 = stream-K gather for another block's piece; 99 = self-test.
IK_EXPORT int ik_gemm_tcgen05_take_wait_record(int* out4) { return ik_take_wait_record(out4); }

// limit_ns is capped at 10 ms: the test is meant to run out quickly.
IK_EXPORT int ik_selftest_wait_expires(int* status, int* result, const int* never_set, unsigned long long limit_ns,
                                       cudaStream_t stream) {
    if (!result || !never_set || limit_ns == 0 || limit_ns > 10000000ull) return IK_BAD_ARGUMENT;
    wait_expiry_kernel<<<1, 96, 0, stream>>>(status, result, never_set, limit_ns);
    IK_LAUNCH_STATUS();
}

#ifdef IK_TIMELINE
IK_EXPORT int ik_gemm_tcgen05_timeline(unsigned long long* out /* [1024][8] */) {
    cudaError_t e = cudaMemcpyFromSymbol(out, ik_timeline, sizeof(unsigned long long) * 1024 * 8);
    if (e != cudaSuccess) return (int)e;
    static unsigned long long zeros[1024 * 8];
    e = cudaMemcpyToSymbol(ik_timeline, zeros, sizeof(zeros));
    return e == cudaSuccess ? IK_OK : (int)e;
}
#endif
#endif  // IK_TCGEN05_PAIRS
