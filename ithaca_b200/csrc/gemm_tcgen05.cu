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
// Every wait on an mbarrier is bounded: after about a second without progress the waiting
// thread sets the status word to IK_STATUS_GEMM_TIMEOUT, raises the block's abort flag and
// every role leaves its loop; TMEM is freed and the block returns.  Blocks that start after
// the status word is set return at once.  Needs K % 8 == 0 and 16-byte aligned rows (TMA
// strides); the host entry returns IK_UNSUPPORTED otherwise.
#define IK_FAMILY 8
#include "tc_common.cuh"
#include "rope_store.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 128;              // weight rows per tile = TMEM lanes
constexpr int BK = 64;               // 64 bf16 = 128 bytes = one swizzle row
constexpr int THREADS = 192;

template <int BN> struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE) > 8 ? 8 : (200 * 1024 / STAGE);
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;           // TMEM columns of one accumulator
    static constexpr int TMEM_COLS = 2 * ACC_COLS;               // two accumulators: one is drained while the other fills
    static constexpr int SMEM = STAGES * STAGE + 1024 /* alignment slack */ + 256 /* barriers */;
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
    bool sk;
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
        if (sk) {
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

// map_w: [N rows, K] box {64, 128};  map_x: [M rows, K] box {64, BN}.
// out: Y (float or bf16) when partial == nullptr, else partial sums [splits][M][N] float.
//
// Persistent: the grid has at most one block per SM and every block walks the tiles
// t = blockIdx.x, blockIdx.x + gridDim.x, ...  Tiles that share a weight tile are neighbours in
// that order, so they run at the same time on different SMs and the weight tile is fetched from
// HBM once.  The accumulator is double-buffered in TMEM: while the epilogue warps drain tile i,
// the MMA warp already fills the other buffer with tile i + 1.
template <int BN, typename TY>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    TY* __restrict__ Y, float* __restrict__ partial, int M, int N, int K, int ldy, int accumulate,
                    int swiglu, int kb_per_split, int n_splits, int stream_k, int* status, const IkRopeStore rope) {
    typedef Cfg<BN> C;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int rope_rows[4][BN];                   // per epilogue warp: the cache row of each of the tile's tokens
    if (ik_status_has(status, IK_STATUS_GEMM_TIMEOUT)) return;     // an earlier block gave up
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(tiles + C::STAGES * C::STAGE);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;            // [2] accumulator written, ready to be drained
    uint64_t* acc_empty = acc_full + 2;                // [2] accumulator drained, free to be overwritten
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BM - 1) / BM, tiles_m = (M + BN - 1) / BN;
    const int nkb_total = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 128); }
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
    const Walk walk_init(stream_k != 0, tiles_m, tiles_n, nkb_total, kb_per_split, n_splits);
    // Weights are written by no kernel: the first stages' weight tiles are asked for before the wait for the kernel
    // before this one (whose results are the tokens), so a product launched early has them on the way by then.
    int pre_issued = 0;
    if (threadIdx.x == 0) {
        Walk walk = walk_init;
        for (Work w; pre_issued < C::STAGES && walk.next(w);)
            for (int i = 0; i < w.nkb && pre_issued < C::STAGES; i++, pre_issued++) {
                mbar_expect_tx(full + pre_issued, C::STAGE);
                tma_load_2d(tiles + pre_issued * C::STAGE, &map_w, (w.kb0 + i) * BK, w.nt * BM, full + pre_issued);
            }
    }
    ik_pdl_wait();                                     // barriers, TMEM and the first weights are under way while the kernel before finishes
    ik_pdl_launch_dependents();

    float* const slice_sums = stream_k ? nullptr : partial;           // data-parallel K slices: [slice][M][N]
    int* const piece_flags = stream_k ? reinterpret_cast<int*>(partial) : nullptr;                        // [block][4]
    float* const pieces = stream_k ? partial + SK_FLAG_INTS : nullptr;  // stream-K: [block][BN][128] raw sums of a piece

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, armed = 0;
            bool ok = true;
            Walk walk = walk_init;
            for (Work w; ok && walk.next(w);) {
                const int n0 = w.nt * BM, m0 = w.mt * BN, kb0 = w.kb0, nkb = w.nkb;
                for (int i = 0; i < nkb; i++, it++) {
                    const int s = it % C::STAGES;
                    unsigned char* a = tiles + s * C::STAGE;
                    if (it >= pre_issued) {             // the first stages are armed and their weights asked for already
                        if (!mbar_wait(empty + s, ((it / C::STAGES) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 1, it)) { ok = false; break; }
                        mbar_expect_tx(full + s, C::STAGE);
                        tma_load_2d(a, &map_w, (kb0 + i) * BK, n0, full + s);
                    }
                    tma_load_2d(a + C::A_BYTES, &map_x, (kb0 + i) * BK, m0, full + s);
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // leave no copy of this block in flight: wait (bounded) for the stages that were armed last
                for (int i = max(0, armed - C::STAGES); i < armed; i++) {
                    const long long c0 = wait_clock();
                    while (!mbar_test(full + i % C::STAGES, (i / C::STAGES) & 1) && !wait_ran_out(c0, 2000000ull)) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BN);
            int it = 0, lt = 0;
            bool ok = true;
            Walk walk = walk_init;
            for (Work w; ok && walk.next(w); lt++) {
                const int nkb = w.nkb;
                const int buf = lt & 1;
                ok = mbar_wait(acc_empty + buf, ((lt >> 1) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 2, lt);   // drained by the epilogue
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * C::ACC_COLS;
                for (int i = 0; i < nkb; i++, it++) {
                    const int s = it % C::STAGES;
                    ok = mbar_wait(full + s, (it / C::STAGES) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 3, it);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a = smem_u32(tiles + s * C::STAGE), b = a + C::A_BYTES;
                    #pragma unroll
                    for (int j = 0; j < BK / 16; j++)
                        umma(acc, umma_desc(a + j * 32), umma_desc(b + j * 32), idesc, (i | j) != 0);
                    umma_commit(empty + s);             // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        // epilogue: warp w owns TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const bool fused_rope = rope.q_out && !slice_sums;
        int lt = 0;
        Walk walk = walk_init;
        for (Work w; walk.next(w); lt++) {
            const int n0 = w.nt * BM, m0 = w.mt * BN, z = w.z;
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
                for (int i = lane; i < BN; i += 32) rope_rows[quarter][i] = ik_rope_cache_row(rope, m0 + i, M);
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
            if (!mbar_wait(acc_full + buf, (lt >> 1) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 4, lt)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * C::ACC_COLS;
            if (hand_over) {
                float* mine = pieces + (size_t)blockIdx.x * BN * BM + row;
                #pragma unroll 1
                for (int c0 = 0; c0 < BN && m0 + c0 < M; c0 += 16) {
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
                if (c_hi == c_lo) return;
                float p[16], q[16];
                #pragma unroll
                for (int i = 0; i < 16; i++) { p[i] = ahead[0][i]; q[i] = ahead[1][i]; }
                if (c0 + 16 < BN && m0 + c0 + 16 < M) {
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
            #pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
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
                            float y[16];
                            #pragma unroll
                            for (int c = 0; c < 16; c++)
                                y[c] = m0 + c0 + c < M ? ik_ld(Y, (size_t)(m0 + c0 + c) * ldy + feature) : 0.f;
                            #pragma unroll
                            for (int c = 0; c < 16; c++) v[c] += y[c];
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
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
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

template <int BN, typename TY>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, float* partial, int M, int N, int K, int ldy,
           int accumulate, int swiglu, int splits, int* status, const IkRopeStore& rope, cudaStream_t stream) {
    typedef Cfg<BN> C;
    auto kern = gemm_tcgen05_kernel<BN, TY>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    const int nkb = (K + BK - 1) / BK;
    const long long tiles = (long long)((N + BM - 1) / BM) * ((M + BN - 1) / BN);
    if (splits == 0) {                  // stream-K: equal shares of all (tile, K step) units, at least four K steps a block
        const long long units = tiles * nkb;
        const int blocks = (int)(units / 4 < 1 ? 1 : units / 4 < max_blocks() ? units / 4 : max_blocks());
        IK_RETURN_IF_ERROR(ik_launch(kern, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, partial, M, N, K, ldy, accumulate,
                                     swiglu, nkb, 1, 1, status, rope));
        return (int)cudaGetLastError();
    }
    const int per = (nkb + splits - 1) / splits;
    const int n_splits = (nkb + per - 1) / per;
    const long long total = tiles * n_splits;
    const int blocks = (int)(total < max_blocks() ? total : max_blocks());
    IK_RETURN_IF_ERROR(ik_launch(kern, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, n_splits > 1 ? partial : nullptr, M,
                                 N, K, ldy, accumulate, swiglu, per, n_splits, 0, status, rope));
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

// Token-tile width the kernel will use for M tokens.
IK_EXPORT int ik_gemm_tcgen05_tile(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// Scratch of the stream-K mode, in bytes: zeroed once by the caller, then left to the kernels (one stream at a time).
IK_EXPORT int ik_gemm_tcgen05_stream_k_bytes() { return (int)stream_k_bytes(); }

// splits > 1 needs `partial`: splits * M * N floats of scratch owned by the caller.
// splits == 0 is the stream-K mode; `partial` is then the scratch described above.
// status: device int; set to 4 if a block gave up waiting (the result is then not to be used).
// swiglu: W holds (gate j, up j) in rows (2j, 2j + 1); Y is [M, N / 2] = silu(gate) * up.
static int gemm_tcgen05_impl(const void* X, const void* W, void* Y, int y_dtype, float* partial, int M, int N, int K,
                             int ldx, int ldw, int ldy, int accumulate, int swiglu, int splits, int* status,
                             const IkRopeStore& rope, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || (!rope.q_out && ldy < (swiglu ? N / 2 : N)) || splits < 0)
        return IK_BAD_ARGUMENT;
    if (swiglu && ((N & 1) || accumulate)) return IK_BAD_ARGUMENT;
    if (y_dtype != IK_F32 && y_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return IK_UNSUPPORTED;
    if (splits != 1 && !partial) return IK_BAD_ARGUMENT;
    if (M == 0) return IK_OK;
    const int bn = ik_gemm_tcgen05_tile(M);
    CUtensorMap mw, mx;
    int st = ik_make_map(&mw, W, N, K, ldw, BM);
    if (st != IK_OK) return st;
    st = ik_make_map(&mx, X, M, K, ldx, bn);
    if (st != IK_OK) return st;
#define IK_TC(BN_)                                                                                                       \
    return y_dtype == IK_F32 ? launch<BN_, float>(mw, mx, Y, partial, M, N, K, ldy, accumulate, swiglu, splits, status, rope, stream) \
                             : launch<BN_, bf16>(mw, mx, Y, partial, M, N, K, ldy, accumulate, swiglu, splits, status, rope, stream)
    switch (bn) {
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
