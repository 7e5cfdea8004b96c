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
                    int swiglu, int kb_per_split, int n_splits, int* status, const IkRopeStore rope) {
    typedef Cfg<BN> C;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int rope_rows[4][BN];                   // per epilogue warp: the cache row of each of the tile's tokens
    ik_pdl_launch_dependents();
    if (status && *(volatile int*)status == IK_STATUS_GEMM_TIMEOUT) return;     // an earlier block gave up
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(tiles + C::STAGES * C::STAGE);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;            // [2] accumulator written, ready to be drained
    uint64_t* acc_empty = acc_full + 2;                // [2] accumulator drained, free to be overwritten
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BM - 1) / BM, tiles_m = (M + BN - 1) / BN;
    const int total_tiles = tiles_n * tiles_m * n_splits;
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
    ik_pdl_wait();

    // tile t -> (K slice z, weight tile nt, token tile mt), token tile fastest
    #define IK_TILE_COORDS(t)                                                   \
        const int mt = (t) % tiles_m, nt = ((t) / tiles_m) % tiles_n, z = (t) / (tiles_m * tiles_n); \
        const int n0 = nt * BM, m0 = mt * BN, kb0 = z * kb_per_split;           \
        const int nkb = min(kb_per_split, nkb_total - kb0);

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, armed = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                IK_TILE_COORDS(t)
                (void)z;
                for (int i = 0; i < nkb; i++, it++) {
                    const int s = it % C::STAGES;
                    if (!mbar_wait(empty + s, ((it / C::STAGES) & 1) ^ 1, abort_flag, status)) { ok = false; break; }
                    unsigned char* a = tiles + s * C::STAGE;
                    mbar_expect_tx(full + s, C::STAGE);
                    tma_load_2d(a, &map_w, (kb0 + i) * BK, n0, full + s);
                    tma_load_2d(a + C::A_BYTES, &map_x, (kb0 + i) * BK, m0, full + s);
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // leave no copy of this block in flight: wait (bounded) for the stages that were armed last
                for (int i = max(0, armed - C::STAGES); i < armed; i++) {
                    const unsigned long long t0 = globaltimer();
                    while (!mbar_test(full + i % C::STAGES, (i / C::STAGES) & 1) && globaltimer() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BN);
            int it = 0, lt = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, lt++) {
                IK_TILE_COORDS(t)
                (void)z; (void)n0; (void)m0; (void)kb0;
                const int buf = lt & 1;
                ok = mbar_wait(acc_empty + buf, ((lt >> 1) & 1) ^ 1, abort_flag, status);   // drained by the epilogue
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * C::ACC_COLS;
                for (int i = 0; i < nkb; i++, it++) {
                    const int s = it % C::STAGES;
                    ok = mbar_wait(full + s, (it / C::STAGES) & 1, abort_flag, status);
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
        const bool fused_rope = rope.q_out && !partial;
        int lt = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, lt++) {
            IK_TILE_COORDS(t)
            (void)kb0; (void)nkb;
            const int buf = lt & 1;
            const int feature = n0 + quarter * 32 + lane;
            if (fused_rope) {
                // each warp keeps its own list of the tile's cache rows (no barrier between warps is needed); the
                // lookups run while the accumulator is still being filled
                __syncwarp();
                for (int i = lane; i < BN; i += 32) rope_rows[quarter][i] = ik_rope_cache_row(rope, m0 + i, M);
                __syncwarp();
            }
            if (!mbar_wait(acc_full + buf, (lt >> 1) & 1, abort_flag, status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * C::ACC_COLS;
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
                                    ? __ldg(cs_base + (size_t)(m0 + col0 + c) * (rope.hd >> 1)) : make_float2(1.f, 0.f);
                    tmem_ld16(acc + c0, v);
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
                tmem_ld16(acc + c0, v);
                if (feature < N || (swiglu && !partial)) {     // N is even under swiglu: a pair is in or out together
                    if (partial) {
                        #pragma unroll
                        for (int c = 0; c < 16; c++)
                            if (m0 + c0 + c < M) partial[((size_t)z * M + m0 + c0 + c) * N + feature] = v[c];
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
        }
    }
    #undef IK_TILE_COORDS
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
    ik_pdl_launch_dependents();
    ik_pdl_wait();
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
    const int per = (nkb + splits - 1) / splits;
    const int n_splits = (nkb + per - 1) / per;
    const long long total = (long long)((N + BM - 1) / BM) * ((M + BN - 1) / BN) * n_splits;
    const int blocks = (int)(total < 148 ? total : 148);
    IK_RETURN_IF_ERROR(ik_launch(kern, blocks, THREADS, C::SMEM, stream, mw, mx, (TY*)Y, n_splits > 1 ? partial : nullptr, M,
                                 N, K, ldy, accumulate, swiglu, per, n_splits, status, rope));
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        const size_t elems = (size_t)M * N;
        const int rblocks = (int)((elems + 255) / 256 < 148 * 8 ? (elems + 255) / 256 : 148 * 8);
        IK_RETURN_IF_ERROR(ik_launch(splitk_reduce_kernel<TY>, rblocks, 256, 0, stream, partial, (TY*)Y, M, N, ldy, n_splits, accumulate, swiglu, rope));
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return IK_OK;
}

}  // namespace

// Token-tile width the kernel will use for M tokens.
IK_EXPORT int ik_gemm_tcgen05_tile(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// splits > 1 needs `partial`: splits * M * N floats of scratch owned by the caller.
// status: device int; set to 4 if a block gave up waiting (the result is then not to be used).
// swiglu: W holds (gate j, up j) in rows (2j, 2j + 1); Y is [M, N / 2] = silu(gate) * up.
static int gemm_tcgen05_impl(const void* X, const void* W, void* Y, int y_dtype, float* partial, int M, int N, int K,
                             int ldx, int ldw, int ldy, int accumulate, int swiglu, int splits, int* status,
                             const IkRopeStore& rope, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || (!rope.q_out && ldy < (swiglu ? N / 2 : N)) || splits < 1)
        return IK_BAD_ARGUMENT;
    if (swiglu && ((N & 1) || accumulate)) return IK_BAD_ARGUMENT;
    if (y_dtype != IK_F32 && y_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return IK_UNSUPPORTED;
    if (splits > 1 && !partial) return IK_BAD_ARGUMENT;
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
