// bfloat16 products on the warp-level tensor-core path (mma.sync m16n8k16, float accumulate):
//   Y[M, N] (+)= X[M, K] * W[N, K]^T,  X and W bfloat16 with rows contiguous, Y float or bfloat16.
//
// Two kernels.
//  * skinny (M <= 64, decode): weights are the 16-row operand, tokens the 8-column operand, so a
//    handful of tokens costs no wasted tensor work.  A block owns 16 weight rows; its 8
//    warps split K between them and their partial sums are added in warp order at the end.
//    Each thread streams 16 contiguous bytes of a weight row per load, straight from global
//    memory to registers: weights are read exactly once.
//  * tiled (any M, prefill): 128 x 128 x 32 tiles through shared memory with a 4-stage
//    cp.async pipeline.
//
// Both feed the MMA without ldmatrix: a thread's 16 bytes (8 consecutive k) serve as the
// fragments of two MMAs, with the same permutation of k applied to both operands (a dot
// product does not care in which order its terms are paired, as long as both sides agree).
//
// The order in which a result's K terms are added depends on K alone (and on which of the
// two kernels runs), never on M or N.  Needs K % 8 == 0 and 16-byte aligned rows; the entry
// points return IK_UNSUPPORTED otherwise and the caller uses the CUDA-core product.
#define IK_FAMILY 2
#include "common.cuh"
#include "rope_store.cuh"

namespace {

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {      // read-once data: do not keep it in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The tokens: written by the kernel before this one.  Not a read-only (ld.global.nc / __ldg) load: the compiler
// may move such a load, which it takes for a read of constant memory, to before the wait for that kernel.
__device__ __forceinline__ uint4 ld_tokens(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void store_out(float* Y, size_t o, float v, int accumulate) {
    Y[o] = accumulate ? Y[o] + v : v;
}
__device__ __forceinline__ void store_out(__nv_bfloat16* Y, size_t o, float v, int accumulate) {
    Y[o] = __float2bfloat16_rn(accumulate ? __bfloat162float(Y[o]) + v : v);
}

// ------------------------------------------------------------------------------------------ skinny
// NT: 8-token column tiles (M <= 8 NT).  A block owns 16 weight rows; each of its 8 warps takes
// every 8th group of U 64-wide K blocks, loads all of the group's weights (16 bytes per thread
// per load, 4 U loads in flight per thread) and tokens, then multiplies.  U trades registers
// (blocks per SM) for bytes in flight; the host picks it per shape.  R = 8: a block owns 8 weight rows (the other half
// of the 16-row MMA operand is zero and never loaded): twice the blocks for a matrix with so few rows that blocks of 16
// would leave half the SMs' slots empty.
template <int NT, int U, typename TY, int R>
__global__ void __launch_bounds__(256)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, TY* __restrict__ Y,
                   int M, int N, int K, int ldx, int ldw, int ldy, int accumulate, int swiglu, const IkRopeStore rope) {
    constexpr int COLS = 8 * NT, H = R / 8;
    static_assert(R == 8 || R == 16, "a block owns 8 or 16 weight rows");
    extern __shared__ float red[];                       // [8 warps][R][COLS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * R;

    float acc[NT][4];
    #pragma unroll
    for (int n = 0; n < NT; n++)
        #pragma unroll
        for (int i = 0; i < 4; i++) acc[n][i] = 0.f;

    const __nv_bfloat16* wrow[H];
    bool wok[H];
    #pragma unroll
    for (int h = 0; h < H; h++) {
        const int row = n0 + h * 8 + g;
        wok[h] = row < N;
        wrow[h] = W + (size_t)(wok[h] ? row : 0) * ldw;
    }
    const __nv_bfloat16* xrow[NT];
    bool xok[NT];
    #pragma unroll
    for (int n = 0; n < NT; n++) {
        const int m = n * 8 + g;
        xok[n] = m < M;
        xrow[n] = X + (size_t)(xok[n] ? m : 0) * ldx;
    }

    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int nblk = (K + 63) / 64;                       // blocks of 64 k = two 32-k chunks, 128 bytes of a row
    // Weights do not depend on the kernel before this one: a warp asks for its first batch of them, and only
    // then waits for that kernel's results (the tokens).  Launched early, the wait hides this kernel's start-up.
    bool waited = false;
    for (int blk0 = warp * U; blk0 < nblk; blk0 += 8 * U) {
        uint4 a[U][2][H], b[U][2][NT];
        #pragma unroll
        for (int u = 0; u < U; u++)
            #pragma unroll
            for (int c = 0; c < 2; c++) {
                const int k = (blk0 + u) * 64 + c * 32 + t * 8;
                const bool kok = k < K;                   // K % 8 == 0: the whole 8 are inside
                #pragma unroll
                for (int h = 0; h < H; h++) a[u][c][h] = (kok && wok[h]) ? ld_stream(wrow[h] + k) : zero;
            }
        if (!waited) { ik_pdl_wait(); waited = true; }
        #pragma unroll
        for (int u = 0; u < U; u++)
            #pragma unroll
            for (int c = 0; c < 2; c++) {
                const int k = (blk0 + u) * 64 + c * 32 + t * 8;
                const bool kok = k < K;
                #pragma unroll
                for (int n = 0; n < NT; n++) b[u][c][n] = (kok && xok[n]) ? ld_tokens(xrow[n] + k) : zero;
            }
        #pragma unroll
        for (int u = 0; u < U; u++)
            #pragma unroll
            for (int c = 0; c < 2; c++)
                #pragma unroll
                for (int n = 0; n < NT; n++) {
                    const uint4 lo = a[u][c][0], hi = H == 2 ? a[u][c][H - 1] : zero;       // rows g and g + 8
                    mma_bf16(acc[n], lo.x, hi.x, lo.y, hi.y, b[u][c][n].x, b[u][c][n].y);
                    mma_bf16(acc[n], lo.z, hi.z, lo.w, hi.w, b[u][c][n].z, b[u][c][n].w);
                }
    }
    if (!waited) ik_pdl_wait();
    ik_pdl_launch_dependents();                           // the kernel after this one may begin its own start-up
    // partial sums of the 8 warps, added in warp order
    float* mine = red + (size_t)warp * R * COLS;
    #pragma unroll
    for (int n = 0; n < NT; n++) {
        const int col = n * 8 + 2 * t;
        mine[g * COLS + col] = acc[n][0];
        mine[g * COLS + col + 1] = acc[n][1];
        if (H == 2) {
            mine[(g + 8) * COLS + col] = acc[n][2];
            mine[(g + 8) * COLS + col + 1] = acc[n][3];
        }
    }
    __syncthreads();
    if (rope.q_out) {
        // rows are rotary pairs of q and k heads, then v heads: rotate and store to q_out and the cache
        for (int idx = threadIdx.x; idx < (R / 2) * COLS; idx += 256) {
            const int m = idx / (R / 2), pr = idx % (R / 2);
            if (m >= M || n0 + 2 * pr + 1 >= N) continue;
            float a = 0.f, b = 0.f;
            #pragma unroll
            for (int w = 0; w < 8; w++) {
                a += red[(size_t)w * R * COLS + (2 * pr) * COLS + m];
                b += red[(size_t)w * R * COLS + (2 * pr + 1) * COLS + m];
            }
            ik_rope_store_pair(rope, m, n0 + 2 * pr, a, b);
        }
        return;
    }
    if (swiglu) {
        // rows are (gate j, up j) pairs: Y[m, (n0 + row) / 2] = silu(gate) * up
        for (int idx = threadIdx.x; idx < (R / 2) * COLS; idx += 256) {
            const int m = idx / (R / 2), pr = idx % (R / 2);
            if (m >= M || n0 + 2 * pr + 1 >= N) continue;
            float gte = 0.f, up = 0.f;
            #pragma unroll
            for (int w = 0; w < 8; w++) {
                gte += red[(size_t)w * R * COLS + (2 * pr) * COLS + m];
                up += red[(size_t)w * R * COLS + (2 * pr + 1) * COLS + m];
            }
            store_out(Y, (size_t)m * ldy + n0 / 2 + pr, ik_swiglu_fast(gte, up), 0);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < R * COLS; idx += 256) {
        const int m = idx / R, row = idx % R;             // consecutive threads: consecutive features
        if (m >= M || n0 + row >= N) continue;
        float s = 0.f;
        #pragma unroll
        for (int w = 0; w < 8; w++) s += red[(size_t)w * R * COLS + row * COLS + m];
        store_out(Y, (size_t)m * ldy + n0 + row, s, accumulate);
    }
}

template <int NT, int U, typename TY, int R = 16>
int launch_skinny(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                  int accumulate, int swiglu, const IkRopeStore& rope, cudaStream_t stream) {
    const size_t smem = (size_t)8 * R * 8 * NT * sizeof(float);
    auto kern = gemm_skinny_kernel<NT, U, TY, R>;
    IK_RETURN_IF_ERROR(ik_launch(kern, (N + R - 1) / R, 256, smem, stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W,
                                 (TY*)Y, M, N, K, ldx, ldw, ldy, accumulate, swiglu, rope));
    IK_LAUNCH_STATUS();
}

// The deeper unroll (more bytes in flight, 2 blocks per SM instead of 3) pays unless the grid then fills
// its last wave of blocks badly.  Depends on N only, so a row's summation order does not depend on M.
bool deep_unroll_pays(int N) {
    const int blocks = (N + 15) / 16, slots = 2 * ik_sm_count();
    const int waves = (blocks + slots - 1) / slots;
    return (double)blocks / ((double)waves * slots) >= 0.8;
}

// Blocks of 8 rows instead of 16: when blocks of 16 would not even give every SM one (2,048 output features are 128
// blocks), and K is long enough for a block's eight warps to have work (at least 16 blocks of 64).  Depends on N and K
// only.  Measured on B200, 8 tokens, 2048 x 8192: see the kernel library's notes.
bool narrow_blocks_pay(int N, int K) {
    return (N + 15) / 16 <= ik_sm_count() && K >= 1024;
}

// ------------------------------------------------------------------------------------------ tiled
constexpr int TBM = 128, TBN = 128, TBK = 32, STAGES = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;                         // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(s), "l"(gmem), "r"(n));
}

template <typename TY>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, TY* __restrict__ Y,
                  int M, int N, int K, int ldx, int ldw, int ldy, int accumulate) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    __nv_bfloat16* xs = (__nv_bfloat16*)smem_raw;                         // [STAGES][TBM][TBK]
    __nv_bfloat16* ws = xs + (size_t)STAGES * TBM * TBK;                  // [STAGES][TBN][TBK]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp >> 2, wn = warp & 3;                              // 2 x 4 warps, each 64 tokens x 32 features
    const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
    const int nk = (K + TBK - 1) / TBK;

    auto load_stage = [&](int stage, int kt) {
        const int k0 = kt * TBK;
        #pragma unroll
        for (int l = 0; l < 2; l++) {
            const int idx = threadIdx.x + l * 256;                        // 512 chunks of 16 bytes per operand
            const int row = idx >> 2, ch = idx & 3;
            const int k = k0 + ch * 8;
            const bool kok = kt < nk && k < K;
            const bool xv = kok && (m0 + row) < M, wv = kok && (n0 + row) < N;
            cp_async16(xs + ((size_t)stage * TBM + row) * TBK + ch * 8, xv ? X + (size_t)(m0 + row) * ldx + k : X, xv);
            cp_async16(ws + ((size_t)stage * TBN + row) * TBK + ch * 8, wv ? W + (size_t)(n0 + row) * ldw + k : W, wv);
        }
        asm volatile("cp.async.commit_group;\n");
    };

    float acc[4][4][4];
    #pragma unroll
    for (int i = 0; i < 4; i++)
        #pragma unroll
        for (int j = 0; j < 4; j++)
            #pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;

    for (int s = 0; s < STAGES - 1; s++) load_stage(s, s);
    for (int kt = 0; kt < nk; kt++) {
        asm volatile("cp.async.wait_group %0;\n" :: "n"(STAGES - 2));
        __syncthreads();
        load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);          // refills the stage read at kt - 1
        const int st = kt % STAGES;
        const __nv_bfloat16* xa = xs + ((size_t)st * TBM + wm * 64) * TBK;
        const __nv_bfloat16* wb = ws + ((size_t)st * TBN + wn * 32) * TBK;
        uint4 a[4][2], b[4];
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            a[i][0] = *(const uint4*)(xa + (i * 16 + g) * TBK + t * 8);
            a[i][1] = *(const uint4*)(xa + (i * 16 + g + 8) * TBK + t * 8);
        }
        #pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *(const uint4*)(wb + (j * 8 + g) * TBK + t * 8);
        #pragma unroll
        for (int i = 0; i < 4; i++)
            #pragma unroll
            for (int j = 0; j < 4; j++) {
                mma_bf16(acc[i][j], a[i][0].x, a[i][1].x, a[i][0].y, a[i][1].y, b[j].x, b[j].y);
                mma_bf16(acc[i][j], a[i][0].z, a[i][1].z, a[i][0].w, a[i][1].w, b[j].z, b[j].w);
            }
    }
    asm volatile("cp.async.wait_group 0;\n");
    #pragma unroll
    for (int i = 0; i < 4; i++)
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + wn * 32 + j * 8 + 2 * t;
            #pragma unroll
            for (int h = 0; h < 2; h++) {
                const int m = m0 + wm * 64 + i * 16 + g + h * 8;
                if (m >= M) continue;
                if (n < N) store_out(Y, (size_t)m * ldy + n, acc[i][j][2 * h], accumulate);
                if (n + 1 < N) store_out(Y, (size_t)m * ldy + n + 1, acc[i][j][2 * h + 1], accumulate);
            }
        }
}

template <typename TY>
int launch_tiled(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy, int accumulate,
                 cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * (TBM + TBN) * TBK * sizeof(__nv_bfloat16);
    auto kern = gemm_tiled_kernel<TY>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((N + TBN - 1) / TBN, (M + TBM - 1) / TBM);
    IK_RETURN_IF_ERROR(ik_launch(kern, grid, 256, smem, stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (TY*)Y, M, N, K, ldx, ldw, ldy,
                                      accumulate));
    IK_LAUNCH_STATUS();
}

bool aligned_ok(const void* X, const void* W, int K, int ldx, int ldw) {
    return K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0;
}

}  // namespace

// kind: 0 = choose by M (skinny for M <= 64, else tiled), 1 = skinny, 2 = tiled.
// swiglu (skinny only): W holds (gate j, up j) in rows (2j, 2j + 1); Y is [M, N / 2] = silu(gate) * up.
static int gemm_bf16_mma_impl(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int ldx, int ldw,
                              int ldy, int accumulate, int kind, int swiglu, const IkRopeStore& rope, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || (!rope.q_out && ldy < (swiglu ? N / 2 : N))) return IK_BAD_ARGUMENT;
    if (swiglu && ((N & 1) || accumulate || kind == 2 || (kind == 0 && M > 64))) return IK_BAD_ARGUMENT;
    if (y_dtype != IK_F32 && y_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    if (!aligned_ok(X, W, K, ldx, ldw)) return IK_UNSUPPORTED;
    if (M == 0) return IK_OK;
    const bool skinny = kind == 1 || (kind == 0 && M <= 64);
    if (skinny && M > 64) return IK_UNSUPPORTED;
#define IK_SK(NT, U)                                                                                           \
    return y_dtype == IK_F32 ? launch_skinny<NT, U, float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, swiglu, rope, stream) \
                             : launch_skinny<NT, U, __nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, swiglu, rope, stream)
    if (skinny) {
        const bool deep = deep_unroll_pays(N);
        if (M <= 8 && narrow_blocks_pay(N, K)) {
            return y_dtype == IK_F32 ? launch_skinny<1, 8, float, 8>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, swiglu, rope, stream)
                                     : launch_skinny<1, 8, __nv_bfloat16, 8>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, swiglu, rope, stream);
        }
        if (M <= 8) { if (deep) { IK_SK(1, 4); } IK_SK(1, 2); }
        if (M <= 16) { if (deep) { IK_SK(2, 2); } IK_SK(2, 1); }
        if (M <= 32) { IK_SK(4, 1); }
        IK_SK(8, 1);
    }
#undef IK_SK
    return y_dtype == IK_F32 ? launch_tiled<float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream)
                             : launch_tiled<__nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
}

IK_EXPORT int ik_gemm_bf16_mma(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int ldx, int ldw,
                               int ldy, int accumulate, int kind, int swiglu, cudaStream_t stream) {
    IkRopeStore none = {};
    return gemm_bf16_mma_impl(X, W, Y, y_dtype, M, N, K, ldx, ldw, ldy, accumulate, kind, swiglu, none, stream);
}

// The fused q/k/v product of up to 64 tokens with the rotary / cache epilogue (rope_store.cuh).  N must be
// (nh + 2 nkv) * hd, hd even.
IK_EXPORT int ik_gemm_qkv_rope_mma(const void* X, const void* W, int M, int N, int K, int ldx, int ldw,
                                   const IkRopeStore* rope, cudaStream_t stream) {
    if (!rope || !rope->q_out || (rope->hd & 1) || N != (rope->nh + 2 * rope->nkv) * rope->hd || M > 64) return IK_BAD_ARGUMENT;
    return gemm_bf16_mma_impl(X, W, nullptr, IK_F32, M, N, K, ldx, ldw, N, 0, 1, 0, *rope, stream);
}
