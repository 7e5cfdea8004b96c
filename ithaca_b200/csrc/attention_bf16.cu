// Attention over the paged bfloat16 cache, specialised at compile time for one head size
// (IK_HD, a multiple of 16).  The file is compiled once per head size a model needs.
//
//  * prefill: causal grouped-query flash attention.  A block owns 16*NW query tokens of one
//    head of one sequence and walks the sequence's pages (64 keys each, aligned to absolute
//    positions).  S = Q K^T and O += P V run on mma.sync m16n8k16 with float accumulators; the
//    running maximum, the sum and the rescaling are float, in base 2 (scale * log2 e folded into
//    the scores).  P is rounded to bfloat16 for the second product, as the reference's
//    flash kernel rounds it to half (src/gx_kernels.cpp:535-690).
//  * decode: one query token per sequence.  A block owns (sequence, kv head, up to 16 of the
//    group's query heads, one chunk of keys) and reads every key and value of its chunk
//    exactly once for all its heads (the reference's k_attn_gqa, src/gpu_kernels.cpp:154-245),
//    on the same mma.sync tiles as prefill with the heads as the tile's rows.
//    Chunks start at absolute multiples of the chunk length; each block writes an
//    unnormalised partial (max, sum, output) and a second kernel merges the partials of a
//    head in chunk order (k_attn_comb, src/gpu_kernels.cpp:131-150).
//
// Keys beyond a sequence's length and outside the window are masked by position, so what lies
// in the unused part of a page never matters.  A page index outside the pool sets *status
// and is not followed.
#include <math.h>
#define IK_FAMILY 4
#include "common.cuh"
#include "tc_common.cuh"

#ifndef IK_HD
#error "compile with -DIK_HD=<head size>"
#endif

namespace {

constexpr int HD = IK_HD;
constexpr int PAGE = 64;
constexpr int LD = HD + 8;                 // padded row: consecutive rows fall into different banks
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 512, "head size must be a multiple of 16 up to 512");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------------------------------ prefill
template <int NW>
__global__ void __launch_bounds__(32 * NW)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                    bf16* __restrict__ out, const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                    const int* __restrict__ table, int table_stride, int nh, int nkv, float scale_log2e, int window,
                    int n_pages, int* status) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    constexpr int BM = 16 * NW, THREADS = 32 * NW, CH = HD / 8;          // CH: 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = (bf16*)smem_raw;                      // [BM][LD]
    bf16* Ks = Qs + BM * LD;                         // [2][PAGE][LD]
    bf16* Vs = Ks + 2 * PAGE * LD;                   // [2][PAGE][LD]

    const int b = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
    const int q_begin = cu_seqlens[b], n_new = cu_seqlens[b + 1] - q_begin;
    const int row0 = tile * BM;
    if (row0 >= n_new) return;
    const int kv_len = kv_lens[b], start = kv_len - n_new;
    const int rows = min(BM, n_new - row0);
    const int pos_lo = start + row0, pos_hi = start + row0 + rows - 1;
    const int j_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int p_lo = j_lo / PAGE, p_hi = pos_hi / PAGE;
    const int kvh = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // Q tile
    for (int idx = threadIdx.x; idx < BM * CH; idx += THREADS) {
        const int r = idx / CH, c = idx % CH;
        const bool v = r < rows;
        cp16(Qs + r * LD + c * 8, v ? q + ((size_t)(q_begin + row0 + r) * nh + h) * HD + c * 8 : q, v);
    }
    auto load_page = [&](int stage, int p) {
        int page = table[(size_t)b * table_stride + p];
        if (page < 0 || page >= n_pages) { if (threadIdx.x == 0) ik_set_status(status, IK_STATUS_READ_NO_PAGE); page = 0; }
        const bf16* kg = k_pages + ((size_t)page * nkv + kvh) * PAGE * HD;
        const bf16* vg = v_pages + ((size_t)page * nkv + kvh) * PAGE * HD;
        bf16* ks = Ks + stage * PAGE * LD;
        bf16* vs = Vs + stage * PAGE * LD;
        for (int idx = threadIdx.x; idx < PAGE * CH; idx += THREADS) {
            const int r = idx / CH, c = idx % CH;
            cp16(ks + r * LD + c * 8, kg + r * HD + c * 8, true);
            cp16(vs + r * LD + c * 8, vg + r * HD + c * 8, true);
        }
    };
    load_page(0, p_lo);
    cp_commit();

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
    #pragma unroll
    for (int d = 0; d < HD / 8; d++)
        #pragma unroll
        for (int e = 0; e < 4; e++) o[d][e] = 0.f;
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    const int my_pos[2] = {pos_lo + warp * 16 + g, pos_lo + warp * 16 + g + 8};
    const bool my_row[2] = {warp * 16 + g < rows, warp * 16 + g + 8 < rows};

    for (int p = p_lo; p <= p_hi; p++) {
        const int stage = (p - p_lo) & 1;
        if (p + 1 <= p_hi) load_page(stage ^ 1, p + 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (p == p_lo) {
            #pragma unroll
            for (int ks = 0; ks < HD / 16; ks++)
                ldsm4(qf[ks], Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* ks_ = Ks + stage * PAGE * LD;
        const bf16* vs_ = Vs + stage * PAGE * LD;
        float s[8][4];
        #pragma unroll
        for (int n = 0; n < 8; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) s[n][e] = 0.f;
        #pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            #pragma unroll
            for (int np = 0; np < 4; np++) {             // pairs of 8-key tiles
                uint32_t bfr[4];
                ldsm4(bfr, ks_ + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma(s[2 * np], qf[ks], bfr[0], bfr[1]);
                mma(s[2 * np + 1], qf[ks], bfr[2], bfr[3]);
            }
        }
        // mask by position, scale into base 2
        const int jbase = p * PAGE + 2 * t;
        float mx[2] = {-INFINITY, -INFINITY};
        #pragma unroll
        for (int n = 0; n < 8; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = e >> 1, j = jbase + n * 8 + (e & 1);
                const bool ok = my_row[r] && j <= my_pos[r] && (window <= 0 || j > my_pos[r] - window);
                const float v = ok ? s[n][e] * scale_log2e : -INFINITY;
                s[n][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        float alpha[2];
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_i[r], mx[r]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = exp2f(m_i[r] - m_use);
            m_i[r] = m_new;
            mx[r] = m_use;
        }
        float rs[2] = {0.f, 0.f};
        #pragma unroll
        for (int n = 0; n < 8; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pv = exp2f(s[n][e] - mx[e >> 1]);
                s[n][e] = pv;
                rs[e >> 1] += pv;
            }
        #pragma unroll
        for (int r = 0; r < 2; r++) l_i[r] = l_i[r] * alpha[r] + rs[r];
        #pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            o[d][0] *= alpha[0]; o[d][1] *= alpha[0]; o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
        }
        #pragma unroll
        for (int kk = 0; kk < 4; kk++) {                 // 16 keys each
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            #pragma unroll
            for (int dp = 0; dp < HD / 16; dp++) {       // pairs of 8-dim tiles
                uint32_t bfr[4];
                ldsm4t(bfr, vs_ + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + (lane >> 4) * 8);
                mma(o[2 * dp], pa, bfr[0], bfr[1]);
                mma(o[2 * dp + 1], pa, bfr[2], bfr[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
    }
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        if (!my_row[r]) continue;
        const float inv = 1.0f / l_i[r];
        bf16* orow = out + ((size_t)(q_begin + row0 + warp * 16 + g + r * 8) * nh + h) * HD;
        #pragma unroll
        for (int d = 0; d < HD / 8; d++)
            *reinterpret_cast<uint32_t*>(orow + d * 8 + 2 * t) = pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------ prefill, tcgen05
// The same attention on the fifth-generation tensor cores, for head sizes 64 and 128.
// A block owns 128 query tokens of one head of one sequence (one TMEM lane per query) and walks
// the sequence's pages, 64 keys at a time:
//   warp 0      TMA: the query tile once, then each page's keys and values into two rings of two stages.  A
//               key stage is free as soon as its S = Q K^T has run, a value stage after its O += P V; the keys
//               are asked for one page ahead of the values, so that neither load's latency shows.
//   warp 1      tcgen05.mma: S = Q K^T into one of two 64-column score buffers in TMEM (the product for
//               page i + 1 is issued before the softmax of page i is done), then O += P V with P read
//               from TMEM and V as an N-contiguous operand straight from the page.
//   warps 2..5  softmax: each thread reads its query's 64 scores from TMEM, masks by position, keeps
//               the running maximum and sum in float (base 2), and writes P as bfloat16 over the first 32
//               columns of the score buffer it has just read.  P of page i and P of page i + 1 thus lie in
//               different buffers, and the tensor core runs its products in the order they were issued, so the
//               softmax of page i + 1 never waits for O += P V of page i; only the rare rescaling of its row of
//               O (the maximum moved by more than a factor 256) does.
// All mbarrier waits are bounded (tc_common.cuh); on a timeout the status word is set and the block
// leaves its loops and frees its TMEM.
#if IK_HD == 64 || IK_HD == 128
constexpr int TC_BM = 128, TC_NS = 2;                          // two blocks per SM: one's softmax runs beside the other's MMAs
constexpr int TC_BOXES = HD / 64;                              // 64-wide swizzled blocks along the head size
constexpr int TC_Q_BYTES = TC_BM * HD * 2;
constexpr int TC_KV_BYTES = PAGE * HD * 2;
constexpr int TC_SMEM = TC_Q_BYTES + TC_NS * 2 * TC_KV_BYTES + 256;   // no slack for alignment: see the check in the kernel
constexpr int TC_TMEM_COLS = 256;                              // scores 2 x 64, output HD (<= 128)
constexpr int TC_O_COL = 128;

__global__ void __launch_bounds__(192, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                       const int* __restrict__ table, int table_stride, int nh, int nkv, float scale_log2e,
                       int window, int n_pages, int* status) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    // Late tiles see the most keys: over the whole grid they are started first (blocks start in the order of their
    // linear index), so that the short ones fill the tail; heads that share keys and values start side by side.
    const int linear = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z), per_tile = gridDim.y * gridDim.z;
    const int tile = gridDim.x - 1 - linear / per_tile, h = (linear % per_tile) % gridDim.y, b = (linear % per_tile) / gridDim.y;
    const int q_begin = cu_seqlens[b], n_new = cu_seqlens[b + 1] - q_begin;
    const int row0 = tile * TC_BM;
    if (row0 >= n_new) return;
    if (ik_status_has(status, IK_STATUS_GEMM_TIMEOUT)) return;
    const int kv_len = kv_lens[b], start = kv_len - n_new;
    const int rows = min(TC_BM, n_new - row0);
    const int pos_lo = start + row0, pos_hi = pos_lo + rows - 1;
    const int j_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int p_lo = j_lo / PAGE, n_iter = pos_hi / PAGE - p_lo + 1;
    const int kvh = h / (nh / nkv);

    // The swizzled tiles need 1024-byte alignment.  Dynamic shared memory of a kernel without static shared
    // memory starts on such a boundary; should it ever not, the block reports it instead of computing garbage.
    if (smem_u32(tc_smem) & 1023) {
        if (threadIdx.x == 0) ik_set_status(status, IK_STATUS_SMEM_ALIGN);
        return;
    }
    unsigned char* Qs = tc_smem;
    unsigned char* Ks = Qs + TC_Q_BYTES;                       // [TC_NS][TC_KV_BYTES]
    unsigned char* Vs = Ks + TC_NS * TC_KV_BYTES;
    uint64_t* q_full = (uint64_t*)(Vs + TC_NS * TC_KV_BYTES);
    uint64_t* k_full = q_full + 1;                             // [TC_NS]
    uint64_t* v_full = k_full + TC_NS;
    uint64_t* k_free = v_full + TC_NS;
    uint64_t* v_free = k_free + TC_NS;
    uint64_t* s_full = v_free + TC_NS;                         // [2]
    uint64_t* p_ready = s_full + 2;                            // [2] the probabilities of a page are written: even pages, odd pages
    uint64_t* pv_done = p_ready + 2;
    uint64_t* o_done = pv_done + 1;                            // the tile's last product has run: used once, so its parity is 0
    uint32_t* tmem_slot = (uint32_t*)(o_done + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < TC_NS; s++) {
            mbar_init(k_full + s, 1); mbar_init(v_full + s, 1); mbar_init(k_free + s, 1); mbar_init(v_free + s, 1);
        }
        mbar_init(s_full, 1); mbar_init(s_full + 1, 1);
        mbar_init(p_ready, 128); mbar_init(p_ready + 1, 128);
        mbar_init(pv_done, 1);
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_v) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"((uint32_t)TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, TC_Q_BYTES);
            for (int bx = 0; bx < TC_BOXES; bx++)
                tma_load_2d(Qs + bx * (TC_BM * 128), &map_q, h * HD + bx * 64, q_begin + row0, q_full);
            auto page_row = [&](int i) -> int {
                int page = table[(size_t)b * table_stride + p_lo + i];
                if (page < 0 || page >= n_pages) { ik_set_status(status, IK_STATUS_READ_NO_PAGE); page = 0; }
                return (page * nkv + kvh) * PAGE;
            };
            // keys of page i, then values of page i - 1
            for (int i = 0; i <= n_iter; i++) {
                if (i < n_iter) {
                    const int s = i % TC_NS;
                    if (!mbar_wait(k_free + s, ((i / TC_NS) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 11, i)) break;
                    const int row = page_row(i);
                    mbar_expect_tx(k_full + s, TC_KV_BYTES);
                    for (int bx = 0; bx < TC_BOXES; bx++)
                        tma_load_2d(Ks + s * TC_KV_BYTES + bx * (PAGE * 128), &map_k, bx * 64, row, k_full + s);
                }
                if (i > 0) {
                    const int s = (i - 1) % TC_NS;
                    if (!mbar_wait(v_free + s, (((i - 1) / TC_NS) & 1) ^ 1, abort_flag, status, IK_WAIT_LIMIT_NS, 12, i)) break;
                    const int row = page_row(i - 1);
                    mbar_expect_tx(v_full + s, TC_KV_BYTES);
                    for (int bx = 0; bx < TC_BOXES; bx++)
                        tma_load_2d(Vs + s * TC_KV_BYTES + bx * (PAGE * 128), &map_v, bx * 64, row, v_full + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc(PAGE), idesc_pv = umma_idesc(HD, 1);
            const uint32_t q_addr = smem_u32(Qs);
            bool ok = mbar_wait(q_full, 0, abort_flag, status, IK_WAIT_LIMIT_NS, 13, 0);
            auto issue_qk = [&](int i) -> bool {
                const int s = i % TC_NS;
                if (!mbar_wait(k_full + s, (i / TC_NS) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 14, i)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = smem_u32(Ks + s * TC_KV_BYTES);
                #pragma unroll
                for (int j = 0; j < HD / 16; j++)
                    umma(tmem + (i & 1) * PAGE, umma_desc(q_addr + (j / 4) * (TC_BM * 128) + (j % 4) * 32),
                         umma_desc(k_addr + (j / 4) * (PAGE * 128) + (j % 4) * 32), idesc_qk, j != 0);
                umma_commit(s_full + (i & 1));
                umma_commit(k_free + s);                   // the key stage is free once these products have read it
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int i = 0; i < n_iter && ok; i++) {
                if (i + 1 < n_iter) { ok = issue_qk(i + 1); if (!ok) break; }     // runs while page i is in the softmax
                const int s = i % TC_NS;
                ok = mbar_wait(p_ready + (i & 1), (i >> 1) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 15, i) && mbar_wait(v_full + s, (i / TC_NS) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 16, i);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = smem_u32(Vs + s * TC_KV_BYTES);
                #pragma unroll
                for (int j = 0; j < PAGE / 16; j++)
                    umma_ts(tmem + TC_O_COL, tmem + (i & 1) * PAGE + j * 8, umma_desc_mn(v_addr + j * 2048, PAGE * 128),
                            idesc_pv, (i | j) != 0);
                umma_commit(v_free + s);
                umma_commit(pv_done);
            }
            if (ok) umma_commit(o_done);
        }
    } else {
        const int quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool row_valid = r < rows;
        const int pos_r = pos_lo + r;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_iter && ok; i++) {
            const int p = p_lo + i;
            ok = mbar_wait(s_full + (i & 1), (i >> 1) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 17, i);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[PAGE];
            #pragma unroll
            for (int c0 = 0; c0 < PAGE; c0 += 16) tmem_ld16_issue(lane_base + (i & 1) * PAGE + c0, sc + c0);
            tmem_ld_wait();
            const bool need_mask = (p * PAGE + PAGE - 1 > pos_lo) || (window > 0 && p * PAGE < pos_hi + 1 - window);
            // Few instructions per score: the maximum is taken over the raw scores and scaled once (the scale is
            // positive), and the scaling of a score is folded into the subtraction of the reference below.  Four
            // independent chains for the maximum (and for the sum): a dependent chain's latency would show.  Rows
            // past the sequence's end are only cut off where a mask is applied anyway (its last pages); before that
            // they compute on whatever the query tile holds there, and are never stored.
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (need_mask) {
                #pragma unroll
                for (int c = 0; c < PAGE; c++) {
                    const int j = p * PAGE + c;
                    const bool in = row_valid && j <= pos_r && (window <= 0 || j > pos_r - window);
                    sc[c] = in ? sc[c] : -INFINITY;
                    mx4[c & 3] = fmaxf(mx4[c & 3], sc[c]);
                }
            } else {
                #pragma unroll
                for (int c = 0; c < PAGE; c += 2) mx4[(c >> 1) & 3] = max3(mx4[(c >> 1) & 3], sc[c], sc[c + 1]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2e;
            // m is the reference the exponentials are taken against.  It follows the running maximum only when
            // that has moved by more than 8 (a factor 256): until then the probabilities may exceed 1 by that
            // factor, which float sums and bfloat16 operands take in their stride, and O needs no rescaling.
            float alpha = 1.f;
            if (mx > m + 8.f) {
                alpha = ik_ex2(m - mx);                                          // 0 on the first page (m = -inf)
                m = mx;
            }
            const float m_use = m == -INFINITY ? 0.f : m;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int c = 0; c < PAGE; c += 2) {            // two scores per multiply-add and per add
                float a0, a1;
                fma_f32x2(a0, a1, sc[c], sc[c + 1], scale_log2e, -m_use);
                sc[c] = ik_ex2(a0);
                sc[c + 1] = ik_ex2(a1);
                add_f32x2(sum4[c & 2], sum4[(c & 2) + 1], sc[c], sc[c + 1]);
            }
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O is at rest between the product of the page before (waited for here) and this page's (which waits
                // for this thread).  The barrier has completed i - 1 or i phases at this point, whatever was waited
                // for earlier, so the parity names the right one.
                ok = mbar_wait(pv_done, (i - 1) & 1, abort_flag, status, IK_WAIT_LIMIT_NS, 18, i);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                #pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float v[32];
                    tmem_ld16_issue(lane_base + TC_O_COL + c0, v);
                    tmem_ld16_issue(lane_base + TC_O_COL + c0 + 16, v + 16);
                    tmem_ld_wait();
                    #pragma unroll
                    for (int c = 0; c < 32; c++) v[c] *= alpha;
                    tmem_st16(lane_base + TC_O_COL + c0, *reinterpret_cast<float(*)[16]>(v));
                    tmem_st16(lane_base + TC_O_COL + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
                }
            }
            // this query's 64 probabilities, two per cell, over the scores they came from
            #pragma unroll
            for (int c0 = 0; c0 < PAGE / 2; c0 += 16) {
                uint32_t pk[16];
                #pragma unroll
                for (int c = 0; c < 16; c++) pk[c] = pack_bf16(sc[2 * (c0 + c)], sc[2 * (c0 + c) + 1]);
                tmem_st16_bits(lane_base + (i & 1) * PAGE + c0, pk);
            }
            tmem_st_wait();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // The arrivals of even and of odd pages are counted on barriers of their own.  A barrier counts arrivals,
            // not threads, and a wait names its phase by parity alone: with one barrier for all pages a thread that is a
            // page ahead (the scores of page i + 1 can be there before everybody has arrived for page i) would complete
            // the phase of one that is behind, and the issuing thread could find the barrier two phases on.  On its
            // own barrier page i meets only pages i - 2 and i + 2: everybody has arrived for page i - 2 before the scores
            // of page i are even asked for, and the scores of page i + 2 are asked for only after the issuing thread
            // has seen everybody arrive for page i.
            mbar_arrive(p_ready + (i & 1));
        }
        // The last product, on a barrier of its own.  pv_done will not do here: a wait names a phase by its parity, which
        // is only safe while the barrier can be at most one phase away from the one meant.  Behind its last arrival a
        // thread knows nothing of pv_done but that it is one or two products short of the end, and while it waits for the
        // product before the last both may complete: the barrier then stands two phases on, at the same parity again, and
        // the wait never ends (seen on one box as an expired wait at this place, in tiles of two pages).
        if (ok && mbar_wait(o_done, 0, abort_flag, status, IK_WAIT_LIMIT_NS, 21, n_iter)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = 1.0f / l;
            bf16* orow = out + ((size_t)(q_begin + row0 + r) * nh + h) * HD;
            #pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 16) {
                float v[16];
                tmem_ld16(lane_base + TC_O_COL + c0, v);
                if (row_valid) {
                    uint4 w0, w1;
                    w0.x = pack_bf16(v[0] * inv, v[1] * inv);   w0.y = pack_bf16(v[2] * inv, v[3] * inv);
                    w0.z = pack_bf16(v[4] * inv, v[5] * inv);   w0.w = pack_bf16(v[6] * inv, v[7] * inv);
                    w1.x = pack_bf16(v[8] * inv, v[9] * inv);   w1.y = pack_bf16(v[10] * inv, v[11] * inv);
                    w1.z = pack_bf16(v[12] * inv, v[13] * inv); w1.w = pack_bf16(v[14] * inv, v[15] * inv);
                    *reinterpret_cast<uint4*>(orow + c0) = w0;
                    *reinterpret_cast<uint4*>(orow + c0 + 8) = w1;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)TC_TMEM_COLS) : "memory");
    }
}
#endif  // head sizes 64 and 128

// ------------------------------------------------------------------------------------------ decode
// One block: (sequence, kv head, up to 16 of the group's query heads, one chunk of pages).
// The query heads are the 16 rows of the MMA tile, so every key and value of the chunk is read
// once for all of them.  Pages stream through an NS-stage cp.async ring; each of the 4 warps
// takes 16 of a page's 64 keys, keeps its own running (max, sum, output) and the four are
// merged in warp order at the end.
template <int NS>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                   float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ kv_lens,
                   const int* __restrict__ table, int table_stride, int nh, int nkv, float scale_log2e, int window,
                   int n_pages, int chunk_pages, int n_splits, int* status) {
    ik_pdl_wait();
    constexpr int CH = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = (bf16*)smem_raw;                      // [16][LD]
    bf16* Ks = Qs + 16 * LD;                         // [NS][PAGE][LD]
    bf16* Vs = Ks + NS * PAGE * LD;                  // [NS][PAGE][LD]

    const int b = blockIdx.x, split = blockIdx.z;
    const int G = nh / nkv, n_hc = (G + 15) / 16;
    const int kvh = blockIdx.y / n_hc, hc = blockIdx.y % n_hc;
    const int len = kv_lens[b], pos = len - 1;
    const int j0 = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int p_first = max(split * chunk_pages, j0 / PAGE);
    const int p_last = min((split + 1) * chunk_pages - 1, pos / PAGE);
    if (p_first > p_last) return;                                  // nothing of this chunk is visible

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int h0 = kvh * G + hc * 16;                               // first query head of this block
    const int n_here = min(16, G - hc * 16);

    for (int idx = threadIdx.x; idx < 16 * CH; idx += 128) {
        const int r = idx / CH, c = idx % CH;
        const bool v = r < n_here;
        cp16(Qs + r * LD + c * 8, v ? q + ((size_t)b * nh + h0 + r) * HD + c * 8 : q, v);
    }
    auto load_page = [&](int stage, int p) {
        int page = table[(size_t)b * table_stride + p];
        if (page < 0 || page >= n_pages) { if (threadIdx.x == 0) ik_set_status(status, IK_STATUS_READ_NO_PAGE); page = 0; }
        const bf16* kg = k_pages + ((size_t)page * nkv + kvh) * PAGE * HD;
        const bf16* vg = v_pages + ((size_t)page * nkv + kvh) * PAGE * HD;
        bf16* ks = Ks + stage * PAGE * LD;
        bf16* vs = Vs + stage * PAGE * LD;
        for (int idx = threadIdx.x; idx < PAGE * CH; idx += 128) {
            const int r = idx / CH, c = idx % CH;
            cp16(ks + r * LD + c * 8, kg + r * HD + c * 8, true);
            cp16(vs + r * LD + c * 8, vg + r * HD + c * 8, true);
        }
    };
    #pragma unroll
    for (int s = 0; s < NS; s++) {
        if (p_first + s <= p_last) load_page(s, p_first + s);
        cp_commit();
    }

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
    #pragma unroll
    for (int d = 0; d < HD / 8; d++)
        #pragma unroll
        for (int e = 0; e < 4; e++) o[d][e] = 0.f;
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    const bool my_row[2] = {g < n_here, g + 8 < n_here};

    for (int p = p_first; p <= p_last; p++) {
        const int stage = (p - p_first) % NS;
        cp_wait<NS - 1>();
        __syncthreads();
        if (p == p_first) {
            #pragma unroll
            for (int ks = 0; ks < HD / 16; ks++)
                ldsm4(qf[ks], Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* ks_ = Ks + (stage * PAGE + warp * 16) * LD;
        const bf16* vs_ = Vs + (stage * PAGE + warp * 16) * LD;
        float s[2][4];
        #pragma unroll
        for (int n = 0; n < 2; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) s[n][e] = 0.f;
        #pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t bfr[4];
            ldsm4(bfr, ks_ + ((lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
            mma(s[0], qf[ks], bfr[0], bfr[1]);
            mma(s[1], qf[ks], bfr[2], bfr[3]);
        }
        const int jbase = p * PAGE + warp * 16 + 2 * t;
        float mx[2] = {-INFINITY, -INFINITY};
        #pragma unroll
        for (int n = 0; n < 2; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = e >> 1, j = jbase + n * 8 + (e & 1);
                const bool ok = my_row[r] && j <= pos && j >= j0;
                const float v = ok ? s[n][e] * scale_log2e : -INFINITY;
                s[n][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        float alpha[2];
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_i[r], mx[r]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = exp2f(m_i[r] - m_use);
            m_i[r] = m_new;
            mx[r] = m_use;
        }
        float rs[2] = {0.f, 0.f};
        #pragma unroll
        for (int n = 0; n < 2; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pv = exp2f(s[n][e] - mx[e >> 1]);
                s[n][e] = pv;
                rs[e >> 1] += pv;
            }
        #pragma unroll
        for (int r = 0; r < 2; r++) l_i[r] = l_i[r] * alpha[r] + rs[r];
        #pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            o[d][0] *= alpha[0]; o[d][1] *= alpha[0]; o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
        }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        #pragma unroll
        for (int dp = 0; dp < HD / 16; dp++) {
            uint32_t bfr[4];
            ldsm4t(bfr, vs_ + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + (lane >> 4) * 8);
            mma(o[2 * dp], pa, bfr[0], bfr[1]);
            mma(o[2 * dp + 1], pa, bfr[2], bfr[3]);
        }
        __syncthreads();                                            // everyone is done with this stage
        if (p + NS <= p_last) load_page(stage, p + NS);
        cp_commit();
    }
    cp_wait<0>();
    ik_pdl_launch_dependents();                                     // every key and value of this block has been read
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
    }
    // the four warps' partial results, merged in warp order (the K/V ring is free now)
    float* sm_o = (float*)Ks;                         // [4][16][HD]
    float* sm_ml = sm_o + 4 * 16 * HD;                // [4][16][2]
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = g + 8 * r;
        #pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            sm_o[(warp * 16 + row) * HD + d * 8 + 2 * t] = o[d][2 * r];
            sm_o[(warp * 16 + row) * HD + d * 8 + 2 * t + 1] = o[d][2 * r + 1];
        }
        if (t == 0) { sm_ml[(warp * 16 + row) * 2] = m_i[r]; sm_ml[(warp * 16 + row) * 2 + 1] = l_i[r]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_here * HD; idx += 128) {
        const int hh = idx / HD, x = idx % HD;
        float mm = -INFINITY;
        #pragma unroll
        for (int w = 0; w < 4; w++) mm = fmaxf(mm, sm_ml[(w * 16 + hh) * 2]);
        const float m_use = mm == -INFINITY ? 0.f : mm;
        float acc = 0.f, ll = 0.f;
        #pragma unroll
        for (int w = 0; w < 4; w++) {
            const float a = exp2f(sm_ml[(w * 16 + hh) * 2] - m_use);
            acc += sm_o[(w * 16 + hh) * HD + x] * a;
            ll += sm_ml[(w * 16 + hh) * 2 + 1] * a;
        }
        const size_t slot = ((size_t)b * nh + h0 + hh) * n_splits + split;
        part_o[slot * HD + x] = acc;
        if (x == 0) { part_ml[slot * 2] = mm; part_ml[slot * 2 + 1] = ll; }
    }
}

// Merges the partials of each (sequence, head) in chunk order and writes the normalised output.
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, const int* __restrict__ kv_lens, int nh, int window,
                                    int chunk_pages, int n_splits) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y;
    const int len = kv_lens[b], pos = len - 1;
    const int j0 = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int s_first = (j0 / PAGE) / chunk_pages, s_last = (pos / PAGE) / chunk_pages;
    const size_t base = ((size_t)b * nh + h) * n_splits;
    float mm = -INFINITY;
    for (int s = s_first; s <= s_last; s++) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    const float m_use = mm == -INFINITY ? 0.f : mm;
    for (int x = threadIdx.x; x < HD; x += blockDim.x) {
        float acc = 0.f, ll = 0.f;
        for (int s = s_first; s <= s_last; s++) {
            const float a = exp2f(part_ml[(base + s) * 2] - m_use);
            acc += part_o[(base + s) * HD + x] * a;
            ll += part_ml[(base + s) * 2 + 1] * a;
        }
        out[((size_t)b * nh + h) * HD + x] = __float2bfloat16_rn(acc / ll);
    }
}

}  // namespace

IK_EXPORT int ik_attn_head_dim() { return HD; }

// Sites of the tcgen05 prefill kernel's waits: 11, 12 = loader for a free key / value stage; 13 = issuer for the
// queries; 14 = issuer for keys; 15 = issuer for the probabilities; 16 = issuer for values; 17 = softmax for scores;
// 18 = softmax for the product before a rescaling; 21 = softmax for the tile's last product.
IK_EXPORT int ik_attn_take_wait_record(int* out4) { return ik_take_wait_record(out4); }

IK_EXPORT int ik_attn_prefill(const void* q, const void* k_pages, const void* v_pages, void* out, const int* cu_seqlens,
                              const int* kv_lens, const int* table, int table_stride, int B, int max_new, int nh,
                              int nkv, float scale, int window, int page_size, int n_pages, int* status,
                              cudaStream_t stream) {
    if (B <= 0 || max_new <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size != PAGE || B > 65535 || nh > 65535)
        return IK_BAD_ARGUMENT;
    constexpr int NW = 4, BM = 16 * NW;
    const size_t smem = (size_t)(BM + 4 * PAGE) * LD * sizeof(bf16);
    auto kern = attn_prefill_kernel<NW>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((max_new + BM - 1) / BM, nh, B);
    IK_RETURN_IF_ERROR(ik_launch(kern, grid, 32 * NW, smem, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out,
                                          cu_seqlens, kv_lens, table, table_stride, nh, nkv,
                                          scale * 1.4426950408889634f, window, n_pages, status));
    IK_LAUNCH_STATUS();
}

// The tcgen05 kernel (head sizes 64 and 128; IK_UNSUPPORTED otherwise).  T: rows of q.
IK_EXPORT int ik_attn_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out, const int* cu_seqlens,
                                 const int* kv_lens, const int* table, int table_stride, int T, int B, int max_new, int nh,
                                 int nkv, float scale, int window, int page_size, int n_pages, int* status,
                                 cudaStream_t stream) {
#if IK_HD == 64 || IK_HD == 128
    if (T <= 0 || B <= 0 || max_new <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size != PAGE || B > 65535 || nh > 65535)
        return IK_BAD_ARGUMENT;
    if (((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16)) return IK_UNSUPPORTED;
    if (!(scale > 0.f)) return IK_UNSUPPORTED;             // the kernel takes the maximum of the raw scores
    CUtensorMap mq, mk, mv;
    int st = ik_make_map(&mq, q, (unsigned long long)T, nh * HD, (unsigned long long)nh * HD, TC_BM);
    if (st != IK_OK) return st;
    const unsigned long long kv_rows = (unsigned long long)n_pages * nkv * PAGE;
    st = ik_make_map(&mk, k_pages, kv_rows, HD, HD, PAGE);
    if (st != IK_OK) return st;
    st = ik_make_map(&mv, v_pages, kv_rows, HD, HD, PAGE);
    if (st != IK_OK) return st;
    auto kern = attn_prefill_tc_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_new + TC_BM - 1) / TC_BM, nh, B);
    IK_RETURN_IF_ERROR(ik_launch(kern, grid, 192, TC_SMEM, stream, mq, mk, mv, (bf16*)out, cu_seqlens, kv_lens, table,
                                 table_stride, nh, nkv, scale * 1.4426950408889634f, window, n_pages, status));
    IK_LAUNCH_STATUS();
#else
    return IK_UNSUPPORTED;
#endif
}

// part_o: [B, nh, n_splits, HD] floats, part_ml: [B, nh, n_splits, 2] floats, both owned by the caller.
// n_splits must cover the longest sequence: n_splits * chunk_pages * 64 >= max kv length.
IK_EXPORT int ik_attn_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o,
                             float* part_ml, const int* kv_lens, const int* table, int table_stride, int B, int nh,
                             int nkv, float scale, int window, int page_size, int n_pages, int chunk_pages,
                             int n_splits, int ring_kb, int* status, cudaStream_t stream) {
    if (B <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size != PAGE || chunk_pages <= 0 || n_splits <= 0 ||
        n_splits > 65535)
        return IK_BAD_ARGUMENT;
    const int G = nh / nkv, n_hc = (G + 15) / 16;
    if ((long long)nkv * n_hc > 65535) return IK_BAD_ARGUMENT;
    dim3 grid(B, nkv * n_hc, n_splits);
    // as many ring stages as fit ring_kb (default 105 KB), at least 2, at most 4
    const size_t q_bytes = (size_t)16 * LD * sizeof(bf16), stage_bytes = (size_t)2 * PAGE * LD * sizeof(bf16);
    if (ring_kb <= 0) ring_kb = 105;
    int ns = (int)(((size_t)ring_kb * 1024 - q_bytes) / stage_bytes);
    ns = ns < 2 ? 2 : ns > 4 ? 4 : ns;
    const size_t smem = q_bytes + ns * stage_bytes;
#define IK_DEC(NS_)                                                                                                  \
    {                                                                                                                \
        auto kern = attn_decode_kernel<NS_>;                                                                         \
        if (smem > 48 * 1024) {                                                                                      \
            cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
            if (e0 != cudaSuccess) return (int)e0;                                                                   \
        }                                                                                                            \
        IK_RETURN_IF_ERROR(ik_launch(kern, grid, 128, smem, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, part_o, part_ml, \
                                          kv_lens, table, table_stride, nh, nkv, scale * 1.4426950408889634f, window, \
                                          n_pages, chunk_pages, n_splits, status));                                   \
    }
    if (ns == 2) IK_DEC(2) else if (ns == 3) IK_DEC(3) else IK_DEC(4)
#undef IK_DEC
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    dim3 grid2(B, nh);
    IK_RETURN_IF_ERROR(ik_launch_family(IK_FAMILY_ATTENTION_MERGE, attn_combine_kernel, grid2, HD < 128 ? HD : 128, 0, stream, part_o, part_ml, (bf16*)out, kv_lens, nh, window,
                                                                    chunk_pages, n_splits));
    IK_LAUNCH_STATUS();
}
