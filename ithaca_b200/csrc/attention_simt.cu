// Attention over the paged cache on the CUDA cores, for prefill and decode alike.
//
// One block per (query token, head).  Keys run from j0 to the token's own position
// (causal by loop bound; j0 > 0 only under a window), in tiles of 128 that start at
// absolute multiples of 128, so the order in which a query's keys are reduced depends
// only on its position, not on how the tokens were cut into steps or batched.
// Scores, the running maximum, the sum and the output are float; exp is the accurate
// function.  This is the 32-bit path's attention and the fallback for head sizes the
// tensor-core kernels do not take.
#include <math.h>
#define IK_FAMILY 4
#include "common.cuh"

namespace {

constexpr int TILE = 128;       // keys per tile = threads per block
constexpr int MAX_R = 4;        // head dims per thread: head_dim <= 512

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(TILE)
attention_simt_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_pages, const TC* __restrict__ v_pages,
                      TO* __restrict__ out, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                      const int* __restrict__ table, int table_stride, int nh, int nkv, int hd, float scale,
                      int window, int page_size, int n_pages, int* status) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem[];
    size_t* row = (size_t*)smem;              // [TILE] element offset of key j's row in the pages
    float* qs = (float*)(row + TILE);         // [hd]
    float* sc = qs + hd;                      // [TILE]
    float* red = sc + TILE;                   // [32]

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (nh / nkv);
    const int pos = token_pos[t], seq = token_seq[t];
    const int j0 = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;

    const TQ* qrow = q + ((size_t)t * nh + h) * hd;
    for (int i = tid; i < hd; i += TILE) qs[i] = ik_ld(qrow, i);

    float m = -INFINITY, l = 0.f, o[MAX_R];
    #pragma unroll
    for (int r = 0; r < MAX_R; r++) o[r] = 0.f;
    __syncthreads();

    for (int base = (j0 / TILE) * TILE; base <= pos; base += TILE) {
        const int j = base + tid;
        const bool valid = j >= j0 && j <= pos;
        float s = -INFINITY;
        size_t off = 0;
        if (valid) {
            const int page = table[(size_t)seq * table_stride + j / page_size];
            if (page < 0 || page >= n_pages) {
                ik_set_status(status, IK_STATUS_READ_NO_PAGE);
                off = 0;
            } else {
                off = (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * hd;
            }
            const TC* kr = k_pages + off;
            float dot = 0.f;
            for (int i = 0; i < hd; i++) dot = fmaf(qs[i], ik_ld(kr, i), dot);
            s = dot * scale;
        }
        row[tid] = off;
        const float tile_max = ik_block_max<TILE>(s, red);
        const float m_new = fmaxf(m, tile_max);
        const float p = valid ? expf(s - m_new) : 0.f;
        sc[tid] = p;
        const float tile_sum = ik_block_sum<TILE>(p, red);     // its barriers also publish sc[] and row[]
        const float alpha = expf(m - m_new);                   // 0 on the first tile (m = -inf)
        l = l * alpha + tile_sum;
        const int n_in_tile = min(TILE, pos - base + 1);
        #pragma unroll
        for (int r = 0; r < MAX_R; r++) {
            const int i = tid + r * TILE;
            if (i < hd) {
                float acc = o[r] * alpha;
                for (int jj = 0; jj < n_in_tile; jj++) {
                    const float pj = sc[jj];
                    if (pj != 0.f) acc = fmaf(pj, ik_ld(v_pages + row[jj], i), acc);
                }
                o[r] = acc;
            }
        }
        m = m_new;
        __syncthreads();                                       // sc[] and row[] are rewritten by the next tile
    }
    TO* orow = out + ((size_t)t * nh + h) * hd;
    const float inv = 1.0f / l;
    #pragma unroll
    for (int r = 0; r < MAX_R; r++) {
        const int i = tid + r * TILE;
        if (i < hd) ik_st(orow, i, o[r] * inv);
    }
}

}  // namespace

IK_EXPORT int ik_attention_simt(const void* q, int q_dtype, const void* k_pages, const void* v_pages, int cache_dtype,
                                void* out, int out_dtype, const int* token_seq, const int* token_pos, const int* table,
                                int table_stride, int T, int nh, int nkv, int hd, float scale, int window,
                                int page_size, int n_pages, int* status, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || hd > TILE * MAX_R || page_size <= 0) return IK_BAD_ARGUMENT;
    if (q_dtype != out_dtype) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    dim3 grid(T, nh);
    const size_t smem = (size_t)(hd + TILE + 32) * sizeof(float) + TILE * sizeof(size_t);
#define IK_ATT(TQ, TC)                                                                                                \
    IK_RETURN_IF_ERROR(ik_launch(attention_simt_kernel<TQ, TC, TQ>, grid, TILE, smem, stream, (const TQ*)q, (const TC*)k_pages, (const TC*)v_pages, \
        (TQ*)out, token_seq, token_pos, table, table_stride, nh, nkv, hd, scale, window, page_size, n_pages, status))
    if (q_dtype == IK_F32 && cache_dtype == IK_F32) IK_ATT(float, float);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_BF16) IK_ATT(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == IK_F32 && cache_dtype == IK_BF16) IK_ATT(float, __nv_bfloat16);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_F32) IK_ATT(__nv_bfloat16, float);
    else return IK_BAD_ARGUMENT;
#undef IK_ATT
    IK_LAUNCH_STATUS();
}
