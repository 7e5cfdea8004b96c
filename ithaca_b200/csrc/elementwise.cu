// Embedding gather, RMS norm, SwiGLU, and rotary position encoding fused with the
// append of keys and values into the paged cache.  Each kernel computes in float
// and converts only when it stores.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] * scale.  Ids are validated by the caller (host ids)
// or produced by the sampler (always in range); an id out of range sets *status
// and writes zeros instead of reading outside the table.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ out,
                             int d, int V, float scale, int* status) {
    ik_pdl_wait();
    IK_AFTER_WAIT(ids);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) ik_set_status(status, IK_STATUS_BAD_TOKEN);
    const TW* row = table + (size_t)(ok ? id : 0) * d;
    float* o = out + (size_t)t * d;
    // this block's slice of the row (a few tokens would otherwise keep a few SMs busy), four elements a thread
    const int per = ((d + gridDim.y - 1) / gridDim.y + 3) & ~3, lo = blockIdx.y * per, hi = min(d, lo + per);
    if ((d & 3) == 0 && ((uintptr_t)row % (4 * sizeof(TW))) == 0) {
        for (int i = lo + 4 * threadIdx.x; i < hi; i += 4 * blockDim.x) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ok) v = make_float4(ik_ld(row, i) * scale, ik_ld(row, i + 1) * scale, ik_ld(row, i + 2) * scale, ik_ld(row, i + 3) * scale);
            *reinterpret_cast<float4*>(o + i) = v;
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) o[i] = ok ? ik_ld(row, i) * scale : 0.f;
    }
}

IK_EXPORT int ik_embed(const int* ids, const void* table, int table_dtype, float* out, int T, int d, int V,
                       float scale, int* status, cudaStream_t stream) {
    if (T < 0 || d <= 0 || V <= 0) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    // few tokens (decode): a row is cut into slices so that the grid has a block for most SMs
    int slices = T >= 128 ? 1 : (128 + T - 1) / T;
    while (slices > 1 && d / slices < 256) slices--;
    if (T > 65535 * 32) return IK_BAD_ARGUMENT;
    const dim3 grid(T, slices);
    if (table_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(embed_kernel<float>, grid, 256, 0, stream, ids, (const float*)table, out, d, V, scale, status));
    else if (table_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(embed_kernel<__nv_bfloat16>, grid, 256, 0, stream, ids, (const __nv_bfloat16*)table, out, d, V, scale, status));
    else
        return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ RMS norm
// y = x * (1 / sqrt(mean(x^2) + eps)) * w, one block per output row.  rows_in selects
// input rows when given (the final norm runs only on the rows whose logits are wanted).
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows_in,
                               const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(rows_in);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* a = x + (size_t)(rows_in ? rows_in[r] : r) * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += 256) { float v = a[i]; ss = fmaf(v, v, ss); }
    ss = ik_block_sum<256>(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += 256) ik_st(o, i, a[i] * s * w[i]);
}

// The same for rows of up to 8192 elements, a multiple of 4: a thread keeps its up to 8 float4 of the row in
// registers (one pass over the row), and asks for its part of the weight, which no kernel writes, before it waits
// for the kernel that writes the row.
constexpr int RMS_VEC = 8;
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_row_in_registers_kernel(const float* __restrict__ x, const int* __restrict__ rows_in,
                                const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    const int n4 = d >> 2;
    float4 wv[RMS_VEC], xv[RMS_VEC];
    #pragma unroll
    for (int j = 0; j < RMS_VEC; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) wv[j] = __ldg(reinterpret_cast<const float4*>(w) + i);
    }
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(rows_in);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float4* a = reinterpret_cast<const float4*>(x + (size_t)(rows_in ? rows_in[r] : r) * d);
    float ss = 0.f;
    #pragma unroll
    for (int j = 0; j < RMS_VEC; j++) {
        const int i = threadIdx.x + j * 256;
        xv[j] = i < n4 ? a[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    #pragma unroll
    for (int j = 0; j < RMS_VEC; j++)
        ss = fmaf(xv[j].x, xv[j].x, fmaf(xv[j].y, xv[j].y, fmaf(xv[j].z, xv[j].z, fmaf(xv[j].w, xv[j].w, ss))));
    ss = ik_block_sum<256>(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
    #pragma unroll
    for (int j = 0; j < RMS_VEC; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4)
            ik_st4(o, (size_t)4 * i, make_float4(xv[j].x * s * wv[j].x, xv[j].y * s * wv[j].y, xv[j].z * s * wv[j].z, xv[j].w * s * wv[j].w));
    }
}

IK_EXPORT int ik_rmsnorm(const float* x, const int* rows_in, const float* w, void* out, int out_dtype, int rows,
                         int d, float eps, cudaStream_t stream) {
    if (rows < 0 || d <= 0) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    if (out_dtype != IK_F32 && out_dtype != IK_BF16) return IK_BAD_ARGUMENT;
    const bool in_registers = d % 4 == 0 && d <= 4 * 256 * RMS_VEC && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
                              ((uintptr_t)out % 16) == 0;
    if (in_registers && out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(rmsnorm_row_in_registers_kernel<float>, rows, 256, 0, stream, x, rows_in, w, (float*)out, d, eps));
    else if (in_registers)
        IK_RETURN_IF_ERROR(ik_launch(rmsnorm_row_in_registers_kernel<__nv_bfloat16>, rows, 256, 0, stream, x, rows_in, w, (__nv_bfloat16*)out, d, eps));
    else if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(rmsnorm_kernel<float>, rows, 256, 0, stream, x, rows_in, w, (float*)out, d, eps));
    else
        IK_RETURN_IF_ERROR(ik_launch(rmsnorm_kernel<__nv_bfloat16>, rows, 256, 0, stream, x, rows_in, w, (__nv_bfloat16*)out, d, eps));
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ SwiGLU
// in: [T, 2*ff] float; gate in columns [0, ff) and up in [ff, 2ff), or, interleaved, gate j in column
// 2j and up j in column 2j + 1.  out[t, j] = silu(g) * u.
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ out, int ff, size_t total, int interleaved) {
    ik_pdl_wait();
    IK_AFTER_WAIT(gu);
    ik_pdl_launch_dependents();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / ff;
        const int j = (int)(idx - t * ff);
        const float g = interleaved ? gu[t * 2 * ff + 2 * j] : gu[t * 2 * ff + j];
        const float u = interleaved ? gu[t * 2 * ff + 2 * j + 1] : gu[t * 2 * ff + ff + j];
        ik_st(out, idx, ik_swiglu(g, u));
    }
}

IK_EXPORT int ik_swiglu(const float* gate_up, void* out, int out_dtype, int T, int ff, int interleaved, cudaStream_t stream) {
    if (T < 0 || ff <= 0) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * ff;
    const int cap = ik_sm_count() * 16;
    const int blocks = (int)((total + 255) / 256 < (size_t)cap ? (total + 255) / 256 : (size_t)cap);
    if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(swiglu_kernel<float>, blocks, 256, 0, stream, gate_up, (float*)out, ff, total, interleaved));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, gate_up, (__nv_bfloat16*)out, ff, total, interleaved));
    else
        return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ rotary + cache append
// qkv: [T, (nh + 2 nkv) * hd] float, q heads first, then k heads, then v heads.
// One block per (token, group of heads): the token's cos/sin are computed once per block.  q heads are rotated and stored to q_out [T, nh*hd];
// k heads are rotated and stored into the token's place in the key pages; v heads are
// stored into the value pages.  A page holds page_size positions of every kv head:
// pages[page][kv_head][position in page][hd].  The page of position p of sequence s is
// table[s * table_stride + p / page_size].
//
// Angle = float(pos) * inv_freq[i] as a single float multiply; cosf/sinf are the accurate
// functions.  pairing 0 rotates (i, i + rot/2), pairing 1 rotates (2i, 2i + 1); dimensions
// from rot upward pass through.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
rope_append_kernel(const float* __restrict__ qkv, TQ* __restrict__ q_out, TC* __restrict__ k_pages,
                   TC* __restrict__ v_pages, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                   const int* __restrict__ table, int table_stride, const float* __restrict__ inv_freq, int nh, int nkv,
                   int hd, int rot, int pairing, int page_size, int n_pages, int write_cache, int heads_per_block,
                   int* status) {
    extern __shared__ __align__(16) float cs[];    // [rot/2] cos, then [rot/2] sin of this token's angles
    ik_pdl_wait();
    IK_AFTER_WAIT(qkv);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    IK_AFTER_WAIT(table);
    ik_pdl_launch_dependents();
    // threads: x runs over a head's elements, y over heads (no division in the loops)
    const int t = blockIdx.x, half = rot / 2, tid = threadIdx.y * blockDim.x + threadIdx.x;
    const int head_lo = blockIdx.y * heads_per_block;                          // over q heads, then k heads, then v heads
    const int head_hi = min(head_lo + heads_per_block, nh + 2 * nkv);
    const int pos = token_pos[t];
    if (head_lo < nh + nkv) {
        for (int i = tid; i < half; i += blockDim.x * blockDim.y) {
            const float ang = __fmul_rn((float)pos, inv_freq[i]);
            cs[i] = cosf(ang);
            cs[half + i] = sinf(ang);
        }
    }
    // where this token's keys and values go
    size_t page_off = 0;
    bool page_ok = false;
    if (write_cache && head_hi > nh) {
        const int page = table[(size_t)token_seq[t] * table_stride + pos / page_size];
        page_ok = page >= 0 && page < n_pages;
        if (!page_ok) { if (tid == 0) ik_set_status(status, IK_STATUS_WRITE_NO_PAGE); }               // never write outside the pool
        else page_off = ((size_t)page * nkv * page_size + (pos % page_size)) * hd;
    }
    __syncthreads();
    const float* src = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    // four pairs per thread where the layout allows 16-byte accesses (half-split pairs, widths in fours)
    const bool vec = pairing == 0 && (half & 3) == 0 && (hd & 3) == 0 && (((nh + 2 * nkv) * hd) & 3) == 0;
    for (int head = head_lo + threadIdx.y; head < head_hi; head += blockDim.y) {
        const float* hsrc = src + (size_t)head * hd;
        if (head < nh + nkv) {
            const bool is_q = head < nh;
            if (!is_q && !page_ok) continue;
            TQ* qdst = q_out + ((size_t)t * nh + head) * hd;
            TC* kdst = k_pages + page_off + (size_t)(head - nh) * page_size * hd;
            if (vec) {
                for (int i = 4 * threadIdx.x; i < half; i += 4 * blockDim.x) {
                    const float4 a = *reinterpret_cast<const float4*>(hsrc + i);
                    const float4 b = *reinterpret_cast<const float4*>(hsrc + half + i);
                    const float4 c = *reinterpret_cast<const float4*>(cs + i);
                    const float4 sn = *reinterpret_cast<const float4*>(cs + half + i);
                    float4 r0, r1;
                    r0.x = __fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, sn.x)); r1.x = __fadd_rn(__fmul_rn(a.x, sn.x), __fmul_rn(b.x, c.x));
                    r0.y = __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, sn.y)); r1.y = __fadd_rn(__fmul_rn(a.y, sn.y), __fmul_rn(b.y, c.y));
                    r0.z = __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, sn.z)); r1.z = __fadd_rn(__fmul_rn(a.z, sn.z), __fmul_rn(b.z, c.z));
                    r0.w = __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, sn.w)); r1.w = __fadd_rn(__fmul_rn(a.w, sn.w), __fmul_rn(b.w, c.w));
                    if (is_q) { ik_st4(qdst, i, r0); ik_st4(qdst, half + i, r1); }
                    else { ik_st4(kdst, i, r0); ik_st4(kdst, half + i, r1); }
                }
                for (int i = rot + 4 * threadIdx.x; i < hd; i += 4 * blockDim.x) {     // beyond the rotated width
                    const float4 v = *reinterpret_cast<const float4*>(hsrc + i);
                    if (is_q) ik_st4(qdst, i, v);
                    else ik_st4(kdst, i, v);
                }
                continue;
            }
            for (int i = threadIdx.x; i < half; i += blockDim.x) {                 // rotated pairs
                const int i0 = pairing == 0 ? i : 2 * i, i1 = pairing == 0 ? i + half : 2 * i + 1;
                const float c = cs[i], sn = cs[half + i];
                const float a = hsrc[i0], b = hsrc[i1];
                const float r0 = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
                const float r1 = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c));
                if (is_q) { ik_st(qdst, i0, r0); ik_st(qdst, i1, r1); }
                else { ik_st(kdst, i0, r0); ik_st(kdst, i1, r1); }
            }
            for (int i = rot + threadIdx.x; i < hd; i += blockDim.x) {              // beyond the rotated width
                if (is_q) ik_st(qdst, i, hsrc[i]);
                else ik_st(kdst, i, hsrc[i]);
            }
        } else if (page_ok) {                                                       // a value head: copied whole
            TC* vdst = v_pages + page_off + (size_t)(head - nh - nkv) * page_size * hd;
            if (vec) {
                for (int i = 4 * threadIdx.x; i < hd; i += 4 * blockDim.x) ik_st4(vdst, i, *reinterpret_cast<const float4*>(hsrc + i));
            } else {
                for (int i = threadIdx.x; i < hd; i += blockDim.x) ik_st(vdst, i, hsrc[i]);
            }
        }
    }
}

// cos_sin[t][i] = (cos, sin) of float(pos_t) * inv_freq_i: made once per step, used by every layer's fused
// q/k/v epilogue.
__global__ void rope_table_kernel(const int* __restrict__ token_pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_sin, int T, int half) {
    ik_pdl_wait();
    IK_AFTER_WAIT(token_pos);
    ik_pdl_launch_dependents();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    const float ang = __fmul_rn((float)token_pos[t], inv_freq[i]);
    cos_sin[2 * (size_t)idx] = cosf(ang);
    cos_sin[2 * (size_t)idx + 1] = sinf(ang);
}

IK_EXPORT int ik_rope_table(const int* token_pos, const float* inv_freq, float* cos_sin, int T, int half,
                            cudaStream_t stream) {
    if (T < 0 || half <= 0) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    IK_RETURN_IF_ERROR(ik_launch(rope_table_kernel, (T * half + 255) / 256, 256, 0, stream, token_pos, inv_freq, cos_sin, T, half));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_rope_append(const float* qkv, void* q_out, int q_dtype, void* k_pages, void* v_pages, int cache_dtype,
                             const int* token_seq, const int* token_pos, const int* table, int table_stride,
                             const float* inv_freq, int T, int nh, int nkv, int hd, int rot, int pairing,
                             int page_size, int n_pages, int write_cache, int* status, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return IK_BAD_ARGUMENT;
    if (rot > 0 && !inv_freq) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    // few tokens (decode): spread a token's heads over many blocks; many tokens: 16 heads a block
    const int hpb = T >= 256 ? 16 : 4;
    dim3 grid(T, (nh + 2 * nkv + hpb - 1) / hpb);
    const dim3 threads(32, 8);
    const size_t smem = (size_t)rot * sizeof(float);
#define IK_ROPE(TQ, TC)                                                                                             \
    IK_RETURN_IF_ERROR(ik_launch(rope_append_kernel<TQ, TC>, grid, threads, smem, stream, qkv, (TQ*)q_out, (TC*)k_pages, (TC*)v_pages, token_seq, \
        token_pos, table, table_stride, inv_freq, nh, nkv, hd, rot, pairing, page_size, n_pages, write_cache, hpb, status))
    if (q_dtype == IK_F32 && cache_dtype == IK_F32) IK_ROPE(float, float);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_BF16) IK_ROPE(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == IK_F32 && cache_dtype == IK_BF16) IK_ROPE(float, __nv_bfloat16);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_F32) IK_ROPE(__nv_bfloat16, float);
    else return IK_BAD_ARGUMENT;
#undef IK_ROPE
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ random weights
// out[i] = offset + scale * (sum of the eight 16-bit fields of two 64-bit hash words - 262140), i the flat index.
// The words are the outputs 2i+1 and 2i+2 of the splitmix64 sequence that starts at `key`.  The sum of eight
// uniform 16-bit integers is close to a normal law (Irwin-Hall, standard deviation 53510.85...) and is formed
// with integer arithmetic and one float multiply and add, so the host (numpy) and this kernel give the same
// bits: a model made on the device has exactly the weights a folder written on the host from the same
// configuration and seed holds.
__device__ __forceinline__ unsigned long long ik_mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename TO>
__global__ void fill_random_kernel(TO* __restrict__ out, size_t n, unsigned long long key, float scale, float offset) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int s = 0;
        #pragma unroll
        for (int j = 1; j <= 2; j++) {
            const unsigned long long h = ik_mix64(key + (2ull * i + j) * 0x9E3779B97F4A7C15ull);
            s += (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)(h >> 48);
        }
        ik_st(out, i, __fadd_rn(offset, __fmul_rn(scale, (float)(s - 262140))));
    }
}

IK_EXPORT int ik_fill_random(void* out, int out_dtype, unsigned long long n, unsigned long long key, float scale, float offset,
                             cudaStream_t stream) {
    if (n == 0) return IK_OK;
    const unsigned long long cap = (unsigned long long)ik_sm_count() * 16;
    const int blocks = (int)((n + 1023) / 1024 < cap ? (n + 1023) / 1024 : cap);
    if (out_dtype == IK_F32) fill_random_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (size_t)n, key, scale, offset);
    else if (out_dtype == IK_BF16) fill_random_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (size_t)n, key, scale, offset);
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}

// Streaming multiprocessors of the current device, for the host side's choices of splits and chunks.
IK_EXPORT int ik_device_sm_count() { return ik_sm_count(); }

// ------------------------------------------------------------------ copy
// dst[i] = src[i] over n 16-byte words: the plain streaming copy that the bandwidth figure of the peaks'
// self-measurement stands on (read + write bytes over its time).
__global__ void __launch_bounds__(256) copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n) {
    constexpr int U = 8;                                   // 128 bytes a thread in flight
    const size_t stride = (size_t)gridDim.x * blockDim.x * U;
    for (size_t i = (size_t)blockIdx.x * blockDim.x * U + threadIdx.x; i < n; i += stride) {
        uint4 v[U];
        #pragma unroll
        for (int j = 0; j < U; j++) if (i + (size_t)j * blockDim.x < n) v[j] = __ldcs(src + i + (size_t)j * blockDim.x);
        #pragma unroll
        for (int j = 0; j < U; j++) if (i + (size_t)j * blockDim.x < n) __stcs(dst + i + (size_t)j * blockDim.x, v[j]);
    }
}

IK_EXPORT int ik_copy(const void* src, void* dst, unsigned long long bytes, cudaStream_t stream) {
    if (bytes % 16 || ((uintptr_t)src % 16) || ((uintptr_t)dst % 16)) return IK_BAD_ARGUMENT;
    if (bytes == 0) return IK_OK;
    const size_t n = bytes / 16;
    const size_t want = (n + 2047) / 2048, cap = (size_t)ik_sm_count() * 8;
    copy_kernel<<<(int)(want < cap ? want : cap), 256, 0, stream>>>((const uint4*)src, (uint4*)dst, n);
    IK_LAUNCH_STATUS();
}
