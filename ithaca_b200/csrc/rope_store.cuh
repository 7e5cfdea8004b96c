// The epilogue that turns the fused q/k/v product straight into rotated queries and cache entries.
//
// The product's output features are the q heads, then the k heads, then the v heads, head_dim each.  Inside a q
// or k head the features come in rotary pairs: (2i, 2i + 1) are the two members of pair i (a model whose pairs
// are (i, i + head_dim / 2) has the rows of its q and k weights reordered when it is loaded; scores do not
// change, since q and k are reordered alike).  For token m and pair i the cosine and sine of
// float(pos_m) * inv_freq_i come from a table made once per step.  Rotated q goes to q_out, rotated k and plain
// v go to the token's place in the paged cache; the [tokens, features] intermediate is never written.
#pragma once
#include "common.cuh"

struct IkRopeStore {
    __nv_bfloat16* q_out;          // [M, nh * hd]; null = this epilogue is off
    __nv_bfloat16* k_pages;        // [pages][nkv][page_size][hd]
    __nv_bfloat16* v_pages;
    const float* cos_sin;          // [M][hd / 2][2]
    const int* token_seq;          // [M] index of the token's sequence in the step
    const int* token_pos;          // [M] absolute position
    const int* table;              // block table [sequences][table_stride]
    int* status;
    int table_stride, nh, nkv, hd, page_size, n_pages, write_cache;
};

// Where token m's keys and values go in a layer's pages, as a row of head_dim elements for kv head 0 (head h lies
// h * page_size rows further), or -1 if nothing is to be written for it.
__device__ __forceinline__ int ik_rope_cache_row(const IkRopeStore& e, int m, int M) {
    if (m >= M || !e.write_cache) return -1;
    const int pos = e.token_pos[m];
    const int page = e.table[(size_t)e.token_seq[m] * e.table_stride + pos / e.page_size];
    if (page < 0 || page >= e.n_pages) {              // never write outside the pool
        ik_set_status(e.status, IK_STATUS_WRITE_NO_PAGE);
        return -1;
    }
    return page * e.nkv * e.page_size + pos % e.page_size;
}

// (a, b): the product's values at features (f0, f0 + 1) of token m, f0 even.
__device__ __forceinline__ void ik_rope_store_pair(const IkRopeStore& e, int m, int f0, float a, float b) {
    const int head = f0 / e.hd, r0 = f0 - head * e.hd;
    float o0 = a, o1 = b;
    if (head < e.nh + e.nkv) {
        const float2 cs = *reinterpret_cast<const float2*>(e.cos_sin + ((size_t)m * (e.hd >> 1) + (r0 >> 1)) * 2);
        o0 = a * cs.x - b * cs.y;
        o1 = a * cs.y + b * cs.x;
    }
    const __nv_bfloat162 packed = __floats2bfloat162_rn(o0, o1);
    if (head < e.nh) {
        *reinterpret_cast<__nv_bfloat162*>(e.q_out + ((size_t)m * e.nh + head) * e.hd + r0) = packed;
        return;
    }
    if (!e.write_cache) return;
    const int pos = e.token_pos[m];
    const int page = e.table[(size_t)e.token_seq[m] * e.table_stride + pos / e.page_size];
    if (page < 0 || page >= e.n_pages) {              // never write outside the pool
        ik_set_status(e.status, IK_STATUS_WRITE_NO_PAGE);
        return;
    }
    const bool is_k = head < e.nh + e.nkv;
    const int kvh = is_k ? head - e.nh : head - e.nh - e.nkv;
    __nv_bfloat16* dst = (is_k ? e.k_pages : e.v_pages) +
                         (((size_t)page * e.nkv + kvh) * e.page_size + (pos % e.page_size)) * e.hd + r0;
    *reinterpret_cast<__nv_bfloat162*>(dst) = packed;
}
