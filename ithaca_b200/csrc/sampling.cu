// Sampling on the device: one block per row of logits.
//
// The rule is the reference's (src/chat.cpp:124-145): each recent id is penalised
// (l > 0 ? l / pen : l * pen, once per occurrence); temperature <= 0 takes the largest
// logit; otherwise the k = clamp(top_k, 1, V) largest are kept, weighted
// exp((l - max) / temperature), and of those the shortest prefix in descending order whose
// share of the weight reaches top_p (the crossing one included).  One of the kept is
// drawn with a uniform number.  Two things are this library's own: the uniform comes from
// Philox-4x32-10 keyed by (seed) with counter (step, stream), so a sequence's draws do not
// depend on what else is in the batch; and the kept candidates are walked in vocabulary
// order (the same law as the reference's descending walk, without a sort).  Equal logits
// are ordered by ascending id.  No sort is done anywhere: the k-th largest value and the
// top_p boundary are found by bisection over the bits of an order-preserving integer key.
#include <math.h>
#define IK_FAMILY 16
#include "common.cuh"

namespace {

constexpr int ST = 1024;

__device__ __forceinline__ uint32_t okey(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unkey(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t stream, uint32_t counter) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    uint32_t c0 = counter, c1 = stream, c2 = 0, c3 = 0;
    #pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t h0 = __umulhi(M0, c0), l0 = M0 * c0, h1 = __umulhi(M1, c2), l1 = M1 * c2;
        const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
        c0 = n0; c1 = l1; c2 = n2; c3 = l0;
        k0 += W0; k1 += W1;
    }
    return ((float)(c0 >> 8) + 0.5f) * (1.0f / 16777216.0f);   // 24 bits: exact in float, inside (0, 1)
}

// Inclusive block scan (fixed order): lanes by shuffle, then the warp totals.
template <typename T>
__device__ __forceinline__ T block_scan_inclusive(T v, T* warp_tot /* [32] */, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    T before = 0, all = 0;
    #pragma unroll
    for (int w = 0; w < ST / 32; w++) { const T x = warp_tot[w]; if (w < warp) before += x; all += x; }
    *total = all;
    return v + before;
}

struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) {      // larger value, then smaller index
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ Best block_argmax(const float* w, int V, Best* sh /* [32] */) {
    Best b{-INFINITY, 0x7fffffff};
    #pragma unroll 8
    for (int i = threadIdx.x; i < V; i += ST) b = better(b, Best{w[i], i});
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best n{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, n);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = b;
    __syncthreads();
    Best r = sh[0];
    for (int wv = 1; wv < ST / 32; wv++) r = better(r, sh[wv]);
    return r;
}

__global__ void __launch_bounds__(ST)
argmax_kernel(const float* __restrict__ logits, int ldl, int* __restrict__ out, int V) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    __shared__ Best sh[32];
    const Best b = block_argmax(logits + (size_t)blockIdx.x * ldl, V, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// The same with a row cut into ARG_SPLITS slices, one block each (a handful of rows would otherwise keep a
// handful of SMs busy).  A slice's block leaves its best in scratch; the block that arrives last merges the
// slices in slice order (so the result does not depend on which block that is) and clears the row's counter.
// The scratch (a counter per row, then a best per row and slice) belongs to the caller: IK_ARGMAX_SCRATCH_BYTES,
// zeroed once; every launch leaves the counters zero.  Launches that share a scratch must follow one another in
// one stream, so a caller with several streams keeps one per stream.
constexpr int ARG_SPLITS = 16, ARG_MAX_ROWS = 256;
constexpr size_t IK_ARGMAX_SCRATCH_BYTES = ARG_MAX_ROWS * sizeof(unsigned int) + (size_t)ARG_MAX_ROWS * ARG_SPLITS * sizeof(Best);

__global__ void __launch_bounds__(ST)
argmax_split_kernel(const float* __restrict__ logits, int ldl, int* __restrict__ out, int V, unsigned int* g_arg_count) {
    Best* const g_arg_part = reinterpret_cast<Best*>(g_arg_count + ARG_MAX_ROWS);
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    __shared__ Best sh[32];
    __shared__ bool last;
    const int row = blockIdx.y, split = blockIdx.x;
    const int per = (V + ARG_SPLITS - 1) / ARG_SPLITS, lo = split * per, hi = min(V, lo + per);
    const float* w = logits + (size_t)row * ldl;
    Best b{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += ST) b = better(b, Best{w[i], i});
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best n{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, n);
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        Best r = sh[0];
        for (int wv = 1; wv < ST / 32; wv++) r = better(r, sh[wv]);
        g_arg_part[row * ARG_SPLITS + split] = r;
        __threadfence();
        last = atomicAdd(&g_arg_count[row], 1u) == ARG_SPLITS - 1;
        if (last) {
            __threadfence();
            const volatile Best* parts = g_arg_part + row * ARG_SPLITS;       // written by other blocks: read from L2
            Best all{parts[0].v, parts[0].i};
            for (int sp = 1; sp < ARG_SPLITS; sp++) all = better(all, Best{parts[sp].v, parts[sp].i});
            out[row] = all.i;
            g_arg_count[row] = 0;
        }
    }
}

// ---- The usual case, k <= 1024 kept candidates (top_k = 40 by default): the k-th largest key is found four bits
// at a time (8 counting passes over the row instead of 32), the k survivors are gathered into shared memory, and
// top-p and the draw run on those alone, one candidate per thread, in vocabulary order.  The rule is the one
// described at the top of this file; equal keys at the boundary are taken by ascending id.  Returns false, having
// written nothing, when more than 1024 candidates tie with the k-th largest (the general path then runs).
constexpr int CAND_CAP = 1024;

__device__ bool sample_few(const float* w, int V, int k, float top_p, float inv_t, float mx, uint64_t seed, uint32_t stream,
                           uint32_t counter, int* out, float* shf /* [32] */, int* shi /* [32] */) {
    __shared__ int cnt_warp[32][16];
    __shared__ int cnt_tot[16];
    __shared__ int cand_i[CAND_CAP], tie_i[CAND_CAP], sort_i[CAND_CAP];
    __shared__ float cand_v[CAND_CAP], sort_v[CAND_CAP], sort_w[CAND_CAP];
    __shared__ int n_gt_sh, n_tie_sh, chosen, last_kept;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // First try (two passes over the row): every thread's own largest key; the k-th largest of those 1024 keys is a
    // lower bound of the k-th largest of the row, and with a few dozen candidates wanted out of a hundred thousand
    // hardly more than k entries lie at or above it.  They are gathered and the k largest of them (lower id first
    // among equals) picked exactly by counting.  If more than 1024 lie above the bound, the digit passes below run.
    __shared__ uint32_t tmax[ST];
    __shared__ uint32_t tau_sh;
    __shared__ int n_above_sh;
    bool gathered = false;
    {
        uint32_t mk = 0u;
        #pragma unroll 8
        for (int i = tid; i < V; i += ST) mk = max(mk, okey(w[i]));
        tmax[tid] = mk;
        if (tid == 0) n_above_sh = 0;
        __syncthreads();
        int rank = 0;
        for (int j = 0; j < ST; j++) rank += tmax[j] > mk || (tmax[j] == mk && j < tid);
        if (rank == k - 1) tau_sh = mk;                    // k <= 1024: exactly one thread
        __syncthreads();
        const uint32_t tau = tau_sh;
        #pragma unroll 8
        for (int i = tid; i < V; i += ST) {
            const float v = w[i];
            if (okey(v) >= tau) {
                const int slot = atomicAdd(&n_above_sh, 1);
                if (slot < CAND_CAP) { tie_i[slot] = i; sort_v[slot] = v; }       // (borrowed as scratch until the sort)
            }
        }
        __syncthreads();
        const int c = n_above_sh;
        if (c <= CAND_CAP) {
            if (tid < c) {
                const uint32_t key = okey(sort_v[tid]);
                const int me = tie_i[tid];
                int r = 0;
                for (int j = 0; j < c; j++) {
                    const uint32_t kj = okey(sort_v[j]);
                    r += kj > key || (kj == key && tie_i[j] < me);
                }
                if (r < k) { cand_i[r] = me; cand_v[r] = sort_v[tid]; }
            }
            gathered = true;
        }
        __syncthreads();
    }

    // Otherwise the key T of the k-th largest: digit by digit from the top; `need` of the candidates that share the
    // prefix found so far are still to be taken
    uint32_t prefix = 0;
    int need = k;
    for (int shift = gathered ? -1 : 28; shift >= 0; shift -= 4) {
        const uint32_t above = shift == 28 ? 0u : (0xFFFFFFFFu << (shift + 4));
        int c[16];
        #pragma unroll
        for (int d = 0; d < 16; d++) c[d] = 0;
        for (int base = tid; base < V; base += ST * 255) {          // 8-bit fields: flushed every 255 elements
            unsigned long long lo8 = 0ull, hi8 = 0ull;
            const int end = min(V, base + ST * 255);
            for (int i0 = base; i0 < end; i0 += ST * 8) {           // eight loads under way per thread
                float v8[8];
                #pragma unroll
                for (int j = 0; j < 8; j++) v8[j] = i0 + j * ST < end ? w[i0 + j * ST] : 0.f;
                #pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t key = okey(v8[j]);
                    if (i0 + j * ST < end && (key & above) == prefix) {
                        const uint32_t d = (key >> shift) & 15u;
                        const unsigned long long one = 1ull << ((d & 7u) * 8u);
                        if (d < 8u) lo8 += one; else hi8 += one;
                    }
                }
            }
            #pragma unroll
            for (int d = 0; d < 8; d++) {
                c[d] += (int)((lo8 >> (d * 8)) & 0xFFull);
                c[d + 8] += (int)((hi8 >> (d * 8)) & 0xFFull);
            }
        }
        #pragma unroll
        for (int d = 0; d < 16; d++) {
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) c[d] += __shfl_xor_sync(0xffffffffu, c[d], o);
        }
        if (lane == 0) {
            #pragma unroll
            for (int d = 0; d < 16; d++) cnt_warp[warp][d] = c[d];
        }
        __syncthreads();
        if (tid < 16) {
            int t = 0;
            for (int wv = 0; wv < ST / 32; wv++) t += cnt_warp[wv][tid];
            cnt_tot[tid] = t;
        }
        __syncthreads();
        int digit = 0;
        for (int d = 15; d >= 0; d--) {
            const int n = cnt_tot[d];
            if (n >= need) { digit = d; break; }
            need -= n;
        }
        prefix |= (uint32_t)digit << shift;
        __syncthreads();                                   // cnt_tot is rewritten by the next pass
    }
    const uint32_t T = prefix;                              // `need` of the candidates with key == T are taken

    // gather: everything above T, and the ties at T apart
    if (tid == 0) { n_gt_sh = 0; n_tie_sh = 0; chosen = ST; last_kept = -1; }
    __syncthreads();
    #pragma unroll 8
    for (int i = gathered ? V : tid; i < V; i += ST) {
        const float v = w[i];
        const uint32_t key = okey(v);
        if (key > T) {
            const int slot = atomicAdd(&n_gt_sh, 1);
            cand_i[slot] = i; cand_v[slot] = v;
        } else if (key == T) {
            const int slot = atomicAdd(&n_tie_sh, 1);
            if (slot < CAND_CAP) tie_i[slot] = i;
        }
    }
    __syncthreads();
    const int n_gt = gathered ? k : n_gt_sh, n_tie = gathered ? 0 : n_tie_sh;
    if (gathered) need = 0;
    if (n_tie > CAND_CAP) return false;
    // the `need` ties with the lowest ids join, in id order
    if (tid < n_tie) {
        const int me = tie_i[tid];
        int rank = 0;
        for (int j = 0; j < n_tie; j++) rank += tie_i[j] < me;
        if (rank < need) { cand_i[n_gt + rank] = me; cand_v[n_gt + rank] = unkey(T); }
    }
    __syncthreads();
    const int n = n_gt + need;                              // == k
    // into vocabulary order (the gather above came in whatever order the atomics fell)
    if (tid < n) {
        const int me = cand_i[tid];
        int pos = 0;
        for (int j = 0; j < n; j++) pos += cand_i[j] < me;
        sort_i[pos] = me; sort_v[pos] = cand_v[tid];
    }
    __syncthreads();
    const float v = tid < n ? sort_v[tid] : 0.f;
    const uint32_t key = okey(v);
    const float wgt = tid < n ? expf((v - mx) * inv_t) : 0.f;
    if (tid < n) sort_w[tid] = wgt;
    float total;
    block_scan_inclusive<float>(wgt, shf, &total);          // (syncs: sort_w is visible afterwards)
    bool kept = tid < n;
    if (top_p < 1.0f && kept) {
        // the weight in front of this candidate in descending order (larger key, or equal key and lower id)
        const float target = top_p * total;
        float before = 0.f;
        for (int j = 0; j < n; j++) {
            const uint32_t kj = okey(sort_v[j]);
            if (kj > key || (kj == key && j < tid)) before += sort_w[j];
        }
        kept = before < target;
    }
    const float mine = kept ? wgt : 0.f;
    float kept_total;
    const float incl = block_scan_inclusive<float>(mine, shf, &kept_total);
    const float u = philox_uniform(seed, stream, counter);
    const float r = fminf(u * kept_total, kept_total);
    if (mine > 0.f) { atomicMax(&last_kept, tid); if (r <= incl) atomicMin(&chosen, tid); }
    __syncthreads();
    if (tid == 0) {
        const int pick = chosen < ST ? chosen : last_kept;
        *out = pick >= 0 ? sort_i[pick] : sort_i[0];
    }
    (void)shi;
    return true;
}

struct Keep {                 // which candidates survive top-k and top-p
    uint32_t tk; int need_k;  // key of the k-th largest; how many of the ties at tk are kept
    uint32_t tp; int need_p;  // key at the top-p boundary; how many of the ties at tp are kept
    bool use_p;
};

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, int ldl, float* __restrict__ work, int* __restrict__ out, int V,
              float temperature, int top_k, float top_p, float rep_pen, const int* __restrict__ recent, int n_recent,
              uint64_t seed, const int* __restrict__ streams, const int* __restrict__ counters) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    __shared__ Best shb[32];
    __shared__ float shf[32];
    __shared__ int shi[32];
    __shared__ int chosen_thread;
    __shared__ int last_thread;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * ldl;
    float* w = work + (size_t)row * V;

    #pragma unroll 8
    for (int i = tid; i < V; i += ST) w[i] = l[i];
    __syncthreads();
    if (rep_pen != 1.0f && tid == 0) {
        for (int n = 0; n < n_recent; n++) {
            const int id = recent[(size_t)row * n_recent + n];
            if (id >= 0 && id < V) { const float v = w[id]; w[id] = v > 0.f ? v / rep_pen : v * rep_pen; }
        }
    }
    __syncthreads();
    const Best top = block_argmax(w, V, shb);
    if (temperature <= 0.f) { if (tid == 0) out[row] = top.i; return; }

    const int k = min(V, max(1, top_k));
    const float inv_t = 1.0f / temperature, mx = top.v;
    if (k <= CAND_CAP &&
        sample_few(w, V, k, top_p, inv_t, mx, seed, (uint32_t)streams[row], (uint32_t)counters[row], out + row, shf, shi))
        return;
    const int per = (V + ST - 1) / ST, lo = min(V, tid * per), hi = min(V, lo + per);
    Keep kp{0u, V, 0u, V, false};

    // ---- top-k: the largest key T with count{key >= T} >= k
    if (k < V) {
        uint32_t T = 0;
        for (int b = 31; b >= 0; b--) {
            const uint32_t cand = T | (1u << b);
            int c = 0;
            for (int i = tid; i < V; i += ST) c += okey(w[i]) >= cand;
            int tot; block_scan_inclusive<int>(c, shi, &tot);
            if (tot >= k) T = cand;
        }
        int c = 0;
        for (int i = tid; i < V; i += ST) c += okey(w[i]) > T;
        int n_gt; block_scan_inclusive<int>(c, shi, &n_gt);
        kp.tk = T; kp.need_k = k - n_gt;
    }
    // rank of this thread's first tie at tk among all ties at tk, in id order
    int tie_k_before;
    {
        int c = 0;
        for (int i = lo; i < hi; i++) c += okey(w[i]) == kp.tk;
        int tot; tie_k_before = block_scan_inclusive<int>(c, shi, &tot) - c;
    }
    int tie_p_before = 0;

    // mass of the kept candidates with key >= bound (bound_incl) or > bound, summed in id order per thread
    auto kept_mass = [&](uint32_t bound, bool strict, const Keep& kk, int tkb, int tpb) {
        float s = 0.f; int rk = tkb, rp = tpb;
        for (int i = lo; i < hi; i++) {
            const uint32_t key = okey(w[i]);
            bool in = key > kk.tk || (key == kk.tk && rk < kk.need_k);
            if (key == kk.tk) rk++;
            if (kk.use_p) { in = in && (key > kk.tp || (key == kk.tp && rp < kk.need_p)); if (key == kk.tp) rp++; }
            if (in && (strict ? key > bound : key >= bound)) s += expf((w[i] - mx) * inv_t);
        }
        return s;
    };

    // ---- top-p over the top-k survivors
    if (top_p < 1.0f) {
        float total; block_scan_inclusive<float>(kept_mass(0u, false, kp, tie_k_before, 0), shf, &total);
        const float target = top_p * total;
        uint32_t T = 0;
        for (int b = 31; b >= 0; b--) {
            const uint32_t cand = T | (1u << b);
            float m; block_scan_inclusive<float>(kept_mass(cand, false, kp, tie_k_before, 0), shf, &m);
            if (m >= target) T = cand;
        }
        float mass_gt; block_scan_inclusive<float>(kept_mass(T, true, kp, tie_k_before, 0), shf, &mass_gt);
        int c = 0;
        { int rk = tie_k_before;
          for (int i = lo; i < hi; i++) { const uint32_t key = okey(w[i]);
              const bool in = key > kp.tk || (key == kp.tk && rk < kp.need_k);
              if (key == kp.tk) rk++;
              c += in && key == T; } }
        int ties; block_scan_inclusive<int>(c, shi, &ties);
        const float wt = expf((unkey(T) - mx) * inv_t);
        int n = 1;
        if (ties > 1 && wt > 0.f) {
            n = (int)fminf((float)ties, fmaxf(1.f, ceilf((target - mass_gt) / wt)));
            while (n > 1 && mass_gt + (float)(n - 1) * wt >= target) n--;
            while (n < ties && mass_gt + (float)n * wt < target) n++;
        }
        int c2 = 0;
        for (int i = lo; i < hi; i++) c2 += okey(w[i]) == T;
        int tot2; tie_p_before = block_scan_inclusive<int>(c2, shi, &tot2) - c2;
        kp.tp = T; kp.need_p = n; kp.use_p = true;
    }

    // ---- draw in vocabulary order
    const float mine = kept_mass(0u, false, kp, tie_k_before, tie_p_before);
    float total;
    const float incl = block_scan_inclusive<float>(mine, shf, &total);
    const float u = philox_uniform(seed, (uint32_t)streams[row], (uint32_t)counters[row]);
    const float r = fminf(u * total, total);
    if (tid == 0) { chosen_thread = ST; last_thread = -1; }
    __syncthreads();
    if (mine > 0.f) { atomicMax(&last_thread, tid); if (r <= incl) atomicMin(&chosen_thread, tid); }
    __syncthreads();
    // the first thread whose running sum reaches r; if rounding left nobody, the last thread that kept anything
    const int owner = chosen_thread < ST ? chosen_thread : last_thread;
    if (tid == owner) {
        float acc = incl - mine; int rk = tie_k_before, rp = tie_p_before, pick = -1, last = -1;
        for (int i = lo; i < hi; i++) {
            const uint32_t key = okey(w[i]);
            bool in = key > kp.tk || (key == kp.tk && rk < kp.need_k);
            if (key == kp.tk) rk++;
            if (kp.use_p) { in = in && (key > kp.tp || (key == kp.tp && rp < kp.need_p)); if (key == kp.tp) rp++; }
            if (!in) continue;
            last = i;
            acc += expf((w[i] - mx) * inv_t);
            if (r <= acc) { pick = i; break; }
        }
        out[row] = pick >= 0 ? pick : (last >= 0 ? last : top.i);
    }
}

}  // namespace

IK_EXPORT int ik_argmax_scratch_bytes() { return (int)IK_ARGMAX_SCRATCH_BYTES; }

// scratch: ik_argmax_scratch_bytes() of device memory, zeroed once by the caller and used by one stream at a time;
// without it (null) every row is searched by one block.
IK_EXPORT int ik_argmax(const float* logits, int ldl, int* out, int rows, int V, void* scratch, cudaStream_t stream) {
    if (rows < 0 || V <= 0 || ldl < V) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    if (scratch && rows <= ARG_MAX_ROWS && rows * ARG_SPLITS <= 1024 && V >= 16 * ST)
        IK_RETURN_IF_ERROR(ik_launch(argmax_split_kernel, dim3(ARG_SPLITS, rows), ST, 0, stream, logits, ldl, out, V,
                                     (unsigned int*)scratch));
    else
        IK_RETURN_IF_ERROR(ik_launch(argmax_kernel, rows, ST, 0, stream, logits, ldl, out, V));
    IK_LAUNCH_STATUS();
}

// work: [rows, V] floats of scratch owned by the caller.  recent: [rows, n_recent] ids, -1 = empty.
IK_EXPORT int ik_sample(const float* logits, int ldl, float* work, int* out, int rows, int V, float temperature,
                        int top_k, float top_p, float rep_pen, const int* recent, int n_recent,
                        unsigned long long seed, const int* streams, const int* counters, cudaStream_t stream) {
    if (rows < 0 || V <= 0 || ldl < V || n_recent < 0 || !(rep_pen > 0.f) || !(top_p > 0.f)) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    IK_RETURN_IF_ERROR(ik_launch(sample_kernel, rows, ST, 0, stream, logits, ldl, work, out, V, temperature, top_k, top_p, rep_pen, recent,
                                           n_recent, (uint64_t)seed, streams, counters));
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// The variant that allocates nothing (see sampling_static.h for who needs it and its rules).
#include <stdio.h>
#include <mutex>
#include "sampling_static.h"

namespace {

// The scratch of ik_sample_static.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_work[IK_SAMPLE_STATIC_MAX_FLOATS];

constexpr int STATIC_MAX_DEVICES = 64;
float* g_static_work_addr[STATIC_MAX_DEVICES];      // per device: the array's address there, null until looked up
std::mutex g_static_mutex;

// The device address of g_static_work on the current device (looked up once per device).
int static_work_address(float** addr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return IK_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_work_addr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_work);
        if (e != cudaSuccess) return (int)e;
        if (!p) return IK_BAD_ARGUMENT;
        g_static_work_addr[dev] = p;
    }
    *addr = g_static_work_addr[dev];
    return IK_OK;
}

}  // namespace

IK_EXPORT int ik_sample_static(const float* logits, int ldl, int* out, int rows, int V, float temperature, int top_k,
                               float top_p, float rep_pen, const int* recent, int n_recent, unsigned long long seed,
                               const int* streams, const int* counters, cudaStream_t stream) {
    if (rows < 0 || V <= 0 || ldl < V || n_recent < 0 || !(rep_pen > 0.f) || !(top_p > 0.f)) return IK_BAD_ARGUMENT;
    if ((long long)rows * V > (long long)IK_SAMPLE_STATIC_MAX_FLOATS) {
        fprintf(stderr, "ik_sample_static: %d rows x %d logits = %lld floats of scratch, the static array holds %d; "
                        "use ik_sample with scratch of your own\n", rows, V, (long long)rows * V,
                IK_SAMPLE_STATIC_MAX_FLOATS);
        return IK_SAMPLE_STATIC_TOO_LARGE;
    }
    if (rows == 0) return IK_OK;
    float* work = nullptr;
    const int st = static_work_address(&work);
    if (st != IK_OK) return st;
    // sample_kernel copies each row's logits into `work` before it reads it: stale contents never show
    IK_RETURN_IF_ERROR(ik_launch(sample_kernel, rows, ST, 0, stream, logits, ldl, work, out, V, temperature, top_k, top_p, rep_pen, recent,
                                           n_recent, (uint64_t)seed, streams, counters));
    IK_LAUNCH_STATUS();
}
