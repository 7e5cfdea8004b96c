// Plain matrix product on the CUDA cores: Y[M, N] (+)= X[M, K] * W[N, K]^T.
//
// This is the 32-bit path's product and the fallback for shapes the tensor-core kernels
// refuse.  Operands are converted to float when loaded; every output element is one
// float accumulator that adds its K products in ascending k, whatever M and N are, so a
// row of Y does not depend on which other rows are in the call.  No split along K, no
// atomics, no reduced-precision matrix mode.
#define IK_FAMILY 2
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ X, const TW* __restrict__ W, TY* __restrict__ Y, int M, int N, int K,
                 int ldx, int ldw, int ldy, int accumulate) {
    ik_pdl_wait();
    IK_AFTER_WAIT(X);                 // the tokens are the kernel before's results; this kernel takes no weight early
    ik_pdl_launch_dependents();
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // tx -> n, ty -> m
    float acc[TM][TN];
    #pragma unroll
    for (int i = 0; i < TM; i++)
        #pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 4 per thread
        #pragma unroll
        for (int l = 0; l < 4; l++) {
            const int idx = threadIdx.x + l * 256;
            const int r = idx / BK, c = idx % BK;
            const int k = k0 + c;
            xs[c][r] = (m0 + r < M && k < K) ? ik_ld(X, (size_t)(m0 + r) * ldx + k) : 0.f;
            ws[c][r] = (n0 + r < N && k < K) ? ik_ld(W, (size_t)(n0 + r) * ldw + k) : 0.f;
        }
        __syncthreads();
        #pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], b[TN];
            #pragma unroll
            for (int i = 0; i < TM; i++) a[i] = xs[kk][ty * TM + i];
            #pragma unroll
            for (int j = 0; j < TN; j++) b[j] = ws[kk][tx + 16 * j];
            #pragma unroll
            for (int i = 0; i < TM; i++)
                #pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    #pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        #pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            const size_t o = (size_t)m * ldy + n;
            float v = acc[i][j];
            if (accumulate) v += ik_ld(Y, o);
            ik_st(Y, o, v);
        }
    }
}

template <typename TX, typename TW, typename TY>
int launch(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy, int accumulate,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    IK_RETURN_IF_ERROR(ik_launch(gemm_simt_kernel<TX, TW, TY>, grid, 256, 0, stream, (const TX*)X, (const TW*)W, (TY*)Y, M, N, K, ldx, ldw, ldy,
                                                            accumulate));
    IK_LAUNCH_STATUS();
}

}  // namespace

// Padding zeros in K contribute exact zeros, and a k beyond K is never added to a real
// product's partial sum out of order: the accumulation order of the real terms is 0..K-1.
IK_EXPORT int ik_gemm_simt(const void* X, int x_dtype, const void* W, int w_dtype, void* Y, int y_dtype, int M, int N,
                           int K, int ldx, int ldw, int ldy, int accumulate, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return IK_BAD_ARGUMENT;
    if (M == 0) return IK_OK;
    const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
    switch (code) {
        case 0: return launch<float, float, float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 1: return launch<float, float, __nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 2: return launch<float, __nv_bfloat16, float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 3: return launch<float, __nv_bfloat16, __nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 4: return launch<__nv_bfloat16, float, float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 5: return launch<__nv_bfloat16, float, __nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 6: return launch<__nv_bfloat16, __nv_bfloat16, float>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        case 7: return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(X, W, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
    }
    return IK_BAD_ARGUMENT;
}
