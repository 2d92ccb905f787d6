// C[M, N] = act(A[M, K] . W[N, K]^T + bias[N]) (+ residual[M, N]) on CUDA cores.
//
// This is the true 32-bit matrix product of the library (float32 operands,
// float32 FMA, no tensor cores and no reduced-precision mode) and also the
// any-shape fallback of the bfloat16 path.  Every output element is one
// running sum over k = 0..K-1 in order, whatever M is and wherever the row
// lies in the batch, so a row's result does not depend on what else is in the
// step.  The reference's counterpart is `apply` over matmulNT/matmulTiled
// (include/ai/LocalModel.hpp:1052-1126; include/ai/Kernels.hpp:184-207, 315-430).
#include "common.cuh"

namespace mu {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16, SG_THREADS = 256;

template <typename TA, typename TC>
__global__ void __launch_bounds__(SG_THREADS)
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
                 const float* residual, TC* C, int M, int N, int K,
                 long long lda, long long ldw, long long ldc, long long ldr, int act) {
    __shared__ float As[SG_BK][SG_BM + 4];
    __shared__ float Ws[SG_BK][SG_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // each thread loads 4 elements of A and 4 of W per k-block: row = tid / 4, k = (tid % 4) * 4 ..
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + i][lr] = (am < M && k < K) ? to_float(A[(long long)am * lda + k]) : 0.0f;
            Ws[lk + i][lr] = (wn < N && k < K) ? to_float(W[(long long)wn * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = apply_act(v, act);
            if (residual) v += residual[(long long)m * ldr + n];
            C[(long long)m * ldc + n] = from_float<TC>(v);
        }
    }
}

}  // namespace mu

// in_bf16: A and W hold bfloat16 (else float32); out_bf16: C holds bfloat16 (else float32).
// residual (float32, leading dimension ldr) may be C itself when C is float32.
MU_EXPORT int mu_gemm_simt(const void* A, const void* W, const float* bias, const float* residual,
                           void* C, int M, int N, int K, long long lda, long long ldw,
                           long long ldc, long long ldr, int act, int in_bf16, int out_bf16,
                           void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (K <= 0 || !A || !W || !C) return MU_ERR_BAD_ARGUMENT;
    if (lda < K || ldw < K || ldc < N || (residual && ldr < N)) return MU_ERR_BAD_ARGUMENT;
    dim3 grid((N + mu::SG_BN - 1) / mu::SG_BN, (M + mu::SG_BM - 1) / mu::SG_BM);
    if (grid.y > 65535) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
#define MU_LAUNCH(TA, TC)                                                                     \
    mu::gemm_simt_kernel<TA, TC><<<grid, mu::SG_THREADS, 0, s>>>(                              \
        (const TA*)A, (const TA*)W, bias, residual, (TC*)C, M, N, K, lda, ldw, ldc, ldr, act)
    if (in_bf16 && out_bf16) MU_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (in_bf16) MU_LAUNCH(__nv_bfloat16, float);
    else if (out_bf16) MU_LAUNCH(float, __nv_bfloat16);
    else MU_LAUNCH(float, float);
#undef MU_LAUNCH
    MU_CHECK_LAUNCH();
    return MU_OK;
}
