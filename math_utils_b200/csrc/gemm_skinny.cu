// The few-row product (see gemm_skinny.cuh): the library's entry points, and the variants with
// bfloat16 output and given activations.  The other variants are gemm_skinny_f32.cu (float32 output),
// gemm_skinny_ln.cu and gemm_skinny_ln_f32.cu (activations made as a LayerNorm inside the kernel).
#include "gemm_skinny.cuh"

namespace mu {
MU_SKINNY_ROWS(__nv_bfloat16, false, 8)
}  // namespace mu

static int skinny_dispatch(const __nv_bfloat16* a, const __nv_bfloat16* w, const float* bias,
                           const float* residual, void* C, int M, int N, int K, long long lda, long long ldw,
                           long long ldc, long long ldr, int act, int out_bf16, const mu::SkinnyNorm* norm,
                           cudaStream_t s) {
    const mu::SkinnyNorm none = {};
    if (norm)
        return out_bf16 ? mu::skinny_rows<__nv_bfloat16, true>(a, w, bias, residual, (__nv_bfloat16*)C, M, N, K, lda,
                                                               ldw, ldc, ldr, act, *norm, s)
                        : mu::skinny_rows<float, true>(a, w, bias, residual, (float*)C, M, N, K, lda, ldw, ldc, ldr,
                                                       act, *norm, s);
    return out_bf16 ? mu::skinny_rows<__nv_bfloat16, false>(a, w, bias, residual, (__nv_bfloat16*)C, M, N, K, lda,
                                                            ldw, ldc, ldr, act, none, s)
                    : mu::skinny_rows<float, false>(a, w, bias, residual, (float*)C, M, N, K, lda, ldw, ldc, ldr,
                                                    act, none, s);
}

// bfloat16 A [M, K] and W [N, K] with K, lda and ldw multiples of 8 and 16-byte aligned bases;
// M <= 64.  C is bfloat16 or float32; residual float32 (may be C itself).
MU_EXPORT int mu_gemm_skinny(const void* A, const void* W, const float* bias, const float* residual,
                             void* C, int M, int N, int K, long long lda, long long ldw, long long ldc,
                             long long ldr, int act, int out_bf16, void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (K <= 0 || !A || !W || !C) return MU_ERR_BAD_ARGUMENT;
    if (M > 64) return MU_ERR_UNSUPPORTED_SIZE;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return MU_ERR_ALIGNMENT;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return MU_ERR_ALIGNMENT;
    if (lda < K || ldw < K || ldc < N || (residual && ldr < N)) return MU_ERR_BAD_ARGUMENT;
    return skinny_dispatch((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, residual, C, M, N, K, lda,
                           ldw, ldc, ldr, act, out_bf16, nullptr, (cudaStream_t)stream);
}

// The same product with A = LayerNorm(x[rows]) made inside the kernel, for M <= 32: x float32 [*, K] with
// leading dimension ldx, rows optional int32 [M], gamma and beta (optional) float32 [K].
MU_EXPORT int mu_gemm_skinny_ln(const float* x, long long ldx, const int* rows, const float* gamma,
                                const float* beta, float eps, const void* W, const float* bias,
                                const float* residual, void* C, int M, int N, int K, long long ldw,
                                long long ldc, long long ldr, int act, int out_bf16, void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (K <= 0 || !x || !gamma || !W || !C) return MU_ERR_BAD_ARGUMENT;
    if (M > 32) return MU_ERR_UNSUPPORTED_SIZE;
    if (K % 8 != 0 || ldw % 8 != 0) return MU_ERR_ALIGNMENT;
    if ((uintptr_t)W & 15) return MU_ERR_ALIGNMENT;
    if (ldx < K || ldw < K || ldc < N || (residual && ldr < N)) return MU_ERR_BAD_ARGUMENT;
    const mu::SkinnyNorm norm = {x, rows, gamma, beta, ldx, eps};
    return skinny_dispatch(nullptr, (const __nv_bfloat16*)W, bias, residual, C, M, N, K, 0, ldw, ldc, ldr,
                           act, out_bf16, &norm, (cudaStream_t)stream);
}
