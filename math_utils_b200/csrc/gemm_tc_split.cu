// The tensor-core product cut along K (the kernel: gemm_tc_kernel.cuh): its kernel variants, compiled apart
// from the uncut ones so that the two files build side by side.  Stages are 64 deep here: the finer cut.
#include "gemm_tc_kernel.cuh"

namespace mu {

int launch_tc_split(int bn, const void* A, const void* W, const float* bias, const float* residual, void* C, int M,
                    int N, int K, long long lda, long long ldw, long long ldc, long long ldr, int act, int out_bf16,
                    int* status, int splits, cudaStream_t s) {
#define MU_TC_SPLIT(BN, ST)                                                                                       \
    (out_bf16 ? launch_tc<BN, ST, 1, __nv_bfloat16, true>(A, W, bias, residual, (__nv_bfloat16*)C, M, N, K, lda,  \
                                                          ldw, ldc, ldr, act, status, splits, s)                 \
              : launch_tc<BN, ST, 1, float, true>(A, W, bias, residual, (float*)C, M, N, K, lda, ldw, ldc, ldr,   \
                                                  act, status, splits, s))
    if (bn == 64) return MU_TC_SPLIT(64, 6);
    if (bn == 128) return MU_TC_SPLIT(128, 5);
    return MU_TC_SPLIT(256, 4);
#undef MU_TC_SPLIT
}

}  // namespace mu
