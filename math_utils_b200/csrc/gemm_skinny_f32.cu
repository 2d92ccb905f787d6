// The few-row product (see gemm_skinny.cuh): float32 output, given activations.
#include "gemm_skinny.cuh"

namespace mu {
MU_SKINNY_ROWS(float, false, 8)
}  // namespace mu
