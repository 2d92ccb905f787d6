// The few-row product (see gemm_skinny.cuh): float32 output, activations made as a LayerNorm inside the kernel.
#include "gemm_skinny.cuh"

namespace mu {
MU_SKINNY_ROWS(float, true, 4)
}  // namespace mu
