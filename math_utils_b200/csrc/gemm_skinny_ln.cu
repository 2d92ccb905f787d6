// The few-row product (see gemm_skinny.cuh): bfloat16 output, activations made as a LayerNorm inside the kernel.
#include "gemm_skinny.cuh"

namespace mu {
MU_SKINNY_ROWS(__nv_bfloat16, true, 4)
}  // namespace mu
