// Embedding gather and LayerNorm.
//
// embed:     x[t, :] = table[id[t], :] + (pos_table ? pos_table[pos[t], :] : 0)
//            -> float32 residual stream (include/ai/LocalModel.hpp:3686-3697).
// layernorm: y = (x - mean) * rsqrt(var + eps) * gamma + beta, biased variance,
//            two passes over the row, all in float32
//            (include/ai/LocalModel.hpp:1355-1367); output in the compute dtype.
#include "common.cuh"

namespace mu {

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const TW* __restrict__ table, const TW* __restrict__ pos_table,
                             float* __restrict__ x, int hidden) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const long long row = ids[t];
    const TW* src = table + row * hidden;
    const TW* psrc = pos_table ? pos_table + (long long)pos[t] * hidden : nullptr;
    float* dst = x + (long long)t * hidden;
#pragma unroll 4
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        float v = to_float(src[d]);
        if (psrc) v += to_float(psrc[d]);
        dst[d] = v;
    }
}

// One block per output row.  The row is staged in shared memory so that the
// mean, the variance and the output each read it once from there.
template <typename TO>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 TO* __restrict__ y, int hidden, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long src_row = rows ? rows[r] : r;
    const float* src = x + src_row * hidden;
    float s = 0.0f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        const float v = src[d];
        row[d] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.0f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        const float c = row[d] - mean;
        q += c * c;
    }
    const float var = block_sum(q, scratch) / (float)hidden;
    const float inv = 1.0f / sqrtf(var + eps);
    TO* dst = y + (long long)r * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        const float v = (row[d] - mean) * inv * gamma[d] + (beta ? beta[d] : 0.0f);
        dst[d] = from_float<TO>(v);
    }
}

// One warp per row, the row read once as float4 into registers (every load of a lane issued
// before the first use), statistics by warp shuffles.  Rows of up to 32 * 16 * 4 = 2048 values.
constexpr int LN_V = 16;
constexpr int LN_WARPS = 4;

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

// MANY: the instantiation for the many rows of a prompt step (it prefers shared memory over L1 like the
// kernels around it there, see prefer_shared_memory); the code is the same.
template <typename TO, bool MANY>
__global__ void __launch_bounds__(LN_WARPS * 32, 4)
layernorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      TO* __restrict__ y, int n_rows, int hidden, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * LN_WARPS + warp;
    const int n4 = hidden / 4;
    // weight and bias are no kernel's output: they are on their way into shared memory while the kernel
    // before this one still runs, so that nothing is fetched after the statistics
    __shared__ __align__(16) float gamma_s[32 * LN_V * 4];
    __shared__ __align__(16) float beta_s[32 * LN_V * 4];
    for (int idx = threadIdx.x; idx < n4; idx += LN_WARPS * 32) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(gamma_s + 4 * idx)),
                     "l"(gamma + 4 * idx) : "memory");
        if (beta)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(beta_s + 4 * idx)),
                         "l"(beta + 4 * idx) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    pdl_trigger();
    pdl_wait();
    const bool real = r < n_rows;
    const long long src_row = real ? (rows ? rows[r] : r) : 0;
    const float4* src4 = reinterpret_cast<const float4*>(x + src_row * hidden);
    float4 v[LN_V];
#pragma unroll
    for (int i = 0; i < LN_V; ++i) {
        const int idx = lane + 32 * i;
        v[i] = (real && idx < n4) ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < LN_V; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = warp_sum(sum) / (float)hidden;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < LN_V; ++i) {
        if (lane + 32 * i < n4) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            sq += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)hidden + eps);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (!real) return;
    const float4* g4 = reinterpret_cast<const float4*>(gamma_s);
    const float4* b4 = reinterpret_cast<const float4*>(beta_s);
    TO* dst = y + (long long)r * hidden;
#pragma unroll
    for (int i = 0; i < LN_V; ++i) {
        const int idx = lane + 32 * i;
        if (idx < n4) {
            const float4 gg = g4[idx];
            const float4 bb = beta ? b4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            store4(dst + 4 * idx, (v[i].x - mean) * inv * gg.x + bb.x, (v[i].y - mean) * inv * gg.y + bb.y,
                   (v[i].z - mean) * inv * gg.z + bb.z, (v[i].w - mean) * inv * gg.w + bb.w);
        }
    }
}

}  // namespace mu

// table_bf16: 1 if the tables hold bfloat16, 0 for float32.
MU_EXPORT int mu_embed(const int* ids, const int* pos, const void* table, const void* pos_table,
                       float* x, int n_tokens, int hidden, int table_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (hidden <= 0 || !ids || !table || !x || (pos_table && !pos)) return MU_ERR_BAD_ARGUMENT;
    const int threads = hidden >= 256 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_bf16)
        return mu::launch_pdl(mu::embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, 1, ids, pos,
                              (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, x, hidden);
    return mu::launch_pdl(mu::embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, 1, ids, pos,
                          (const float*)table, (const float*)pos_table, x, hidden);
}

// rows: optional int32 row indices into x (n_rows of them); out_bf16 picks the output dtype.
MU_EXPORT int mu_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                           void* y, int n_rows, int hidden, float eps, int out_bf16, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (hidden <= 0 || !x || !gamma || !y) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = hidden % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                         ((uintptr_t)gamma & 15) == 0 && (!beta || ((uintptr_t)beta & 15) == 0);
    if (aligned && hidden <= 32 * mu::LN_V * 4) {
        const unsigned blocks = (n_rows + mu::LN_WARPS - 1) / mu::LN_WARPS;
        if (n_rows > 64) {
            if (out_bf16) {
                mu::prefer_shared_memory(reinterpret_cast<const void*>(mu::layernorm_rows_kernel<__nv_bfloat16, true>));
                return mu::launch_pdl(mu::layernorm_rows_kernel<__nv_bfloat16, true>, dim3(blocks), dim3(mu::LN_WARPS * 32),
                                      0, s, 1, x, rows, gamma, beta, (__nv_bfloat16*)y, n_rows, hidden, eps);
            }
            mu::prefer_shared_memory(reinterpret_cast<const void*>(mu::layernorm_rows_kernel<float, true>));
            return mu::launch_pdl(mu::layernorm_rows_kernel<float, true>, dim3(blocks), dim3(mu::LN_WARPS * 32), 0, s, 1,
                                  x, rows, gamma, beta, (float*)y, n_rows, hidden, eps);
        }
        if (out_bf16)
            return mu::launch_pdl(mu::layernorm_rows_kernel<__nv_bfloat16, false>, dim3(blocks), dim3(mu::LN_WARPS * 32), 0,
                                  s, 1, x, rows, gamma, beta, (__nv_bfloat16*)y, n_rows, hidden, eps);
        return mu::launch_pdl(mu::layernorm_rows_kernel<float, false>, dim3(blocks), dim3(mu::LN_WARPS * 32), 0, s, 1, x,
                              rows, gamma, beta, (float*)y, n_rows, hidden, eps);
    }
    if (hidden > 12288) return MU_ERR_UNSUPPORTED_SIZE;   // the row must fit 48 KB of shared memory
    const int threads = hidden >= 1024 ? 256 : 128;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (out_bf16)
        mu::layernorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, s>>>(
            x, rows, gamma, beta, (__nv_bfloat16*)y, hidden, eps);
    else
        mu::layernorm_kernel<float><<<n_rows, threads, smem, s>>>(
            x, rows, gamma, beta, (float*)y, hidden, eps);
    MU_CHECK_LAUNCH();
    return MU_OK;
}

// Turns programmatic dependent launch of the single-token kernels on (1, the default) or off (0).
MU_EXPORT int mu_set_pdl(int enabled) {
    mu::pdl_enabled() = enabled ? 1 : 0;
    return MU_OK;
}

// A plain asynchronous copy on the stream (either direction; host memory should be pinned).  For copies
// that are recorded into a CUDA graph together with the kernels.
MU_EXPORT int mu_copy_async(void* dst, const void* src, long long n_bytes, void* stream) {
    if (n_bytes <= 0) return MU_OK;
    if (!dst || !src) return MU_ERR_BAD_ARGUMENT;
    return cudaMemcpyAsync(dst, src, (size_t)n_bytes, cudaMemcpyDefault, (cudaStream_t)stream) == cudaSuccess
               ? MU_OK : MU_ERR_LAUNCH;
}
