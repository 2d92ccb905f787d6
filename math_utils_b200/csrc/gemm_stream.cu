// C[M, N] = act(A[M, K] . W[N, K]^T + bias) for up to 16 rows and very many output columns: an output head.
//
// Such a product is the time it takes to read W once (77 MB for GPT-2's head), so the kernel is built around
// the fastest way this GPU reads a long run of memory: bulk copies (cp.async.bulk) into a ring in shared
// memory, a hundred kilobytes in flight per SM, with nothing of it held in registers.  The few-rows kernel of
// gemm_skinny.cuh keeps its weights in flight in registers; two blocks of it fill the register file with
// 128 KB, which is where its rate stops (3.8 TB/s of 6.5).
//
//   * A block takes tiles of 64 consecutive weight rows (output columns), tile after tile (as many blocks as
//     SMs, each walking over its tiles); 64 rows of a row-major W are one contiguous run, a warp's strip of 16
//     of them another: one bulk copy a strip, counted by the strip's own mbarrier.
//   * Two such tiles fit the shared memory: while the four warps work on one, the next one is on its way.
//   * A warp turns its strip into tensor-core work exactly as the few-rows kernel does (mma.sync.m16n8k16 with
//     the weight rows as the 16-row operand; fragments are 16-byte pieces of a row, read from shared memory
//     here), against the activations, which the block keeps in shared memory: given as bfloat16, or made as
//     the LayerNorm of float32 rows by the block itself (mean and biased variance in float32), once.
//   * Every wait on a copy is bounded; a wait that runs out sets *status to 8 and the block stops.
//
// The reference's counterpart is matmulNTBias (include/ai/Kernels.hpp:433-447).
#include "gemm_skinny.cuh"
#include "tcgen05.cuh"

namespace mu {

constexpr int GS_WARPS = 4;                       // each owns a strip of 16 weight rows of the block's tile
constexpr int GS_ROWS = 16 * GS_WARPS;
constexpr int GS_THREADS = 32 * GS_WARPS;

__device__ __forceinline__ void gs_bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Dynamic shared memory, 128-byte aligned: [2][GS_ROWS][K] bfloat16 (the two tiles), [MP][K + 8] bfloat16 (the
// activations; rows 16 bytes apart modulo 128, so a quarter of a warp reads them without bank conflicts), and
// with a norm 2 K floats (gamma, beta).
template <int MT, typename TC>
__global__ void __launch_bounds__(GS_THREADS)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, TC* __restrict__ C, int M, int N, int K, long long ldc, int act,
                   SkinnyNorm norm, int* status) {
    constexpr int MP = 8 * MT;
    extern __shared__ __align__(128) unsigned char gs_raw[];
    const size_t tile_bytes = (size_t)GS_ROWS * K * sizeof(__nv_bfloat16);
    const size_t strip_bytes = tile_bytes / GS_WARPS;
    __nv_bfloat16* act_smem = reinterpret_cast<__nv_bfloat16*>(gs_raw + 2 * tile_bytes);
    const int act_ld = K + 8;
    float* gamma_s = reinterpret_cast<float*>(gs_raw + 2 * tile_bytes + (size_t)MP * act_ld * sizeof(__nv_bfloat16));
    float* beta_s = gamma_s + K;
    __shared__ uint64_t full[2][GS_WARPS];
    __shared__ int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // this block's strips of 16 weight rows: an even share of all of them, one after another, taken four at a
    // time (a tile); the last tile of a block may be short
    const int n_strips = (N + 15) / 16;
    const int strip0 = (int)((long long)n_strips * blockIdx.x / gridDim.x);
    const int strip1 = (int)((long long)n_strips * (blockIdx.x + 1) / gridDim.x);
    const int n_tiles = (strip1 - strip0 + GS_WARPS - 1) / GS_WARPS;
    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int b = 0; b < 2; ++b)
            for (int w = 0; w < GS_WARPS; ++w) mbar_init(&full[b][w], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();
    // one thread asks for the four strips of a tile (fewer rows, or none, at the end of W)
    auto ask = [&](int tile, int buf) {
        for (int w = 0; w < GS_WARPS; ++w) {
            const int strip = strip0 + tile * GS_WARPS + w;
            const long long first = 16ll * strip;
            const long long rows = strip >= strip1 ? 0 : (N - first < 16 ? N - first : 16);
            const uint32_t bytes = (uint32_t)(rows * K * (long long)sizeof(__nv_bfloat16));
            mbar_expect_tx(&full[buf][w], bytes);
            if (bytes) gs_bulk_load(gs_raw + (size_t)buf * tile_bytes + (size_t)w * strip_bytes, W + first * K, bytes, &full[buf][w]);
        }
    };
    // weights are written by no kernel: the first tile sets off before the wait for the kernel before, and so do
    // the norm's parameters
    if (threadIdx.x == 0 && n_tiles > 0) ask(0, 0);
    if (norm.x) {
        for (int k = threadIdx.x * 4; k < K; k += GS_THREADS * 4) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(gamma_s + k)), "l"(norm.gamma + k));
            if (norm.beta)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(beta_s + k)), "l"(norm.beta + k));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    pdl_wait();                                            // the activations are the work of earlier kernels

    if (norm.x) {
        // A warp takes two rows at a time, both read into registers before either is reduced (all loads issued
        // back to back: one trip to the L2 for the pair); the arithmetic is the few-rows kernel's.
        constexpr int LNV = 8;                               // float4 a lane: rows of up to 1,024 (see mu_gemm_stream_fits)
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int n4 = K / 4;
        const float4* g4 = reinterpret_cast<const float4*>(gamma_s);
        const float4* b4 = reinterpret_cast<const float4*>(beta_s);
        for (int m0 = warp; m0 < MP; m0 += 2 * GS_WARPS) {
            float4 v[2][LNV];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + h * GS_WARPS;
                const float4* src4 = reinterpret_cast<const float4*>(
                    norm.x + (long long)(m < M ? (norm.rows ? norm.rows[m] : m) : 0) * norm.ldx);
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    const int idx = lane + 32 * i;
                    v[h][i] = (m < M && idx < n4) ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + h * GS_WARPS;
                if (m >= MP) continue;
                __nv_bfloat16* dst = act_smem + (long long)m * act_ld;
                if (m >= M) {                                // a padded row: zeros
                    for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                    continue;
                }
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < LNV; ++i) sum += (v[h][i].x + v[h][i].y) + (v[h][i].z + v[h][i].w);
                const float mean = warp_sum(sum) / (float)K;
                float sq = 0.0f;
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    if (lane + 32 * i < n4) {
                        const float a = v[h][i].x - mean, b = v[h][i].y - mean, c = v[h][i].z - mean, d = v[h][i].w - mean;
                        sq += (a * a + b * b) + (c * c + d * d);
                    }
                }
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    const int idx = lane + 32 * i;
                    if (idx < n4) {
                        const float4 gg = g4[idx];
                        const float4 bb = norm.beta ? b4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        __nv_bfloat162 lo = __floats2bfloat162_rn((v[h][i].x - mean) * inv * gg.x + bb.x,
                                                                  (v[h][i].y - mean) * inv * gg.y + bb.y);
                        __nv_bfloat162 hi = __floats2bfloat162_rn((v[h][i].z - mean) * inv * gg.z + bb.z,
                                                                  (v[h][i].w - mean) * inv * gg.w + bb.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(dst + 4 * idx) = packed;
                    }
                }
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < MP * (K / 8); idx += GS_THREADS) {
            const int m = idx / (K / 8), k = (idx % (K / 8)) * 8;
            *reinterpret_cast<uint4*>(act_smem + (long long)m * act_ld + k) =
                m < M ? *reinterpret_cast<const uint4*>(A + (long long)m * lda + k) : make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    const __nv_bfloat16* xrow[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) xrow[j] = act_smem + (long long)(8 * j + g) * act_ld + 8 * t;
    const int k_blocks = (K + 31) / 32;
    const bool to_bf16 = sizeof(TC) == 2;

    int tile = 0;
    for (; tile < n_tiles; ++tile) {
        const int buf = tile & 1;
        // the other half was read in the turn before (the barrier at the end of it): the next tile may land there
        if (threadIdx.x == 0 && tile + 1 < n_tiles) ask(tile + 1, buf ^ 1);
        bool ok = mbar_wait(&full[buf][warp], (uint32_t)((tile >> 1) & 1));
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) {
            if (lane == 0) { atomicExch(status, 8); gave_up = 1; }
        } else if (strip0 + tile * GS_WARPS + warp < strip1) {      // (a short last tile leaves some warps without a strip)
            const __nv_bfloat16* strip = reinterpret_cast<const __nv_bfloat16*>(gs_raw + (size_t)buf * tile_bytes + (size_t)warp * strip_bytes);
            const __nv_bfloat16* w0 = strip + (long long)g * K + 8 * t;
            const __nv_bfloat16* w1 = strip + (long long)(g + 8) * K + 8 * t;
            float acc[MT][4];
#pragma unroll
            for (int j = 0; j < MT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
#pragma unroll 4
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int k = kb * 32;
                const bool in = (k + 8 * t) < K;                  // K is a multiple of 8
                const uint4 a = in ? *reinterpret_cast<const uint4*>(w0 + k) : make_uint4(0, 0, 0, 0);
                const uint4 b = in ? *reinterpret_cast<const uint4*>(w1 + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    const uint4 xb = in ? *reinterpret_cast<const uint4*>(xrow[j] + k) : make_uint4(0, 0, 0, 0);
                    mma_bf16_16816(acc[j], a.x, b.x, a.y, b.y, xb.x, xb.y);
                    mma_bf16_16816(acc[j], a.z, b.z, a.w, b.w, xb.z, xb.w);
                }
            }
            // accumulator layout: c0, c1 = (weight row g, activation rows 8 j + 2 t, + 1); c2, c3 = weight row g + 8
            const int n0 = 16 * (strip0 + tile * GS_WARPS + warp) + g;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = n0 + (i >= 2 ? 8 : 0), m = 8 * j + 2 * t + (i & 1);
                    if (n < N && m < M) {
                        float v = acc[j][i] + (bias ? bias[n] : 0.0f);
                        v = to_bf16 ? apply_act_bf16(v, act) : apply_act(v, act);
                        C[(long long)m * ldc + n] = from_float<TC>(v);
                    }
                }
            }
        }
        __syncthreads();                                    // every warp has read this half
        if (gave_up) break;
    }
    // a block that gave up leaves with its copies landed: the one asked for last may still be under way
    if (gave_up && threadIdx.x == 0 && tile + 1 < n_tiles) {
        for (int w = 0; w < GS_WARPS; ++w) mbar_wait(&full[(tile + 1) & 1][w], (uint32_t)(((tile + 1) >> 1) & 1));
    }
}

template <int MT, typename TC>
static int launch_stream(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* W, const float* bias, TC* C, int M,
                         int N, int K, long long ldc, int act, const SkinnyNorm& norm, int* status, size_t smem,
                         cudaStream_t s) {
    auto kernel = gemm_stream_kernel<MT, TC>;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) != cudaSuccess)
            return MU_ERR_LAUNCH;
        raised = true;
    }
    const int sms = sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    const int n_tiles = (N + GS_ROWS - 1) / GS_ROWS;        // (fewer blocks than SMs only for a short W)
    return launch_pdl(kernel, dim3(n_tiles < sms ? n_tiles : sms), dim3(GS_THREADS), smem, s, 1, A, lda, W, bias, C, M,
                      N, K, ldc, act, norm, status);
}

}  // namespace mu

// Whether mu_gemm_stream takes this product: up to 16 rows, contiguous weight rows (ldw == K) of a length that
// lets two tiles and the activations share an SM's shared memory (K up to about 800), K a multiple of 8.
MU_EXPORT int mu_gemm_stream_fits(int M, int K, long long ldw, int with_norm) {
    if (M <= 0 || M > 16 || K <= 0 || K % 8 != 0 || ldw != K) return 0;
    if (with_norm && K > 1024) return 0;                   // (the norm keeps a row in registers, 8 float4 a lane)
    const size_t mp = M <= 8 ? 8 : 16;
    const size_t smem = 2 * (size_t)mu::GS_ROWS * K * 2 + mp * (K + 8) * 2 + (with_norm ? 2 * (size_t)K * 4 : 0);
    return smem <= 220 * 1024 ? 1 : 0;
}

// A: bfloat16 [M, K] (lda), or null with x: then A = LayerNorm(x[rows]) of float32 rows (ldx), gamma and optional
// beta float32 [K].  W bfloat16 [N, K], rows one after another, 16-byte aligned.  C bfloat16 or float32 (ldc).
// `status` as mu_gemm_tc (code 8 here).
MU_EXPORT int mu_gemm_stream(const void* A, long long lda, const float* x, long long ldx, const int* rows,
                             const float* gamma, const float* beta, float eps, const void* W, const float* bias,
                             void* C, int M, int N, int K, long long ldw, long long ldc, int act, int out_bf16,
                             int* status, void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (!W || !C || !status || (!A && !x) || (x && !gamma)) return MU_ERR_BAD_ARGUMENT;
    if (!mu_gemm_stream_fits(M, K, ldw, x ? 1 : 0)) return MU_ERR_UNSUPPORTED_SIZE;
    if ((uintptr_t)W & 15) return MU_ERR_ALIGNMENT;
    if (A && (lda % 8 != 0 || lda < K || ((uintptr_t)A & 15))) return MU_ERR_ALIGNMENT;
    if (x && (ldx < K || ldx % 4 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)gamma & 15) || (beta && ((uintptr_t)beta & 15))))
        return MU_ERR_ALIGNMENT;
    if (ldc < N) return MU_ERR_BAD_ARGUMENT;
    const mu::SkinnyNorm norm = {x, rows, gamma, beta, ldx, eps};
    const size_t mp = M <= 8 ? 8 : 16;
    const size_t smem = 2 * (size_t)mu::GS_ROWS * K * 2 + mp * (K + 8) * 2 + (x ? 2 * (size_t)K * 4 : 0);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
#define MU_GS(MT)                                                                                                   \
    (out_bf16 ? mu::launch_stream<MT, __nv_bfloat16>(a, lda, w, bias, (__nv_bfloat16*)C, M, N, K, ldc, act, norm,    \
                                                     status, smem, s)                                               \
              : mu::launch_stream<MT, float>(a, lda, w, bias, (float*)C, M, N, K, ldc, act, norm, status, smem, s))
    return M <= 8 ? MU_GS(1) : MU_GS(2);
#undef MU_GS
}
