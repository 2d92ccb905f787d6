// C[M, N] = act(A[M, K] . W[N, K]^T + bias) (+ residual) for few rows (M <= 64), bfloat16.
//
// With a handful of rows the product is bound by reading W once from HBM, so
// the kernel is built around streaming W: the weight rows are the 16-row
// operand of mma.sync.m16n8k16 (bf16 in, fp32 accumulate) and the activations
// the 8-column operand, so a warp turns 16 weight rows x 32 k into tensor-core
// work for up to 64 activation rows without any shuffle or shared-memory
// staging: each thread loads 16 contiguous bytes of a weight row and of an
// activation row and feeds both to the same k slots of the instruction (the
// sum over k does not care which k sits in which slot as long as both operands
// agree).  A block is 8 warps laid out as WN groups of 16 weight rows x WK
// slices of K; the slices are summed through shared memory in a fixed order,
// then bias, activation and residual are applied and the result written with
// consecutive threads on consecutive columns.  When the output is narrow (few
// blocks) and K long, CK blocks of a thread-block cluster share one output
// tile, each taking a part of K; the others hand their partial tile to the
// first block through distributed shared memory, which adds them in rank
// order, so the sum does not depend on timing.
//
// This is the path of single-token steps (the reference runs them through
// matmulNTBias, one dot product per output: include/ai/Kernels.hpp:433-447).
#pragma once
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace mu {

constexpr int SK_WARPS = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const __nv_bfloat16* p) {
    // weights are read once per step: keep them out of L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// With LN the activations are not given but made: row m of A is the LayerNorm
// of row ln_rows[m] (or m) of the float32 matrix ln_x, computed by the block
// into shared memory as bfloat16 (mean and biased variance in float32, as
// mu_layernorm does), so that the norm costs no launch of its own.
struct SkinnyNorm {
    const float* x;
    const int* rows;
    const float* gamma;
    const float* beta;
    long long ldx;
    float eps;
};

template <int MT, int WN, int WK, int CK, typename TC, bool LN>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, const float* residual, TC* C, int M, int N, int K,
                   long long lda, long long ldw, long long ldc, long long ldr, int act, SkinnyNorm norm) {
    static_assert(WN * WK == SK_WARPS, "a block is 8 warps");
    constexpr int ROWS = 16 * WN;          // weight rows (output columns) per block
    constexpr int MP = 8 * MT;             // activation rows, padded
    __shared__ float red[WK][ROWS][MP + 1];
    __shared__ float peer[CK > 1 ? CK - 1 : 1][CK > 1 ? ROWS : 1][CK > 1 ? MP + 1 : 1];   // partial tiles of the other blocks
    extern __shared__ __align__(16) unsigned char skinny_dyn[];
    __nv_bfloat16* act_smem = reinterpret_cast<__nv_bfloat16*>(skinny_dyn);   // [MP][K + 8] with LN
    const int act_ld = K + 8;              // rows 16 bytes apart modulo 128: no bank conflicts

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wn = warp % WN, wk = warp / WN;
    const int g = lane >> 2, t = lane & 3;
    const int rank = CK > 1 ? (int)blockIdx.y : 0;         // the cluster spans grid.y
    // A block takes the tiles of ROWS output columns blockIdx.x, + gridDim.x, ...: one tile, unless the launcher
    // starts fewer blocks than tiles (many output columns: as many blocks as are resident at once, each norming
    // its rows once and then streaming tile after tile).
    const int n_tiles = (N + ROWS - 1) / ROWS;
    int tile = blockIdx.x;
    int n_base = tile * ROWS + wn * 16;

    // K is cut into CK * WK slices on 32-element boundaries
    const int k_blocks = (K + 31) / 32;
    const int per = (k_blocks + CK * WK - 1) / (CK * WK);
    const int kb0 = (rank * WK + wk) * per, kb1 = min(k_blocks, kb0 + per);

    // rows past the end are clamped for loading and dropped when writing
    const __nv_bfloat16* w0 = W + (long long)min(n_base + g, N - 1) * ldw + 8 * t;
    const __nv_bfloat16* w1 = W + (long long)min(n_base + g + 8, N - 1) * ldw + 8 * t;

    // the first weights are asked for before anything else: they do not depend on the activations
    constexpr int UNROLL = 4;
    // two register sets when the accumulators are few: the next batch of weights is on its way
    // while the tensor cores work on this one
    constexpr bool DOUBLE = MT <= 2;
    uint4 wa[UNROLL], wb[UNROLL], wa2[DOUBLE ? UNROLL : 1], wb2[DOUBLE ? UNROLL : 1];
    auto load_into = [&](int kb, uint4* a, uint4* b) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (kb + u) * 32;
            const bool in = (kb + u) < kb1 && (k + 8 * t) < K;      // K is a multiple of 8
            a[u] = in ? load_stream(w0 + k) : make_uint4(0, 0, 0, 0);
            b[u] = in ? load_stream(w1 + k) : make_uint4(0, 0, 0, 0);
        }
    };
    auto load_weights = [&](int kb) { load_into(kb, wa, wb); };
    pdl_trigger();
    load_weights(kb0);
    // bias and norm parameters are weights too: they set off before the wait as well
    __shared__ float bias_s[ROWS];
    if (threadIdx.x < ROWS) {
        const int n = tile * ROWS + threadIdx.x;
        bias_s[threadIdx.x] = (bias && n < N) ? bias[n] : 0.0f;
    }
    float* gamma_s = reinterpret_cast<float*>(skinny_dyn + (size_t)MP * act_ld * sizeof(__nv_bfloat16));
    float* beta_s = gamma_s + K;
    if (LN) {
        for (int k = threadIdx.x * 4; k < K; k += SK_WARPS * 32 * 4) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(gamma_s + k)),
                         "l"(norm.gamma + k));
            if (norm.beta)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(beta_s + k)),
                             "l"(norm.beta + k));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    pdl_wait();                                            // activations and residual from here on
    // the residual of this thread's first two outputs, asked for now and used in the epilogue
    float res_pre[2] = {0.0f, 0.0f};
    if (residual && rank == 0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * SK_WARPS * 32;
            const int m = idx / ROWS, n = tile * ROWS + idx % ROWS;
            if (idx < ROWS * M && n < N) res_pre[i] = residual[(long long)m * ldr + n];
        }
    }

    if (LN) {
        // One warp per row.  The row is read once, as float4, into registers (all loads of a lane
        // issued back to back: one round trip to L2 instead of one per element); rows too long for
        // that are read three times with the same arithmetic.
        constexpr int LNV = 16;                               // float4 per lane kept in registers
        const int w = threadIdx.x >> 5, ln = threadIdx.x & 31;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                      // gamma and beta are in shared memory
        const int n4 = K / 4;
        const bool pairs = MT >= 2 && n4 <= 32 * 8 && (norm.ldx % 4 == 0) && (((uintptr_t)norm.x & 15) == 0);
        if (pairs) {
            // more than eight rows, MT a warp: two rows at a time are read into registers before either is
            // reduced, so a pair costs one trip to the L2 (rows of up to 1,024: eight float4 a lane and row)
            constexpr int LNP = 8;
            const float4* g4 = reinterpret_cast<const float4*>(gamma_s);
            const float4* b4 = reinterpret_cast<const float4*>(beta_s);
#pragma unroll
            for (int h0 = 0; h0 < MT; h0 += 2) {
            float4 v[2][LNP];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = w + (h0 + h) * SK_WARPS;
                const bool real = h0 + h < MT && m < M;
                const float4* src4 = reinterpret_cast<const float4*>(
                    norm.x + (long long)(real ? (norm.rows ? norm.rows[m] : m) : 0) * norm.ldx);
#pragma unroll
                for (int i = 0; i < LNP; ++i) {
                    const int idx = ln + 32 * i;
                    v[h][i] = (real && idx < n4) ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h0 + h >= MT) continue;
                const int m = w + (h0 + h) * SK_WARPS;
                __nv_bfloat16* dst = act_smem + (long long)m * act_ld;
                if (m >= M) {
                    for (int k = ln * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                    continue;
                }
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < LNP; ++i) sum += (v[h][i].x + v[h][i].y) + (v[h][i].z + v[h][i].w);
                const float mean = warp_sum(sum) / (float)K;
                float sq = 0.0f;
#pragma unroll
                for (int i = 0; i < LNP; ++i) {
                    if (ln + 32 * i < n4) {
                        const float a = v[h][i].x - mean, b = v[h][i].y - mean, c = v[h][i].z - mean, d = v[h][i].w - mean;
                        sq += (a * a + b * b) + (c * c + d * d);
                    }
                }
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
#pragma unroll
                for (int i = 0; i < LNP; ++i) {
                    const int idx = ln + 32 * i;
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
        }
        for (int m = pairs ? MP : w; m < MP; m += SK_WARPS) {
            __nv_bfloat16* dst = act_smem + (long long)m * act_ld;
            if (m >= M) {
                for (int k = ln * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const float* src = norm.x + (long long)(norm.rows ? norm.rows[m] : m) * norm.ldx;
            if (n4 <= 32 * LNV && (norm.ldx % 4 == 0) && (((uintptr_t)norm.x & 15) == 0)) {
                const float4* src4 = reinterpret_cast<const float4*>(src);
                float4 v[LNV];
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    const int idx = ln + 32 * i;
                    v[i] = idx < n4 ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < LNV; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                const float mean = warp_sum(sum) / (float)K;
                float sq = 0.0f;
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    if (ln + 32 * i < n4) {
                        const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                        sq += (a * a + b * b) + (c * c + d * d);
                    }
                }
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
                const float4* g4 = reinterpret_cast<const float4*>(gamma_s);
                const float4* b4 = reinterpret_cast<const float4*>(beta_s);
#pragma unroll
                for (int i = 0; i < LNV; ++i) {
                    const int idx = ln + 32 * i;
                    if (idx < n4) {
                        const float4 gg = g4[idx];
                        const float4 bb = norm.beta ? b4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        __nv_bfloat162 lo = __floats2bfloat162_rn((v[i].x - mean) * inv * gg.x + bb.x,
                                                                  (v[i].y - mean) * inv * gg.y + bb.y);
                        __nv_bfloat162 hi = __floats2bfloat162_rn((v[i].z - mean) * inv * gg.z + bb.z,
                                                                  (v[i].w - mean) * inv * gg.w + bb.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(dst + 4 * idx) = packed;
                    }
                }
            } else {
                float sum = 0.0f;
#pragma unroll 8
                for (int k = ln; k < K; k += 32) sum += src[k];
                const float mean = warp_sum(sum) / (float)K;
                float sq = 0.0f;
#pragma unroll 8
                for (int k = ln; k < K; k += 32) { const float c = src[k] - mean; sq += c * c; }
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
#pragma unroll 8
                for (int k = ln; k < K; k += 32)
                    dst[k] = __float2bfloat16_rn((src[k] - mean) * inv * gamma_s[k] + (norm.beta ? beta_s[k] : 0.0f));
            }
        }
        __syncthreads();
    }

    const __nv_bfloat16* xrow[MT];
    bool xvalid[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        const int m = 8 * j + g;
        xvalid[j] = LN || m < M;           // padded rows of the shared copy hold zeros
        xrow[j] = LN ? act_smem + (long long)m * act_ld + 8 * t : A + (long long)min(m, M - 1) * lda + 8 * t;
    }

    for (;;) {                                     // over this block's tiles
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

    auto multiply = [&](int kb, const uint4* a, const uint4* b) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (kb + u) * 32;
            const bool in = (kb + u) < kb1 && (k + 8 * t) < K;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                uint4 xb = make_uint4(0, 0, 0, 0);
                if (in && xvalid[j]) xb = *reinterpret_cast<const uint4*>(xrow[j] + k);
                mma_bf16_16816(acc[j], a[u].x, b[u].x, a[u].y, b[u].y, xb.x, xb.y);
                mma_bf16_16816(acc[j], a[u].z, b[u].z, a[u].w, b[u].w, xb.z, xb.w);
            }
        }
    };
    if (DOUBLE) {
        for (int kb = kb0; kb < kb1; kb += 2 * UNROLL) {
            if (kb + UNROLL < kb1) load_into(kb + UNROLL, wa2, wb2);
            multiply(kb, wa, wb);
            if (kb + 2 * UNROLL < kb1) load_into(kb + 2 * UNROLL, wa, wb);
            if (kb + UNROLL < kb1) multiply(kb + UNROLL, wa2, wb2);
        }
    } else {
        for (int kb = kb0; kb < kb1; kb += UNROLL) {
            if (kb != kb0) load_weights(kb);
            multiply(kb, wa, wb);
        }
    }

    // accumulator layout: c0,c1 = (weight row g, activation rows 8j+2t, +1); c2,c3 = weight row g+8
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[wk][wn * 16 + g][8 * j + 2 * t] = acc[j][0];
        red[wk][wn * 16 + g][8 * j + 2 * t + 1] = acc[j][1];
        red[wk][wn * 16 + g + 8][8 * j + 2 * t] = acc[j][2];
        red[wk][wn * 16 + g + 8][8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (CK > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        if (rank != 0) {
            float* dst = cluster.map_shared_rank(&peer[0][0][0], 0) + (long long)(rank - 1) * ROWS * (MP + 1);
            for (int idx = threadIdx.x; idx < ROWS * MP; idx += SK_WARPS * 32) {
                const int r = idx / MP, m = idx % MP;
                float v = 0.0f;
#pragma unroll
                for (int s = 0; s < WK; ++s) v += red[s][r][m];
                dst[r * (MP + 1) + m] = v;
            }
        }
        cluster.sync();
        if (rank != 0) return;
    }
    const int col0 = tile * ROWS;
    for (int idx = threadIdx.x; idx < ROWS * M; idx += SK_WARPS * 32) {
        const int m = idx / ROWS, r = idx % ROWS;
        const int n = col0 + r;
        if (n >= N) continue;
        float v = 0.0f;
#pragma unroll
        for (int s = 0; s < WK; ++s) v += red[s][r][m];
        if (CK > 1) {
#pragma unroll
            for (int c = 0; c < CK - 1; ++c) v += peer[c][r][m];
        }
        v += bias_s[r];
        v = sizeof(TC) == 2 ? apply_act_bf16(v, act) : apply_act(v, act);
        if (residual) {
            const int turn = idx / (SK_WARPS * 32);
            v += turn == 0 ? res_pre[0] : turn == 1 ? res_pre[1] : residual[(long long)m * ldr + n];
        }
        C[(long long)m * ldc + n] = from_float<TC>(v);
    }
    tile += gridDim.x;
    if (CK > 1 || tile >= n_tiles) break;
    // the next tile of this block: its first weights set off, then the shared arrays change hands
    n_base = tile * ROWS + wn * 16;
    w0 = W + (long long)min(n_base + g, N - 1) * ldw + 8 * t;
    w1 = W + (long long)min(n_base + g + 8, N - 1) * ldw + 8 * t;
    load_weights(kb0);
    __syncthreads();                               // everyone has read red and bias_s
    if (threadIdx.x < ROWS) {
        const int n = tile * ROWS + threadIdx.x;
        bias_s[threadIdx.x] = (bias && n < N) ? bias[n] : 0.0f;
    }
    res_pre[0] = res_pre[1] = 0.0f;
    if (residual) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * SK_WARPS * 32;
            const int m = idx / ROWS, n = tile * ROWS + idx % ROWS;
            if (idx < ROWS * M && n < N) res_pre[i] = residual[(long long)m * ldr + n];
        }
    }
    }
}

template <int MT, int WN, int WK, int CK, typename TC, bool LN>
static int launch_skinny_as(const __nv_bfloat16* A, const __nv_bfloat16* W, const float* bias,
                            const float* residual, TC* C, int M, int N, int K, long long lda, long long ldw,
                            long long ldc, long long ldr, int act, const SkinnyNorm& norm, cudaStream_t s) {
    auto kernel = gemm_skinny_kernel<MT, WN, WK, CK, TC, LN>;
    size_t dyn = 0;
    if (LN) {
        dyn = (size_t)8 * MT * (K + 8) * sizeof(__nv_bfloat16) + (size_t)2 * K * sizeof(float);   // rows, gamma, beta
        if (dyn > 160 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
        if (dyn > 24 * 1024) {
            // more than the default limit allows next to the static part; asked for once per variant
            static bool raised = false;
            if (!raised) {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) !=
                    cudaSuccess)
                    return MU_ERR_LAUNCH;
                raised = true;
            }
        }
    }
    {
        // Half of an SM's memory as shared memory for these kernels.  Left to itself the driver picks the
        // smallest split a block fits in, which differs from kernel to kernel, and an SM changes its split
        // only when it is empty: the blocks of the next kernel then cannot move in beside the last blocks of
        // this one.  (All of it as shared memory costs more in the L1 than it gains.)
        static bool asked = false;
        if (!asked) {
            cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 50);
            asked = true;
        }
    }
    int blocks = (N + 16 * WN - 1) / (16 * WN);
    if (CK == 1) {
        // more tiles than blocks are resident at once: that many blocks, each walking over its tiles (it norms
        // its rows once, and no second wave of blocks starts from nothing)
        static int per_sm = 0;
        static size_t per_sm_dyn = ~(size_t)0;
        if (per_sm_dyn != dyn) {
            per_sm = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SK_WARPS * 32, dyn) != cudaSuccess)
                per_sm = 0;
            per_sm_dyn = dyn;
        }
        const long long resident = (long long)per_sm * sm_count();
        if (resident > 0 && blocks > resident) blocks = (int)resident;
    }
    return launch_pdl(kernel, dim3(blocks, CK, 1), dim3(SK_WARPS * 32), dyn, s, CK, A, W, bias,
                      residual, C, M, N, K, lda, ldw, ldc, ldr, act, norm);
}

template <int MT, typename TC, bool LN>
static int launch_skinny(const __nv_bfloat16* A, const __nv_bfloat16* W, const float* bias,
                         const float* residual, TC* C, int M, int N, int K, long long lda, long long ldw,
                         long long ldc, long long ldr, int act, const SkinnyNorm& norm, cudaStream_t s) {
    // many output columns: whole K per warp; few: K cut over the warps of a block, and over the
    // blocks of a cluster when even that leaves most SMs idle
#define MU_SK(WN, WK, CK) \
    return launch_skinny_as<MT, WN, WK, CK, TC, LN>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, ldr, act, norm, s)
    const int tiles = (N + 15) / 16, k_blocks = (K + 31) / 32;
    const int sms = sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    const long long wave = 16ll * 2 * sms;            // output columns that two blocks per SM of one tile each cover
    if (N >= 8 * wave && K <= 2048) MU_SK(8, 1, 1);
    else if (N >= 4 * wave) MU_SK(4, 2, 1);
    else if (N >= 2 * wave) MU_SK(2, 4, 1);
    else if (2 * tiles < sms && k_blocks >= 64) MU_SK(1, 8, 4);
    else if (tiles < sms && k_blocks >= 48) MU_SK(1, 8, 2);
    else MU_SK(1, 8, 1);
#undef MU_SK
}

// The variants for M rows (MT blocks of 8 rows, up to MAX_MT of them).  One (output type, norm) pair per
// source file, declared here and defined there, so that the files compile side by side.
template <typename TC, bool LN>
int skinny_rows(const __nv_bfloat16* a, const __nv_bfloat16* w, const float* bias, const float* residual, TC* C,
                int M, int N, int K, long long lda, long long ldw, long long ldc, long long ldr, int act,
                const SkinnyNorm& norm, cudaStream_t s);

#define MU_SKINNY_ARGS a, w, bias, residual, C, M, N, K, lda, ldw, ldc, ldr, act, norm, s
#define MU_SKINNY_ROWS(TC, LN, MAX_MT)                                                                       \
    template <>                                                                                              \
    int skinny_rows<TC, LN>(const __nv_bfloat16* a, const __nv_bfloat16* w, const float* bias,               \
                            const float* residual, TC* C, int M, int N, int K, long long lda, long long ldw, \
                            long long ldc, long long ldr, int act, const SkinnyNorm& norm, cudaStream_t s) { \
        const int mt = (M + 7) / 8;                                                                          \
        if (mt > MAX_MT) return MU_ERR_UNSUPPORTED_SIZE;                                                     \
        if (mt <= 1) return launch_skinny<1, TC, LN>(MU_SKINNY_ARGS);                                        \
        if (mt <= 2) return launch_skinny<2, TC, LN>(MU_SKINNY_ARGS);                                        \
        if constexpr (MAX_MT > 2) {                                                                          \
            if (mt <= 4) return launch_skinny<4, TC, LN>(MU_SKINNY_ARGS);                                    \
            if constexpr (MAX_MT > 4) return launch_skinny<8, TC, LN>(MU_SKINNY_ARGS);                       \
        }                                                                                                    \
        return MU_ERR_UNSUPPORTED_SIZE;                                                                      \
    }

}  // namespace mu
