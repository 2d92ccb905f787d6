// C[M, N] = act(A[M, K] . W[N, K]^T + bias) (+ residual) on the 5th-generation tensor cores.
//
// The product kernel of whole prompts (bfloat16 in, float32 accumulate).  A
// block per SM walks over the 128 x BN tiles of C; in each block:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//            of 128 x 64 tiles of A and BN x 64 tiles of W into a ring of
//            shared-memory stages and arms each stage's "full" mbarrier;
//   warp 1   allocates 2 x BN columns of tensor memory (two accumulators that take turns, so
//            that one tile is read out while the next is being computed); one lane issues
//            tcgen05.mma (kind::f16, M = 128, N = BN, K = 16) four times per
//            stage with shared-memory descriptors, the accumulator staying in
//            tensor memory, and commits each stage back to the producer
//            ("empty" mbarrier) and at the end the accumulator to the epilogue;
//   warps 2-9  read the accumulator with tcgen05.ld (each warp 32 rows and half the columns
//            of the tile), add bias, apply the activation, add the
//            float32 residual and store bfloat16 or float32.
// Rows of A and W beyond M, N and K are zero-filled by TMA; the epilogue
// predicates its stores.  When C has far fewer tiles than there are SMs (a
// batch of single tokens: one row of tiles) and K is long, K is cut into
// `splits` parts (the SPLIT variant; mu_gemm_tc decides), and
// every (tile, part) is a work item of its own: a block leaves its partial
// tile in a float32 workspace and takes a ticket; the block that draws a
// tile's last ticket adds the parts in the order of K (so the sum does not
// depend on timing), finishes the tile and leaves the ticket at zero.  No
// block waits for another.  Every wait on an mbarrier is bounded: if it runs out
// the block records a code in `status`, lets its copies land, frees its tensor
// memory and returns, so a wrong phase shows up as an error and not as a hang.
//
// The reference's counterpart is matmulTiled (include/ai/Kernels.hpp:315-430).
#pragma once
#include "tcgen05.cuh"


namespace mu {

constexpr int TC_BM = 128, TC_BK = 64, TC_EPI_WARPS = 8, TC_THREADS = 64 + 32 * TC_EPI_WARPS;
constexpr int TC_PATCH_PITCH = 33;               // floats per row of an epilogue patch: odd, so columns and rows both spread over the banks

template <int ACT> __device__ __forceinline__ float tc_act(float x, bool to_bf16) {
    if (ACT == ACT_GELU_NEW) return to_bf16 ? gelu_new_fast(x) : gelu_new(x);
    if (ACT == ACT_GELU_ERF) return gelu_erf(x);
    return x;
}

// One 32 x 32 block of the accumulator (thread = row, r = its 32 columns) to C, with bias, activation and
// residual.  tcgen05.ld hands every thread one row; stored like that, a warp's instruction would touch 32
// rows at once (measured: some 450 cycles per 16-byte store instruction).  So the block is turned in the
// warp's patch of shared memory and written so that an instruction covers whole runs of a row:
//   packed (bfloat16, no residual, 16-byte aligned rows): four lanes write a row's 64 bytes, eight rows per
//     instruction;
//   otherwise: a lane per column, row after row (128 bytes of float32 per instruction); all of the residual
//     is asked for before any of it is used (it may be C itself: every element is read and written by the
//     same lane).
template <int ACT, typename TC>
__device__ __forceinline__ void tc_finish_block(const uint32_t (&r)[32], float* patch, int lane,
                                                const float* __restrict__ bias, const float* bias_lane,
                                                const float* residual, TC* C, int M, int N, int row0, int nb,
                                                long long ldc, long long ldr, bool packed) {
    const int n_rows = min(32, M - row0);
    __syncwarp();                                                   // the patch's last readers are done
#pragma unroll
    for (int i = 0; i < 32; ++i) patch[lane * TC_PATCH_PITCH + i] = __uint_as_float(r[i]);
    __syncwarp();
    if (packed) {
        // four lanes write a row's 64 bytes, eight rows per instruction; a lane's eight columns are the same
        // in every row, so their bias (bias_lane[0..7]) was fetched long before
        __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row0 * ldc + nb;
        const int part = lane & 3;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int row = 8 * it + (lane >> 2);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = tc_act<ACT>(patch[row * TC_PATCH_PITCH + 8 * part + e] + bias_lane[e], true);
            uint4 piece;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
            piece.x = *reinterpret_cast<uint32_t*>(&h0);
            piece.y = *reinterpret_cast<uint32_t*>(&h1);
            piece.z = *reinterpret_cast<uint32_t*>(&h2);
            piece.w = *reinterpret_cast<uint32_t*>(&h3);
            if (row < n_rows) *reinterpret_cast<uint4*>(cb + (long long)row * ldc + 8 * part) = piece;
        }
        return;
    }
    const int n = nb + lane;
    const bool live = n < N;
    const float bv = bias_lane[0];
    TC* cc = C + (long long)row0 * ldc + n;
    const float* rr = (residual && live) ? residual + (long long)row0 * ldr + n : nullptr;
    float x[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = (rr && i < n_rows) ? rr[(long long)i * ldr] : 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] += tc_act<ACT>(patch[i * TC_PATCH_PITCH + lane] + bv, sizeof(TC) == 2);
    if (live) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < n_rows) cc[(long long)i * ldc] = from_float<TC>(x[i]);
    }
}

// The same block through a bulk store: every thread lays its row (bias and activation applied) into the warp's
// patch, row after row, and one lane hands the 32 x 32 box to the copy engine, which writes it (or, where the
// result is to be added to the float32 matrix that is there already, adds it: the residual stream never passes
// through registers) and leaves out what lies beyond the matrix.  The warp goes on at once; it waits for the
// engine to have read the patch only when it needs the patch again.
template <int ACT, typename TC>
__device__ __forceinline__ void tc_finish_block_bulk(const uint32_t (&r)[32], float* patch, int lane,
                                                     const float* __restrict__ bias, const CUtensorMap* map_c,
                                                     int N, int row0, int nb, bool add) {
    float v[32];
    if (bias) {
        if (nb + 32 <= N && (((uintptr_t)(bias + nb)) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + nb) + i);      // the same for every lane
                v[4 * i] = b4.x; v[4 * i + 1] = b4.y; v[4 * i + 2] = b4.z; v[4 * i + 3] = b4.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = nb + i < N ? __ldg(bias + nb + i) : 0.0f;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = tc_act<ACT>(__uint_as_float(r[i]) + v[i], sizeof(TC) == 2);
    if (lane == 0) tma_store_wait_read();                  // the copy engine has read what the patch held before
    __syncwarp();
    if (sizeof(TC) == 2) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(patch) + lane * 64);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(patch) + lane * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        if (add) tma_add_2d(map_c, patch, nb, row0);
        else tma_store_2d(map_c, patch, nb, row0);
    }
}

// A 32 x 32 block of a partial accumulator to the workspace (a tile's part is [128][BN] float32), turned in
// the patch so that an instruction stores 128 bytes of one row.
__device__ __forceinline__ void tc_store_partial(const uint32_t (&r)[32], float* patch, int lane, float* ws_block,
                                                 int bn, int n_rows) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; ++i) patch[lane * TC_PATCH_PITCH + i] = __uint_as_float(r[i]);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (i < n_rows) __stcg(ws_block + (long long)i * bn + lane, patch[i * TC_PATCH_PITCH + lane]);
}

// A tile of C from its parts, by all the epilogue threads together (`who` of `n_threads`): a thread takes
// four neighbouring columns of a row at a time and asks for up to eight parts of them at once (one round
// trip to the L2 instead of one per part), then adds them in the order of K, whoever wrote them when.
// ws_tile: the tile's parts, each [128][BN] float32; rows: the tile's real rows.
template <int ACT, typename TC, int BN>
__device__ __forceinline__ void tc_finish_split(const float* ws_tile, int splits, int who, int n_threads,
                                                const float* __restrict__ bias, const float* residual, TC* C,
                                                int N, int m0, int n0, int rows, long long ldc, long long ldr) {
    constexpr int QUADS = BN / 4;                         // groups of four columns in a row of the tile
    constexpr long long PART = (long long)TC_BM * BN;
    const bool wide_ok = (ldc % 4 == 0) && (((uintptr_t)C) % 16 == 0);
    for (int f = who; f < rows * QUADS; f += n_threads) {
        const int row = f / QUADS, col = 4 * (f % QUADS);
        const int n = n0 + col;
        if (n >= N) continue;
        const float* src = ws_tile + (long long)row * BN + col;
        float4 part[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
            part[sp] = sp < splits ? __ldcg(reinterpret_cast<const float4*>(src + sp * PART))
                                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float v[4] = {part[0].x, part[0].y, part[0].z, part[0].w};
#pragma unroll
        for (int sp = 1; sp < 8; ++sp)
            if (sp < splits) { v[0] += part[sp].x; v[1] += part[sp].y; v[2] += part[sp].z; v[3] += part[sp].w; }
        for (int sp = 8; sp < splits; ++sp) {
            const float4 more = __ldcg(reinterpret_cast<const float4*>(src + sp * PART));
            v[0] += more.x; v[1] += more.y; v[2] += more.z; v[3] += more.w;
        }
        const long long m = m0 + row;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const bool live = n + e < N;
            const float b = (bias && live) ? bias[n + e] : 0.0f;
            const float r = (residual && live) ? residual[m * ldr + n + e] : 0.0f;
            v[e] = r + tc_act<ACT>(v[e] + b, sizeof(TC) == 2);
        }
        TC* dst = C + m * ldc + n;
        if (wide_ok && n + 3 < N) {
            if (sizeof(TC) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = packed;
            } else {
                *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (n + e < N) dst[e] = from_float<TC>(v[e]);
        }
    }
}

// KSUB: 64-deep sub-tiles per stage (a stage is 64 * KSUB deep: with two, the issuing thread waits and
// commits half as often, which pays where the products are narrow and issuing them sets the pace).
template <int BN, int STAGES, int KSUB>
struct TcSmem {
    __nv_bfloat16 a[STAGES][KSUB][TC_BM * TC_BK];      // each sub-tile 1024-byte aligned: rows of 128 bytes
    __nv_bfloat16 b[STAGES][KSUB][BN * TC_BK];
    // where each epilogue warp turns a 32 x 32 block before it stores it, or lays it out row after row for a bulk
    // store: 4,224 bytes each, a multiple of 128 (what a bulk store's source must be aligned to)
    alignas(128) float patch[TC_EPI_WARPS][32 * TC_PATCH_PITCH];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];                        // an accumulator is complete (tensor cores -> epilogue)
    uint64_t acc_empty[2];                       // an accumulator has been read out (epilogue -> tensor cores)
    uint64_t split_stored;                       // all epilogue warps have left their part in the workspace
    uint64_t split_decided;                      // ... and one of them has drawn the tile's ticket
    uint32_t tmem_base;
    int split_last;                              // this block drew the last ticket: it finishes the tile
};

// Persistent: a block per SM walks over the tiles of C (tile = block, block + grid, ...); the ring of
// shared-memory stages runs on across tiles, and two accumulators in tensor memory take turns, so the
// read-out and the stores of one tile overlap the products of the next.
// SPLIT: the variant for products cut along K (see the top of the file); without it `splits` is 1.
template <int BN, int STAGES, int KSUB, typename TC, bool SPLIT>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, const float* __restrict__ bias, const float* residual, TC* C,
               int M, int N, int K, long long ldc, long long ldr, int act, int* status, int splits, float* split_ws,
               int* split_tickets, int bulk_out) {
    extern __shared__ unsigned char tc_raw[];
    TcSmem<BN, STAGES, KSUB>& sm =
        *reinterpret_cast<TcSmem<BN, STAGES, KSUB>*>(((uintptr_t)tc_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (!SPLIT) splits = 1;
    const int num_kb = (K + KSUB * TC_BK - 1) / (KSUB * TC_BK);          // a sub-tile past K is zero-filled
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles * splits;        // work items: (tile, part of K), parts of a tile side by side
    constexpr uint32_t STAGE_BYTES = KSUB * (TC_BM + BN) * TC_BK * sizeof(__nv_bfloat16);
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    bool ok = true;

    if (threadIdx.x == 0) {
        tma_prefetch_map(&map_a);
        tma_prefetch_map(&map_w);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], TC_EPI_WARPS); }
        mbar_init(&sm.split_stored, TC_EPI_WARPS);
        mbar_init(&sm.split_decided, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;
    pdl_trigger();
    pdl_wait();                                  // barriers and tensor memory are set up while the kernel before ends

    // consecutive tiles share a column block of W and differ in their rows of A, so the blocks that
    // run at the same time read few distinct tiles of either operand
    if (warp == 0) {
        if (lane == 0) {
            long long it = 0, issued = 0;
            int local = 0;
            for (int item = blockIdx.x; item < tiles && ok; item += gridDim.x, ++local) {
                const int tile = item / splits, part = item - tile * splits;
                const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
                const int kb_begin = (int)((long long)num_kb * part / splits);
                const int kb_end = (int)((long long)num_kb * (part + 1) / splits);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    ok = mbar_wait(&sm.empty[s], (uint32_t)(((it / STAGES) & 1) ^ 1));   // passes at once the first time round
                    if (!ok) break;
                    mbar_expect_tx(&sm.full[s], STAGE_BYTES);
#pragma unroll
                    for (int u = 0; u < KSUB; ++u) {
                        tma_load_2d(sm.a[s][u], &map_a, (kb * KSUB + u) * TC_BK, m0, &sm.full[s]);
                        tma_load_2d(sm.b[s][u], &map_w, (kb * KSUB + u) * TC_BK, n0, &sm.full[s]);
                    }
                    issued = it + 1;
                }
            }
            if (!ok) {
                atomicExch(status, 1);
                // let the copies already under way land before the block goes away
                for (long long j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j)
                    mbar_wait(&sm.full[j % STAGES], (uint32_t)((j / STAGES) & 1));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TC_BM, BN);
            // The descriptors of stage 0, sub-tile 0, k = 0; every other operand tile is a fixed number of
            // 16-byte units further on (the address sits in the low bits of the descriptor), so that one
            // issuing thread, whose every instruction waits for the one before, spends an addition per
            // operand and not a dozen instructions building it.
            const uint64_t a_desc0 = smem_desc_sw128(smem_u32(sm.a[0][0]));
            const uint64_t b_desc0 = smem_desc_sw128(smem_u32(sm.b[0][0]));
            constexpr uint32_t A_SUB = TC_BM * TC_BK * sizeof(__nv_bfloat16) / 16, B_SUB = BN * TC_BK * sizeof(__nv_bfloat16) / 16;
            long long it = 0;
            int local = 0;
            for (int item = blockIdx.x; item < tiles && ok; item += gridDim.x, ++local) {
                const int buf = local & 1;
                const int part = item % splits;
                const int kb_begin = (int)((long long)num_kb * part / splits);
                const int kb_end = (int)((long long)num_kb * (part + 1) / splits);
                ok = mbar_wait(&sm.acc_empty[buf], (uint32_t)(((local >> 1) & 1) ^ 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    ok = mbar_wait(&sm.full[s], (uint32_t)((it / STAGES) & 1));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t a_stage = a_desc0 + (uint64_t)((uint32_t)s * (KSUB * A_SUB));
                    const uint64_t b_stage = b_desc0 + (uint64_t)((uint32_t)s * (KSUB * B_SUB));
#pragma unroll
                    for (int u = 0; u < KSUB; ++u) {
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k) {
                            // 16 elements of k = 32 bytes (two units) further along the swizzled 128-byte rows
                            umma_bf16(tmem_d, a_stage + (uint64_t)(u * A_SUB + 2 * k), b_stage + (uint64_t)(u * B_SUB + 2 * k),
                                      idesc, (kb > kb_begin || u > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&sm.empty[s]);            // the stage is free once these have read it
                }
                if (ok) umma_commit(&sm.acc_full[buf]);   // the accumulator is complete
            }
            if (!ok) atomicExch(status, 2);
        }
    } else {
        // epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31; two warps share each
        // quarter of the rows and take half of the columns each, so that every scheduler of the SM
        // has two epilogue warps to switch between.  tcgen05.ld hands every thread one row of a 32 x 32
        // block.
        const int quad = warp & 3;
        const int half = (warp - 2) / 4;
        constexpr int COLS = BN / (TC_EPI_WARPS / 4);
        float* patch = sm.patch[warp - 2];
        constexpr int CHUNKS = COLS / 32;
        const bool vec_ok = sizeof(TC) == 2 && ((ldc * sizeof(TC)) % 16 == 0) && (((uintptr_t)C) % 16 == 0) && !residual &&
                            (((uintptr_t)bias) % 16 == 0);
        int local = 0;
        for (int item = blockIdx.x; item < tiles && ok; item += gridDim.x, ++local) {
            const int buf = local & 1;
            const int tile = item / splits;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
            const int row0 = m0 + quad * 32;
            // float32 path: the bias of this lane's columns, fetched while the tensor cores are still at work
            // lane-per-column path: one value per block; packed path: the lane's eight columns of every block
            float bias_col[CHUNKS][8];
#pragma unroll
            for (int q = 0; q < CHUNKS; ++q) {
                const int nq = n0 + half * COLS + 32 * q;
                if (vec_ok && nq + 32 <= N) {
                    const float4* b4 = reinterpret_cast<const float4*>(bias + nq + 8 * (lane & 3));
                    const float4 lo = bias ? b4[0] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    const float4 hi = bias ? b4[1] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    bias_col[q][0] = lo.x; bias_col[q][1] = lo.y; bias_col[q][2] = lo.z; bias_col[q][3] = lo.w;
                    bias_col[q][4] = hi.x; bias_col[q][5] = hi.y; bias_col[q][6] = hi.z; bias_col[q][7] = hi.w;
                } else {
                    bias_col[q][0] = (bias && nq + lane < N) ? bias[nq + lane] : 0.0f;
                }
            }
            ok = mbar_wait(&sm.acc_full[buf], (uint32_t)((local >> 1) & 1));
            if (!ok) {
                if (lane == 0) atomicExch(status, 3);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // (asking for the next block before this one is finished measured slower)
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + half * COLS);
            if constexpr (SPLIT) {
                // a part of K: leave it in the workspace, draw the tile's ticket, and finish the tile if
                // it was the last one
                const int n_rows = min(32, M - row0);                 // may be <= 0: nothing of this warp's is real
                float* ws_tile = split_ws + (long long)tile * splits * (TC_BM * BN);
                float* ws_mine = ws_tile + (long long)(item - tile * splits) * (TC_BM * BN) + (quad * 32) * BN + half * COLS;
#pragma unroll
                for (int q = 0; q < CHUNKS; ++q) {
                    uint32_t r[32];
                    tmem_ld_32x32(acc_addr + 32 * q, r);
                    if (q == CHUNKS - 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
                    }
                    if (n_rows > 0 && n0 + half * COLS + 32 * q < N)
                        tc_store_partial(r, patch, lane, ws_mine + 32 * q, BN, n_rows);
                }
                __threadfence();                                      // the part is out before the ticket is drawn
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.split_stored);
                const uint32_t phase = (uint32_t)(local & 1);
                if (warp == 2) {
                    const bool all_stored = mbar_wait(&sm.split_stored, phase);
                    if (lane == 0) {
                        int last = 0;
                        if (all_stored) {
                            last = atomicAdd(&split_tickets[tile], 1) == splits - 1;
                            if (last) split_tickets[tile] = 0;        // as the next launch expects it
                            __threadfence();
                        }
                        sm.split_last = last;
                        mbar_arrive(&sm.split_decided);
                    }
                    __syncwarp();
                    if (!all_stored) ok = false;
                }
                if (!mbar_wait(&sm.split_decided, phase)) ok = false;
                const int last = sm.split_last;
                if (!ok) {
                    if (lane == 0) atomicExch(status, 3);
                    break;
                }
                if (last) {
                    __threadfence();
                    const int who = (int)threadIdx.x - 64, rows = min(TC_BM, M - m0);
                    if (act == ACT_GELU_NEW)
                        tc_finish_split<ACT_GELU_NEW, TC, BN>(ws_tile, splits, who, TC_EPI_WARPS * 32, bias, residual, C, N,
                                                              m0, n0, rows, ldc, ldr);
                    else if (act == ACT_GELU_ERF)
                        tc_finish_split<ACT_GELU_ERF, TC, BN>(ws_tile, splits, who, TC_EPI_WARPS * 32, bias, residual, C, N,
                                                              m0, n0, rows, ldc, ldr);
                    else
                        tc_finish_split<0, TC, BN>(ws_tile, splits, who, TC_EPI_WARPS * 32, bias, residual, C, N, m0, n0,
                                                   rows, ldc, ldr);
                }
            } else {
#pragma unroll
            for (int q = 0; q < CHUNKS; ++q) {
                const int c0 = half * COLS + 32 * q;
                uint32_t r[32];
                tmem_ld_32x32(acc_addr + 32 * q, r);
                if (q == CHUNKS - 1) {
                    // this warp has read all it needs of the accumulator: the tensor cores may have it back
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
                }
                const int nb = n0 + c0;
                if (row0 >= M || nb >= N) continue;                   // the same for the whole warp
                if (bulk_out) {
                    // bulk_out 1: stored; 2: added to the matrix that is there (the residual, in place)
                    if (act == ACT_GELU_NEW)
                        tc_finish_block_bulk<ACT_GELU_NEW, TC>(r, patch, lane, bias, &map_c, N, row0, nb, bulk_out == 2);
                    else if (act == ACT_GELU_ERF)
                        tc_finish_block_bulk<ACT_GELU_ERF, TC>(r, patch, lane, bias, &map_c, N, row0, nb, bulk_out == 2);
                    else
                        tc_finish_block_bulk<0, TC>(r, patch, lane, bias, &map_c, N, row0, nb, bulk_out == 2);
                    continue;
                }
                // the activation is the same for the whole launch: chosen here, outside the loops over the
                // elements (inside them the compiler evaluated every activation for every element)
                if (act == ACT_GELU_NEW)
                    tc_finish_block<ACT_GELU_NEW, TC>(r, patch, lane, bias, bias_col[q], residual, C, M, N,
                                                      row0, nb, ldc, ldr, vec_ok && nb + 32 <= N);
                else if (act == ACT_GELU_ERF)
                    tc_finish_block<ACT_GELU_ERF, TC>(r, patch, lane, bias, bias_col[q], residual, C, M, N,
                                                      row0, nb, ldc, ldr, vec_ok && nb + 32 <= N);
                else
                    tc_finish_block<0, TC>(r, patch, lane, bias, bias_col[q], residual, C, M, N, row0, nb,
                                           ldc, ldr, vec_ok && nb + 32 <= N);
            }
            }
        }
    }
    if (bulk_out && warp >= 2 && lane == 0) tma_store_wait_all();      // this warp's bulk stores have landed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Where the parts of split products go (mu_gemm_tc_split_workspace); one device and one stream at a time
// use the library, as its status word already assumes.
struct SplitWorkspace {
    float* parts = nullptr;
    long long parts_bytes = 0;
    int* tickets = nullptr;
    int n_tickets = 0;
};
extern SplitWorkspace g_split;

template <int BN, int STAGES, int KSUB, typename TC, bool SPLIT>
static int launch_tc(const void* A, const void* W, const float* bias, const float* residual, TC* C, int M, int N,
                     int K, long long lda, long long ldw, long long ldc, long long ldr, int act, int* status,
                     int splits, cudaStream_t s) {
    CUtensorMap map_a, map_w, map_c;
    if (!tensor_map_bf16(&map_a, A, M, K, lda, TC_BM) || !tensor_map_bf16(&map_w, W, N, K, ldw, BN)) return MU_ERR_LAUNCH;
    // The epilogue hands whole 32 x 32 boxes to the copy engine where the output allows it (16-byte aligned
    // rows) and the residual, if any, is the output itself (then the boxes are added in place); products cut
    // along K finish their tiles from the workspace instead.
    int bulk_out = 0;
    if (!SPLIT && (((uintptr_t)C) & 15) == 0 && (ldc * (long long)sizeof(TC)) % 16 == 0 &&
        (residual == nullptr || (sizeof(TC) == 4 && (const void*)residual == (const void*)C && ldr == ldc)) &&
        tensor_map_out(&map_c, C, M, N, ldc, sizeof(TC) == 2))
        bulk_out = residual ? 2 : 1;
    if (!bulk_out) map_c = map_a;                    // a valid descriptor that is never used
    auto kernel = gemm_tc_kernel<BN, STAGES, KSUB, TC, SPLIT>;
    const size_t smem = sizeof(TcSmem<BN, STAGES, KSUB>) + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MU_ERR_LAUNCH;
        prefer_shared_memory(reinterpret_cast<const void*>(kernel));
        raised = true;
    }
    const int sms = sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    const int num_kb = (K + KSUB * TC_BK - 1) / (KSUB * TC_BK);
    if (SPLIT) {
        // the caller has checked these: every part has at least one stage of products, and the workspace holds
        // a partial tile per work item and a ticket per tile
        if (splits < 1 || splits > num_kb || !g_split.parts || tiles > g_split.n_tickets ||
            tiles * splits * (long long)(TC_BM * BN * sizeof(float)) > g_split.parts_bytes)
            return MU_ERR_BAD_ARGUMENT;
    } else {
        splits = 1;
    }
    const long long items = tiles * splits;
    dim3 grid((unsigned)(items < sms ? items : sms));
    return launch_pdl(kernel, grid, dim3(TC_THREADS), smem, s, 1, map_a, map_w, map_c, bias, residual, C, M, N, K, ldc, ldr,
                      act, status, splits, g_split.parts, g_split.tickets, bulk_out);
}

}  // namespace mu
