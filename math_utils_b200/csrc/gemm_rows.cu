// C[M, N] = act(A[M, K] . W[N, K]^T + bias) (+ residual) for up to 64 rows, on the 5th-generation tensor
// cores, with the WEIGHTS as the 128-row operand of the instruction and the batch as its narrow side.
//
// A step of 17 to 64 single tokens reads each weight once and does almost no arithmetic.  What bounds it is
// how many weight bytes a block turns over per tcgen05.mma it issues (one thread issues them, some hundred
// cycles apart) and how many SMs pull weights at the same time.  So:
//   * a tile is 128 rows of W (128 output columns) by all M rows of A: D[128, NB] = W_tile . A^T with
//     NB = M rounded up to 16, 32 or 64; one instruction covers 128 x 16 weights (4 KB);
//   * tiles are few (18 for 2,304 outputs), so K is cut over the blocks of a thread-block cluster (up to 16
//     where the device allows it): tiles x splits blocks fill the SMs, and a block issues K / splits / 16
//     instructions, a handful;
//   * the partial accumulators meet on chip: every block of the cluster owns 128 / splits of the tile's
//     output columns; a block lays its partial tile out in shared memory and sends each owner its share with
//     one bulk copy through distributed shared memory (cp.async.bulk.shared::cluster, counted by the owner's
//     mbarrier); the owner adds the shares in rank order, so the sum does not depend on timing, finishes its
//     columns (bias, activation, residual) and stores them; no trip through the L2, no ticket, no block
//     that only waits;
//   * a block asks for its whole share of K at once where it fits (a ring of k-blocks of 64: 128 rows of W
//     and NB rows of A by TMA with the 128-byte swizzle); the weight copies are issued before the wait for
//     the kernel before (weights are written by no kernel), the activation copies right after it;
//   * warp 0 issues the copies, warp 1 owns the tensor memory and issues tcgen05.mma, warps 2-5 read the
//     accumulator (tcgen05.ld: a thread per output column, the batch along its registers), so stores of one
//     batch row by a warp cover 32 consecutive columns.
// Every wait on an mbarrier is bounded and reports through `status` (codes 1-3 as the large product kernel);
// a block whose wait ran out still passes the cluster barriers, so nobody hangs on it.
//
// The reference's counterpart is matmulNTBias (include/ai/Kernels.hpp:433-447).
#include "tcgen05.cuh"

namespace mu {

constexpr int GR_BM = 128;                       // rows of W (output columns) per tile
constexpr int GR_BK = 64;                        // elements of k per stage: one 128-byte swizzled row
constexpr int GR_MAX_ROWS = 64;                  // rows of A (the batch)
constexpr int GR_THREADS = 192;                  // loader, issuer, four epilogue warps
constexpr int GR_MAX_SPLIT = 16;
constexpr uint32_t GR_W_BYTES = GR_BM * GR_BK * sizeof(__nv_bfloat16);          // 16 KB

template <int NB> __device__ __forceinline__ void tmem_ld_row(uint32_t taddr, uint32_t (&r)[NB]);
template <> __device__ __forceinline__ void tmem_ld_row<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
template <> __device__ __forceinline__ void tmem_ld_row<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_32x32(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_row<64>(uint32_t taddr, uint32_t (&r)[64]) {
    uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
    uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
    tmem_ld_32x32_nowait(taddr, lo);
    tmem_ld_32x32_nowait(taddr + 32, hi);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ float gr_act(float x, int act, bool to_bf16) {
    if (act == ACT_GELU_NEW) return to_bf16 ? gelu_new_fast(x) : gelu_new(x);
    if (act == ACT_GELU_ERF) return gelu_erf(x);
    return x;
}

// grid.x = tiles * splits; the blocks of a cluster (splits of them, along x; a power of two up to 16) share a
// tile and cut K.  Dynamic shared memory, 1024-byte aligned: stages x [W 16 KB], stages x [A NB x 128 B], and
// with splits > 1 the shares this block is sent and its own partial tile, each [128][NB + 4] float32 at most.
template <int NB, typename TC>
__global__ void __launch_bounds__(GR_THREADS)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const float* __restrict__ bias, const float* residual, TC* C, int M, int N, int K,
                 long long ldc, long long ldr, int act, int* status, int splits, int stages, int outbox_on_stages) {
    constexpr uint32_t A_BYTES = NB * GR_BK * sizeof(__nv_bfloat16);
    extern __shared__ unsigned char gr_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)gr_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* w_smem = base;                                                 // [stages][16 KB]
    unsigned char* a_smem = w_smem + (size_t)stages * GR_W_BYTES;                 // [stages][NB x 128 B]
    float* part = reinterpret_cast<float*>(a_smem + (size_t)stages * A_BYTES);    // [splits][128 / splits][pitch]: shares sent here
    // [128][pitch]: this block's partial tile; written when the stages are no longer read, so it may lie on them
    float* outbox = outbox_on_stages ? reinterpret_cast<float*>(base) : part + (size_t)GR_BM * (NB + 4);
    __shared__ uint64_t full[32], empty[32], acc_full, parts_in;
    __shared__ uint32_t tmem_slot;
    __shared__ float bias_s[GR_BM];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = splits > 1 ? (int)cluster_rank() : 0;
    const int tile = blockIdx.x / splits;
    const int n0 = tile * GR_BM;
    const int num_kb = (K + GR_BK - 1) / GR_BK;
    const int kb_begin = (int)((long long)num_kb * rank / splits);
    const int kb_end = (int)((long long)num_kb * (rank + 1) / splits);
    const int my_kb = kb_end - kb_begin;                      // at least one: the host keeps splits <= num_kb
    bool ok = true;

    if (threadIdx.x == 0) {
        tma_prefetch_map(&map_a);
        tma_prefetch_map(&map_w);
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&parts_in, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)(NB < 32 ? 32 : NB)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (threadIdx.x >= 64) {                                  // the bias is a weight: it may be read at once
        const int n = n0 + (int)threadIdx.x - 64;
        bias_s[threadIdx.x - 64] = (bias && n < N) ? bias[n] : 0.0f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_slot;
    pdl_trigger();
    // every block of the cluster is running before anyone writes into another's shared memory
    if (splits > 1) cluster_arrive();

    if (warp == 0) {
        if (lane == 0) {
            const int first = my_kb < stages ? my_kb : stages;
            // weights are written by no kernel: their copies set off before the wait for the kernel before
            for (int i = 0; i < first; ++i) {
                mbar_expect_tx(&full[i], GR_W_BYTES + A_BYTES);
                tma_load_2d(w_smem + (size_t)i * GR_W_BYTES, &map_w, (kb_begin + i) * GR_BK, n0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < first; ++i)
                tma_load_2d(a_smem + (size_t)i * A_BYTES, &map_a, (kb_begin + i) * GR_BK, 0, &full[i]);
            int issued = first;
            for (int i = first; i < my_kb && ok; ++i) {
                const int s = i % stages;
                ok = mbar_wait(&empty[s], (uint32_t)((i / stages - 1) & 1));
                if (!ok) break;
                mbar_expect_tx(&full[s], GR_W_BYTES + A_BYTES);
                tma_load_2d(w_smem + (size_t)s * GR_W_BYTES, &map_w, (kb_begin + i) * GR_BK, n0, &full[s]);
                tma_load_2d(a_smem + (size_t)s * A_BYTES, &map_a, (kb_begin + i) * GR_BK, 0, &full[s]);
                issued = i + 1;
            }
            if (!ok) {
                atomicExch(status, 1);
                // let the copies already under way land before the block goes away
                for (int j = issued > stages ? issued - stages : 0; j < issued; ++j)
                    mbar_wait(&full[j % stages], (uint32_t)((j / stages) & 1));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(GR_BM, NB);
            for (int i = 0; i < my_kb && ok; ++i) {
                const int s = i % stages;
                ok = mbar_wait(&full[s], (uint32_t)((i / stages) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t w_addr = smem_u32(w_smem + (size_t)s * GR_W_BYTES);
                const uint32_t a_addr = smem_u32(a_smem + (size_t)s * A_BYTES);
#pragma unroll
                for (int k = 0; k < GR_BK / 16; ++k)      // the weights are the instruction's 128-row operand
                    umma_bf16(tmem_acc, smem_desc_sw128(w_addr + k * 32), smem_desc_sw128(a_addr + k * 32), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(&acc_full);
            else atomicExch(status, 2);
        }
    } else {
        // epilogue warps: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31; a lane is an output column
        const int quad = warp & 3;
        const int col = quad * 32 + lane;                   // the tile's column this thread holds: n0 + col
        float acc[NB];
        ok = mbar_wait(&acc_full, 0);
        if (!ok) {
            if (lane == 0) atomicExch(status, 3);
#pragma unroll
            for (int m = 0; m < NB; ++m) acc[m] = 0.0f;
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[NB];
            tmem_ld_row<NB>(tmem_acc + ((uint32_t)(quad * 32) << 16), r);
#pragma unroll
            for (int m = 0; m < NB; ++m) acc[m] = __uint_as_float(r[m]);
        }
        if (splits == 1) {
            const int n = n0 + col;
            if (ok && n < N) {
                pdl_wait();                                 // the residual is the work of earlier kernels
                const float b = bias_s[col];
                const bool to_bf16 = sizeof(TC) == 2;
                // all of the residual is asked for before anything is stored: it may be C itself, and a load
                // that had to wait for the store before it would make the rows a chain of round trips
                float res[NB];
#pragma unroll
                for (int m = 0; m < NB; ++m) res[m] = (residual && m < M) ? residual[(long long)m * ldr + n] : 0.0f;
#pragma unroll
                for (int m = 0; m < NB; ++m)
                    if (m < M) C[(long long)m * ldc + n] = from_float<TC>(gr_act(acc[m] + b, act, to_bf16) + res[m]);
            }
        } else {
            const int cols_per = GR_BM / splits;            // output columns each block of the cluster finishes
            const int groups = (M + 3) / 4;                 // batch rows travel four at a time
            const int pitch = 4 * groups + 4;               // floats between columns: rows of 16 bytes, and the
                                                            // reads below spread over all the banks
            const uint32_t slice_bytes = (uint32_t)(cols_per * pitch) * 4u;     // one block's share of a part
            // this thread's partial column goes to the outbox, where the columns of each owner lie together
            {
                float* mine = outbox + (size_t)col * pitch;
#pragma unroll
                for (int g = 0; g < NB / 4; ++g)
                    if (g < groups)
                        *reinterpret_cast<float4*>(mine + 4 * g) = make_float4(acc[4 * g], acc[4 * g + 1], acc[4 * g + 2], acc[4 * g + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");        // the copies below read what was stored here
            asm volatile("bar.sync 1, 128;" ::: "memory");                      // the four epilogue warps
            __syncwarp();
            cluster_wait();                                 // (the arrive was at the top) everyone is running
            if (threadIdx.x == 64) {
                // what the others will send: splits - 1 shares; then this block's shares set off, one bulk copy
                // per owner, into part[this block's rank] of the owner, counted by the owner's barrier
                mbar_expect_tx(&parts_in, (uint32_t)(splits - 1) * slice_bytes);
                for (int step = 1; step < splits; ++step) {
                    const int owner = (rank + step) % splits;                   // not everyone at the same owner first
                    uint32_t dst, bar;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                                 : "=r"(dst) : "r"(smem_u32(part + (size_t)rank * cols_per * pitch)), "r"(owner));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(smem_u32(&parts_in)), "r"(owner));
                    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dst), "r"(smem_u32(outbox + (size_t)owner * cols_per * pitch)), "r"(slice_bytes), "r"(bar)
                                 : "memory");
                }
            }
            const bool arrived = mbar_wait(&parts_in, 0);   // every share for this block's columns is here
            if (!arrived && lane == 0) atomicExch(status, 3);
            __syncwarp();
            cluster_arrive();                               // (waited for before the block ends: see below)
            pdl_wait();
            const bool to_bf16 = sizeof(TC) == 2;
            const int who = (int)threadIdx.x - 64, total = groups * cols_per;
            // an item is four batch rows of one column; consecutive threads take consecutive columns, so a
            // warp's stores of one batch row cover a run of columns
            for (int idx = who; idx < total && arrived; idx += 128) {
                const int g = idx / cols_per, i = idx - g * cols_per;
                const int c = rank * cols_per + i, n = n0 + c;
                if (n >= N) continue;
                float res[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)                 // asked for before anything is stored (it may be C itself)
                    res[e] = (residual && 4 * g + e < M) ? residual[(long long)(4 * g + e) * ldr + n] : 0.0f;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int r = 0; r < splits; ++r) {          // in rank order, whoever sent when
                    const float* src = r == rank ? outbox + (size_t)c * pitch : part + ((size_t)r * cols_per + i) * pitch;
                    const float4 p = *reinterpret_cast<const float4*>(src + 4 * g);
                    v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                }
                const float b = bias_s[c];
                const float out4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (4 * g + e < M)
                        C[(long long)(4 * g + e) * ldc + n] = from_float<TC>(gr_act(out4[e] + b, act, to_bf16) + res[e]);
            }
            // nobody leaves while a copy may still read its outbox: once every block has seen all of its
            // shares arrive, every copy of every block is complete
            __syncwarp();
            cluster_wait();
        }
    }
    if (splits > 1 && warp < 2) {
        // the loader and the issuer pass the same two cluster barriers as the epilogue warps
        __syncwarp();
        cluster_wait();
        cluster_arrive();
        cluster_wait();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_acc), "r"((uint32_t)(NB < 32 ? 32 : NB)) : "memory");
    }
}

template <int NB, typename TC>
static int launch_rows(const CUtensorMap& map_a, const CUtensorMap& map_w, const float* bias, const float* residual,
                       TC* C, int M, int N, int K, long long ldc, long long ldr, int act, int* status, int splits,
                       int stages, int outbox_on_stages, size_t smem, cudaStream_t s) {
    auto kernel = gemm_rows_kernel<NB, TC>;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
            return MU_ERR_LAUNCH;
        // clusters of 16 are beyond the portable size: allowed on this device if it says so
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaGetLastError();
        raised = true;
    }
    const int tiles = (N + GR_BM - 1) / GR_BM;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * splits));
    cfg.blockDim = dim3(GR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (splits > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)splits;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, map_a, map_w, bias, residual, C, M, N, K, ldc, ldr, act, status, splits,
                              stages, outbox_on_stages) == cudaSuccess ? MU_OK : MU_ERR_LAUNCH;
}

// Whether clusters of 16 blocks of this kernel can be scheduled here (asked once).
static int max_cluster() {
    static int limit = 0;
    if (limit == 0) {
        limit = 8;
        auto kernel = gemm_rows_kernel<64, float>;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) == cudaSuccess &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(16);
            cfg.blockDim = dim3(GR_THREADS);
            cfg.dynamicSmemBytes = 96 * 1024;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 16;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters > 0) limit = 16;
        }
        cudaGetLastError();
    }
    return limit;
}

}  // namespace mu

// bfloat16 A [M, K] (lda) with M <= 64 and W [N, K] (ldw): K, lda, ldw multiples of 8, bases 16-byte aligned.
// C bfloat16 or float32 (ldc); residual float32 (ldr), may be C itself.  splits: blocks that share a tile of
// 128 output columns and cut K (a power of two up to 16; 0: chosen here so that tiles x splits fill the SMs).
// `status` as mu_gemm_tc.
MU_EXPORT int mu_gemm_rows(const void* A, const void* W, const float* bias, const float* residual, void* C,
                           int M, int N, int K, long long lda, long long ldw, long long ldc, long long ldr,
                           int act, int out_bf16, int splits, int* status, void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (M > mu::GR_MAX_ROWS) return MU_ERR_UNSUPPORTED_SIZE;
    if (K <= 0 || !A || !W || !C || !status) return MU_ERR_BAD_ARGUMENT;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return MU_ERR_ALIGNMENT;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return MU_ERR_ALIGNMENT;
    if (lda < K || ldw < K || ldc < N || (residual && ldr < N)) return MU_ERR_BAD_ARGUMENT;
    if (splits < 0 || splits > mu::GR_MAX_SPLIT || (splits & (splits - 1))) return MU_ERR_BAD_ARGUMENT;
    const int sms = mu::sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    const long long tiles = (N + mu::GR_BM - 1) / mu::GR_BM;
    const int num_kb = (K + mu::GR_BK - 1) / mu::GR_BK;
    if (tiles * mu::GR_MAX_SPLIT > 2147483647ll) return MU_ERR_UNSUPPORTED_SIZE;
    const int limit = mu::max_cluster();
    if (splits == 0) {
        // the largest power of two that keeps tiles x splits within the SMs (and a third more: two blocks
        // share an SM) and a k-block for every block
        splits = 1;
        while (splits * 2 <= limit && tiles * splits * 2 <= sms + sms / 3 && splits * 2 <= num_kb) splits *= 2;
        // a block that would stream more than 128 KB of weights through its ring is cut once more, up to two
        // blocks an SM: with that much to read, bytes in flight count for more than a short exchange of parts
        const long long block_bytes = (long long)mu::GR_BM * K * (long long)sizeof(__nv_bfloat16) / splits;
        if (block_bytes > 128 * 1024 && splits * 2 <= limit && splits * 2 <= num_kb && tiles * splits * 2 <= 2ll * sms)
            splits *= 2;
    }
    while (splits > limit || splits > num_kb) splits /= 2;
    const int nb = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    const size_t stage_bytes = mu::GR_W_BYTES + (size_t)nb * mu::GR_BK * sizeof(__nv_bfloat16);
    const size_t tile_bytes = (size_t)(nb + 4) * mu::GR_BM * sizeof(float);      // a partial tile as it travels
    // A ring as long as a block's share of K where that fits (everything in flight at once), but no more
    // shared memory than lets two blocks share an SM: then the blocks of the next kernel are in place, their
    // weights on the way, while this one ends.  With splits, room for the shares sent here, and for this
    // block's own partial tile unless it fits on the stages (it is written when they are no longer read).
    const int per_block = (num_kb + splits - 1) / splits;
    const size_t room = 108 * 1024;
    size_t fixed = 1024 + (splits > 1 ? tile_bytes : 0);
    int stages = (int)((room - fixed) / stage_bytes);
    if (stages > per_block) stages = per_block;
    if (stages > 32) stages = 32;
    if (stages < 1) return MU_ERR_UNSUPPORTED_SIZE;
    int outbox_on_stages = 0;
    if (splits > 1) {
        outbox_on_stages = (size_t)stages * stage_bytes >= tile_bytes;
        if (!outbox_on_stages) {
            fixed += tile_bytes;
            while (stages > 1 && fixed + (size_t)stages * stage_bytes > room) --stages;
        }
    }
    const size_t smem = fixed + (size_t)stages * stage_bytes;
    CUtensorMap map_a, map_w;
    if (!mu::tensor_map_bf16(&map_a, A, M, K, lda, nb) || !mu::tensor_map_bf16(&map_w, W, N, K, ldw, mu::GR_BM))
        return MU_ERR_LAUNCH;
    cudaStream_t s = (cudaStream_t)stream;
#define MU_ROWS(NB)                                                                                                  \
    (out_bf16 ? mu::launch_rows<NB, __nv_bfloat16>(map_a, map_w, bias, residual, (__nv_bfloat16*)C, M, N, K, ldc, ldr, \
                                                   act, status, splits, stages, outbox_on_stages, smem, s)            \
              : mu::launch_rows<NB, float>(map_a, map_w, bias, residual, (float*)C, M, N, K, ldc, ldr, act, status,   \
                                           splits, stages, outbox_on_stages, smem, s))
    if (nb == 16) return MU_ROWS(16);
    if (nb == 32) return MU_ROWS(32);
    return MU_ROWS(64);
#undef MU_ROWS
}
