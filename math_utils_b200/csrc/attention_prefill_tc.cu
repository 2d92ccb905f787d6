// Causal attention of whole prompts over the paged cache on the 5th-generation tensor cores
// (bfloat16, head size 64, pages of 64 positions).
//
// A block takes up to 128 consecutive query tokens of one sequence and one head and walks the
// sequence's cache pages.  Both products of a page run as tcgen05.mma with the accumulators in tensor
// memory, and the operands come by TMA in the layout the instruction reads:
//   S = Q K^T   Q [128 queries][64 dims] is loaded once; a page's keys are [64 positions][64 dims],
//               64 contiguous rows of the cache: the right operand, K-major, as it lies;
//   O = P V     a page's values lie dimension-major in the cache, [64 dims][64 positions]: again the
//               right operand, K-major, as it lies.  P is written by the softmax threads into shared
//               memory in the 128-byte-swizzled layout the left operand wants.
// Roles: warp 0 loads queries and keys, warp 3 values, warp 1 owns tensor memory and issues S, warp 2 issues P V (one lane each:
// an issue costs the issuing thread some 80 cycles, so the two products of a page have a thread each), warps
// 4-11 are the softmax in two groups that take the tile's pages in turn: a thread of a group owns a query row
// (tcgen05.ld hands a thread a row, so maximum and sum need no shuffle), reads its 64 scores of the page
// from tensor memory, writes its row of P, and adds each of its pages' P V, which the tensor cores leave in a
// buffer of its own, into the float32 output row in its registers, scaled by the change of the running
// maximum; at the end the two groups' rows are merged.  A group has a score buffer and two P and P V buffers, so the products
// of the next page run while the softmax of this one is computed.
// Softmax, running maximum and sum, and the output accumulation are float32; P is rounded to bfloat16 for
// the second product, as in the mma.sync kernel (attention_prefill.cu), which stays for other head sizes.
// Every mbarrier wait is bounded; a wait that runs out sets *status (5 loads, 6 products, 7 softmax) and the
// block leaves without storing.
//
// Formulas: include/ai/Kernels.hpp:132-161.
#include "tcgen05.cuh"

#include <math.h>

namespace mu {

constexpr int PT_Q = 128;            // queries per block
constexpr int PT_K = 64;             // keys per page
constexpr int PT_D = 64;             // head size
constexpr int PT_STAGES = 3;         // pages of keys in flight
constexpr int PT_VSTAGES = 4;        // pages of values in flight (a page of values is held until its P V is complete)
constexpr int PT_THREADS = 384;      // key loader, two issuers, value loader, two groups of four softmax warps

struct PtSmem {
    __nv_bfloat16 q[PT_Q * PT_D];                    // 1024-byte aligned tiles, rows of 128 bytes, swizzled
    __nv_bfloat16 k[PT_STAGES][PT_K * PT_D];
    __nv_bfloat16 v[PT_VSTAGES][PT_D * PT_K];
    __nv_bfloat16 p[2][2][PT_Q * PT_K];              // per softmax group, two buffers that take turns
    uint64_t q_full;
    uint64_t k_full[PT_STAGES], k_empty[PT_STAGES];
    uint64_t v_full[PT_VSTAGES], v_empty[PT_VSTAGES];
    uint64_t s_full[2], s_free[2];                   // per group: scores ready (products -> softmax) / read
    uint64_t p_full[2][2];                           // per group and buffer: P written; free again when its P V is complete
    uint64_t pv_full[2][2], pv_free[2][2];           // per group and buffer: P V ready / read
    uint64_t x_full;                                 // the second group's rows are handed over
    float hand_ml[PT_Q][2];                          // ... their running maximum and sum (the outputs go where its P was)
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(PT_THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, long long ldo, const int* __restrict__ block_table,
                            int max_pages, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                            const int* __restrict__ tiles, int n_heads, int n_kv_heads, float scale, int window,
                            int* status) {
    extern __shared__ unsigned char pt_raw[];
    PtSmem& sm = *reinterpret_cast<PtSmem*>(((uintptr_t)pt_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x;
    const int tile = item / n_heads, h = item % n_heads, kvh = h / (n_heads / n_kv_heads);
    constexpr uint32_t TMEM_COLS = 512;              // scores of group g at 64 g; its P V buffers at 128 + 128 g + {0, 64}
    constexpr uint32_t PAGE_BYTES = PT_K * PT_D * sizeof(__nv_bfloat16);

    if (threadIdx.x == 0) {
        tma_prefetch_map(&map_q);
        tma_prefetch_map(&map_kv);
        mbar_init(&sm.q_full, 1);
        // (a stage is declared free by the four softmax warps that have seen the product that read it complete:
        // an arrival of theirs is cheaper than another commit of the issuing thread)
        for (int s = 0; s < PT_STAGES; ++s) { mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 4); }
        for (int s = 0; s < PT_VSTAGES; ++s) { mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 4); }
        for (int g = 0; g < 2; ++g) {
            mbar_init(&sm.s_full[g], 1); mbar_init(&sm.s_free[g], 4);
            for (int b = 0; b < 2; ++b) {
                mbar_init(&sm.p_full[g][b], 4);
                mbar_init(&sm.pv_full[g][b], 1); mbar_init(&sm.pv_free[g][b], 4);
            }
        }
        mbar_init(&sm.x_full, 4);
        sm.failed = 0;
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
    pdl_wait();                                      // queries and this step's cache rows come from the kernels before

    const int flat0 = tiles[2 * tile], nq = tiles[2 * tile + 1];
    const int pos0 = tok_pos[flat0];
    const int* pages = block_table + (long long)tok_seq[flat0] * max_pages;
    const int pos_last = pos0 + nq - 1;
    const int first_key = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int first_page = first_key / PT_K, last_page = pos_last / PT_K;
    const int n_pages = last_page - first_page + 1;
    bool ok = true;

    if (warp == 0) {
        // the queries, then the keys of every page (a loader of their own, so that keys, which are free again
        // as soon as the scores are computed, never wait behind values)
        if (lane == 0) {
            mbar_expect_tx(&sm.q_full, PT_Q * PT_D * sizeof(__nv_bfloat16));
            tma_load_2d(sm.q, &map_q, h * PT_D, flat0, &sm.q_full);
            int issued = 0;
            for (int j = 0; j < n_pages; ++j) {
                const int s = j % PT_STAGES;
                const long long page = pages[first_page + j];
                const int krow = (int)(((page * 2 + 0) * n_kv_heads + kvh) * PT_K);      // rows of 64 elements
                ok = mbar_wait_poll(&sm.k_empty[s], (uint32_t)(((j / PT_STAGES) & 1) ^ 1));
                if (!ok) break;
                mbar_expect_tx(&sm.k_full[s], PAGE_BYTES);
                tma_load_2d(sm.k[s], &map_kv, 0, krow, &sm.k_full[s]);
                issued = j + 1;
            }
            if (!ok) {
                atomicExch(status, 5);
                sm.failed = 1;
            }
            // every copy has landed before the block may go away (in the good case they have long been used)
            mbar_wait(&sm.q_full, 0);
            for (int j = issued > PT_STAGES ? issued - PT_STAGES : 0; j < issued; ++j)
                mbar_wait(&sm.k_full[j % PT_STAGES], (uint32_t)((j / PT_STAGES) & 1));
        }
    } else if (warp == 3) {
        // the values of every page
        if (lane == 0) {
            int issued = 0;
            for (int j = 0; j < n_pages; ++j) {
                const int s = j % PT_VSTAGES;
                const long long page = pages[first_page + j];
                const int vrow = (int)(((page * 2 + 1) * n_kv_heads + kvh) * PT_D);
                ok = mbar_wait_poll(&sm.v_empty[s], (uint32_t)(((j / PT_VSTAGES) & 1) ^ 1));
                if (!ok) break;
                mbar_expect_tx(&sm.v_full[s], PAGE_BYTES);
                tma_load_2d(sm.v[s], &map_kv, 0, vrow, &sm.v_full[s]);
                issued = j + 1;
            }
            if (!ok) {
                atomicExch(status, 5);
                sm.failed = 1;
            }
            for (int j = issued > PT_VSTAGES ? issued - PT_VSTAGES : 0; j < issued; ++j)
                mbar_wait(&sm.v_full[j % PT_VSTAGES], (uint32_t)((j / PT_VSTAGES) & 1));
        }
    } else if (warp == 1) {
        // S = Q K^T of every page into the score buffer of the page's softmax group
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(PT_Q, PT_K);
            const uint32_t q_addr = smem_u32(sm.q);
            ok = mbar_wait_poll(&sm.q_full, 0);
            for (int j = 0; j < n_pages && ok; ++j) {
                const int g = j & 1, u = j >> 1, s = j % PT_STAGES;
                ok = mbar_wait_poll(&sm.k_full[s], (uint32_t)((j / PT_STAGES) & 1));
                if (!ok) break;
                ok = mbar_wait_poll(&sm.s_free[g], (uint32_t)((u & 1) ^ 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = smem_u32(sm.k[s]);
#pragma unroll
                for (int k = 0; k < PT_D / 16; ++k)
                    umma_bf16(tmem_base + 64 * g, smem_desc_sw128(q_addr + k * 32), smem_desc_sw128(k_addr + k * 32), idesc,
                              k > 0 ? 1u : 0u);
                umma_commit(&sm.s_full[g]);
            }
            if (!ok) {
                atomicExch(status, 6);
                sm.failed = 1;
            }
        }
    } else if (warp == 2) {
        // O_page = P V of every page into one of the two P V buffers of the page's group
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(PT_Q, PT_D);
            for (int j = 0; j < n_pages && ok; ++j) {
                const int g = j & 1, u = j >> 1, b = u & 1, s = j % PT_VSTAGES;
                ok = mbar_wait_poll(&sm.p_full[g][b], (uint32_t)((u >> 1) & 1));
                if (!ok) break;
                ok = mbar_wait_poll(&sm.v_full[s], (uint32_t)((j / PT_VSTAGES) & 1));
                if (!ok) break;
                ok = mbar_wait_poll(&sm.pv_free[g][b], (uint32_t)(((u >> 1) & 1) ^ 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t p_addr = smem_u32(sm.p[g][b]), v_addr = smem_u32(sm.v[s]);
#pragma unroll
                for (int k = 0; k < PT_K / 16; ++k)
                    umma_bf16(tmem_base + 128 + 128 * g + 64 * b, smem_desc_sw128(p_addr + k * 32),
                              smem_desc_sw128(v_addr + k * 32), idesc, k > 0 ? 1u : 0u);
                umma_commit(&sm.pv_full[g][b]);
            }
            if (!ok) {
                atomicExch(status, 6);
                sm.failed = 1;
            }
        }
    } else {
        // softmax: two groups of four warps; group g takes the pages j = g, g + 2, ... of the tile; thread `row`
        // of a group owns query row `row`; at the end the second group hands its running maximum, sum and
        // output row to the first, which stores
        const int quad = warp & 3, grp = (warp - 4) >> 2;
        const int row = quad * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_col = 64 * grp, pv_col = 128 + 128 * grp;
        const int qpos = pos0 + row;
        const float c_log2 = scale * 1.4426950408889634f;      // scores are exponentiated in base 2
        float m_run = -INFINITY, l_run = 0.0f, corr_prev = 0.0f;
        float o[PT_D];
#pragma unroll
        for (int d = 0; d < PT_D; ++d) o[d] = 0.0f;
        const int n_mine = n_pages > grp ? (n_pages - grp + 1) / 2 : 0;      // pages of this group

        // P V of this group's u-th page joins the output row
        auto take_pv = [&](int u, float corr) -> bool {
            const int b = u & 1;
            if (!mbar_wait(&sm.pv_full[grp][b], (uint32_t)((u >> 1) & 1))) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r0[32], r1[32];
            tmem_ld_32x32_nowait(lane_base + pv_col + 64 * b, r0);
            tmem_ld_32x32_nowait(lane_base + pv_col + 64 * b + 32, r1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sm.pv_free[grp][b]);
                mbar_arrive(&sm.v_empty[(2 * u + grp) % PT_VSTAGES]);      // the product is complete: the values have been read
            }
#pragma unroll
            for (int d = 0; d < 32; ++d) {
                o[d] = fmaf(o[d], corr, __uint_as_float(r0[d]));
                o[32 + d] = fmaf(o[32 + d], corr, __uint_as_float(r1[d]));
            }
            return true;
        };

        for (int u = 0; u < n_mine; ++u) {
            const int j = 2 * u + grp, b = u & 1;
            const int key0 = (first_page + j) * PT_K;
            ok = mbar_wait(&sm.s_full[grp], (uint32_t)(u & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the row's 64 scores, in two pieces; the buffer is free for this group's next page right away
            uint32_t r[2][32];
            tmem_ld_32x32_nowait(lane_base + s_col, r[0]);
            tmem_ld_32x32_nowait(lane_base + s_col + 32, r[1]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sm.s_free[grp]);
                mbar_arrive(&sm.k_empty[j % PT_STAGES]);         // the scores are complete: the keys have been read
            }
            // columns [lo, hi] of the page are visible to this row (all 64 if the page lies before the tile)
            const int hi = min(qpos - key0, PT_K - 1);
            const int lo = window > 0 ? max(qpos - window + 1 - key0, 0) : 0;
            const bool plain = lo == 0 && hi == PT_K - 1;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    float sc = __uint_as_float(r[half][c]);
                    if (!plain && (32 * half + c < lo || 32 * half + c > hi)) sc = -INFINITY;
                    r[half][c] = __float_as_uint(sc);
                    mx4[c & 3] = fmaxf(mx4[c & 3], sc);
                }
            // maximum and exponent in units of scale * log2(e) (scale > 0)
            const float mx = fmaxf(m_run, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c_log2);
            const float base = (mx == -INFINITY) ? 0.0f : mx;          // a row that has seen no key yet
            const float corr = fast_exp2(m_run - base);
            m_run = mx;
            // P goes to buffer b of the group: the product that read it last (page u - 2) was taken in round u - 1
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            unsigned char* prow = reinterpret_cast<unsigned char*>(sm.p[grp][b]) + row * 128;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(r[half][c]), c_log2, -base));      // 0 for a hidden key
                    const float p1 = fast_exp2(fmaf(__uint_as_float(r[half][c + 1]), c_log2, -base));
                    sum4[(c >> 1) & 3] += p0 + p1;
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    r[half][c >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                }
                // 16-byte piece c of a row sits at piece (c ^ (row & 7)) of its 128 bytes
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int piece = (4 * half + c) ^ (row & 7);
                    *reinterpret_cast<uint4*>(prow + 16 * piece) =
                        make_uint4(r[half][4 * c], r[half][4 * c + 1], r[half][4 * c + 2], r[half][4 * c + 3]);
                }
            }
            l_run = fmaf(l_run, corr, (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the tensor cores read P through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full[grp][b]);
            // the group's page before this one: its P V joins the output row
            if (u >= 1) {
                ok = take_pv(u - 1, corr_prev);
                if (!ok) break;
            }
            corr_prev = corr;
        }
        if (ok && n_mine >= 1) ok = take_pv(n_mine - 1, corr_prev);
        if (!ok && lane == 0) {
            atomicExch(status, 7);
            sm.failed = 1;
        }
        // The second group's P buffers are free once it has taken its last P V; it leaves its output rows there
        float* hand = reinterpret_cast<float*>(sm.p[1][0]);             // [128][64] floats: 32 KB, both buffers
        const bool two = n_pages >= 2;
        if (grp == 1 && two) {
#pragma unroll
            for (int d = 0; d < PT_D; d += 4)
                *reinterpret_cast<float4*>(hand + ((d / 4) * PT_Q + row) * 4) = make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]);
            sm.hand_ml[row][0] = m_run;
            sm.hand_ml[row][1] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.x_full);
        }
        if (grp == 0) {
            float w0 = 1.0f, w1 = 0.0f, l1 = 0.0f;
            if (two && ok) {
                ok = mbar_wait(&sm.x_full, 0);
                if (ok) {
                    const float m1 = sm.hand_ml[row][0];
                    l1 = sm.hand_ml[row][1];
                    const float m = fmaxf(m_run, m1);                    // finite for a row that is stored
                    w0 = fast_exp2(m_run - m);
                    w1 = fast_exp2(m1 - m);
                }
            }
            if (ok && !sm.failed && row < nq) {
                const float inv = 1.0f / (l_run * w0 + l1 * w1);
                __nv_bfloat16* dst = out + (long long)(flat0 + row) * ldo + h * PT_D;
#pragma unroll
                for (int d = 0; d < PT_D; d += 8) {
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; e += 4) {
                        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (two) x = *reinterpret_cast<const float4*>(hand + (((d + e) / 4) * PT_Q + row) * 4);
                        v[e] = (o[d + e] * w0 + x.x * w1) * inv;
                        v[e + 1] = (o[d + e + 1] * w0 + x.y * w1) * inv;
                        v[e + 2] = (o[d + e + 2] * w0 + x.z * w1) * inv;
                        v[e + 3] = (o[d + e + 3] * w0 + x.w * w1) * inv;
                    }
                    uint4 packed;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
                    packed.x = *reinterpret_cast<uint32_t*>(&h0);
                    packed.y = *reinterpret_cast<uint32_t*>(&h1);
                    packed.z = *reinterpret_cast<uint32_t*>(&h2);
                    packed.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(dst + d) = packed;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace mu

// q: bfloat16 rows of n_heads x 64 (ldq elements apart, n_tokens of them); kv: the paged cache of
// n_cache_pages pages; tiles: int32 [n_tiles][2] = (flat index of the tile's first query token, number of
// queries <= 128), a tile's queries belonging to one sequence and following one another, longest tiles
// first (blocks start in this order).  out rows ldo apart, 16-byte aligned.  head_dim 64, pages of 64.
// k_new, v_new (optional, both or neither): this step's keys and values, rows ldk / ldv apart, appended to
// the cache first (mu_kv_append with append_tiles: tiles of up to 64 tokens) - one call for both launches.
extern "C" int mu_kv_append(const void* k, long long ldk, const void* v, long long ldv, const int* tok_pos,
                            const int* tok_seq, const int* block_table, int max_pages, int page_tokens,
                            int n_tokens, int n_kv_heads, int head_dim, void* kv, int is_bf16, const int* tiles,
                            int n_tiles, void* stream);

MU_EXPORT int mu_attention_prefill_tc(const void* q, long long ldq, int n_tokens, void* out, long long ldo,
                                      void* kv, long long n_cache_pages, const int* block_table,
                                      int max_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                                      const int* tiles, int n_tiles, int n_heads, int n_kv_heads, int head_dim,
                                      float scale, int window, const void* k_new, long long ldk,
                                      const void* v_new, long long ldv, const int* append_tiles,
                                      int n_append_tiles, int* status, void* stream) {
    if (n_tiles <= 0) return MU_OK;
    if ((k_new == nullptr) != (v_new == nullptr)) return MU_ERR_BAD_ARGUMENT;
    if (k_new) {
        if (int e = mu_kv_append(k_new, ldk, v_new, ldv, tok_pos, tok_seq, block_table, max_pages, page_tokens,
                                 n_tokens, n_kv_heads, head_dim, kv, 1, append_tiles, n_append_tiles, stream))
            return e;
    }
    if (page_tokens != mu::PT_K || head_dim != mu::PT_D) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0 || n_tokens <= 0 || !(scale > 0.0f))
        return MU_ERR_BAD_ARGUMENT;                  // (the row maximum is taken before the scores are scaled)
    if (!q || !out || !kv || !block_table || !tok_pos || !tok_seq || !tiles || !status) return MU_ERR_BAD_ARGUMENT;
    if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kv & 15) || ldo % 8 != 0 || ((uintptr_t)out & 15))
        return MU_ERR_ALIGNMENT;
    const long long kv_rows = n_cache_pages * 2 * n_kv_heads * mu::PT_K;
    const long long items = (long long)n_tiles * n_heads;
    if (kv_rows > 2147483647ll || items > 2147483647ll) return MU_ERR_UNSUPPORTED_SIZE;
    CUtensorMap map_q, map_kv;
    if (!mu::tensor_map_bf16(&map_q, q, n_tokens, n_heads * mu::PT_D, ldq, mu::PT_Q) ||
        !mu::tensor_map_bf16(&map_kv, kv, kv_rows, mu::PT_D, mu::PT_D, mu::PT_K))
        return MU_ERR_LAUNCH;
    auto kernel = mu::attention_prefill_tc_kernel;
    const size_t smem = sizeof(mu::PtSmem) + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MU_ERR_LAUNCH;
        mu::prefer_shared_memory(reinterpret_cast<const void*>(kernel));
        raised = true;
    }
    return mu::launch_pdl(kernel, dim3((unsigned)items), dim3(mu::PT_THREADS), smem, (cudaStream_t)stream, 1, map_q,
                          map_kv, (__nv_bfloat16*)out, ldo, block_table, max_pages, tok_pos, tok_seq, tiles, n_heads,
                          n_kv_heads, scale, window, status);
}
