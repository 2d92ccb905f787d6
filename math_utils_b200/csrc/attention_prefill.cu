// Causal attention of whole prompts over the paged cache on tensor cores (bfloat16).
//
// Flash-style: a block takes 64 consecutive query tokens of one sequence and one
// head and walks the sequence's cache pages in two groups of 4 warps (16 queries
// a warp), one group on the even and one on the odd pages, which are merged at the
// end; a page is 64 keys, contiguous per head, and is copied with cp.async into
// padded shared memory (two pages in flight per group).  Per page: S = Q K^T with mma.sync.m16n8k16
// (K fragments by ldmatrix), scale, causal / window mask, online softmax in
// float32 registers (running max and sum per query row), P rounded to bfloat16
// and fed straight back as the A operand of O += P V (V fragments by ldmatrix
// too: a page keeps its values dimension-major).  Queries sit at absolute positions (the cache may already
// hold earlier tokens of the sequence), so a prompt fed in parts gives the same
// result as a prompt fed whole.  The step's own keys and values must have been
// appended before (mu_kv_append).
//
// Formulas: include/ai/Kernels.hpp:132-161.  Head sizes 16..128 in steps of 16.
#include "common.cuh"


#include <math.h>

namespace mu {

constexpr int FP_QT = 64;       // queries per block
constexpr int FP_KT = 64;       // keys per page
constexpr int FP_THREADS = 256;  // two groups of 4 warps: each group takes every other page of the tile's keys
constexpr int FP_GROUP = 128;

__device__ __forceinline__ void group_sync(int grp) {     // the 128 threads of one group
    if (grp == 0) asm volatile("bar.sync 1, %0;" ::"n"(FP_GROUP) : "memory");
    else asm volatile("bar.sync 2, %0;" ::"n"(FP_GROUP) : "memory");
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// KD = head_dim / 16.  Shared memory: Q [64][P], two stages of K [64][P] (P = head_dim + 8) and two
// stages of V [head_dim][72]: values lie dimension-major in the cache, which is the layout the second
// product wants for its right operand, so both products take their fragments by plain ldmatrix.
template <int KD>
__global__ void __launch_bounds__(FP_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, __nv_bfloat16* __restrict__ out,
                         long long ldo, const __nv_bfloat16* __restrict__ kv, const int* __restrict__ block_table,
                         int max_pages, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                         const int* __restrict__ tiles, int n_items, int* counter, int n_heads, int n_kv_heads,
                         float scale, int window) {
    constexpr int DH = 16 * KD, P = DH + 8;
    constexpr int CHUNKS = DH / 8;                 // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char fp_smem[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(fp_smem);
    constexpr int VP = FP_KT + 8;                  // pitch of a value row (one dimension, 64 positions)
    constexpr int GROUP_ELEMS = 2 * FP_KT * P + 2 * DH * VP;     // a group's two stages of keys and of values
    const int tid = threadIdx.x, lane = tid & 31;
    const int grp = tid / FP_GROUP, gtid = tid % FP_GROUP, warp = gtid >> 5;      // warp: which 16 queries
    __nv_bfloat16* k_s = q_s + FP_QT * P + grp * GROUP_ELEMS;    // [2][64][P]
    __nv_bfloat16* v_s = k_s + 2 * FP_KT * P;                    // [2][DH][VP]
    float* merge_o = reinterpret_cast<float*>(q_s + FP_QT * P + GROUP_ELEMS);      // over the second group's stages
    float* merge_ml = merge_o + FP_QT * DH;                      // [64][2]
    const int g = lane >> 2, t = lane & 3;
    __shared__ int next_item;
    pdl_trigger();
    pdl_wait();                                    // queries and this step's cache rows come from the kernels before
    // The blocks take (tile, head) items from a counter until none is left.  The caller lists the tiles
    // longest first, so the long ones start at once on every SM and the short ones fill the gaps.
    for (;;) {
    if (tid == 0) next_item = atomicAdd(&counter[0], 1);
    __syncthreads();
    const int item = next_item;
    if (item >= n_items) break;
    const int tile = item / n_heads;
    const int flat0 = tiles[2 * tile], nq = tiles[2 * tile + 1];
    const int h = item % n_heads, kvh = h / (n_heads / n_kv_heads);
    const int pos0 = tok_pos[flat0];
    const int* pages = block_table + (long long)tok_seq[flat0] * max_pages;
    const int pos_last = pos0 + nq - 1;
    const int first_key = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int first_page = first_key / FP_KT, last_page = pos_last / FP_KT;
    const long long head_stride = (long long)FP_KT * DH;

    auto load_page = [&](int page_idx, int stage) {
        const __nv_bfloat16* kp = kv + ((long long)pages[page_idx] * 2 * n_kv_heads + kvh) * head_stride;
        const __nv_bfloat16* vp = kp + (long long)n_kv_heads * head_stride;
        __nv_bfloat16* ks = k_s + stage * FP_KT * P;
        __nv_bfloat16* vs = v_s + stage * DH * VP;
        for (int c = gtid; c < FP_KT * CHUNKS; c += FP_GROUP) {
            const int r = c / CHUNKS, o = (c % CHUNKS) * 8;
            cp_async16(ks + r * P + o, kp + r * DH + o);
        }
        for (int c = gtid; c < DH * (FP_KT / 8); c += FP_GROUP) {
            const int r = c / (FP_KT / 8), o = (c % (FP_KT / 8)) * 8;
            cp_async16(vs + r * VP + o, vp + r * FP_KT + o);
        }
    };

    // queries of the tile (rows past nq are zero) and the first page
    for (int c = tid; c < FP_QT * CHUNKS; c += FP_THREADS) {
        const int r = c / CHUNKS, o = (c % CHUNKS) * 8;
        if (r < nq) cp_async16(q_s + r * P + o, q + (long long)(flat0 + r) * ldq + h * DH + o);
        else *reinterpret_cast<uint4*>(q_s + r * P + o) = make_uint4(0, 0, 0, 0);
    }
    const int my_first = first_page + grp;         // this group's pages: my_first, my_first + 2, ...
    if (my_first <= last_page) load_page(my_first, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    uint32_t qf[KD][4];
#pragma unroll
    for (int kk = 0; kk < KD; ++kk)
        ldmatrix_x4(qf[kk], q_s + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8);

    float o_acc[2 * KD][4];
#pragma unroll
    for (int j = 0; j < 2 * KD; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[j][i] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float c_log2 = scale * 1.4426950408889634f;          // scores are exponentiated in base 2
    const int qpos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};

    for (int page_idx = my_first; page_idx <= last_page; page_idx += 2) {
        const int stage = ((page_idx - my_first) >> 1) & 1;
        if (page_idx + 2 <= last_page) load_page(page_idx + 2, stage ^ 1);
        cp_async_commit();
        const __nv_bfloat16* ks = k_s + stage * FP_KT * P;
        const __nv_bfloat16* vs = v_s + stage * DH * VP;

        // S = Q K^T for 64 keys: 8 tiles of 8 keys
        float s_acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s_acc[j][i] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, ks + (8 * j + (lane & 7) + 8 * (lane >> 4)) * P + 16 * kk + ((lane >> 3) & 1) * 8);
                mma_16816(s_acc[j], qf[kk], b[0], b[1]);
                mma_16816(s_acc[j + 1], qf[kk], b[2], b[3]);
            }
        }

        // mask, running max, exponentials
        const int key0 = page_idx * FP_KT;
        const bool edge = (key0 + FP_KT - 1 > pos0 + warp * 16) || (window > 0);     // some key may be hidden
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float s = s_acc[j][i] * c_log2;
                if (edge) {
                    const int key = key0 + 8 * j + 2 * t + (i & 1);
                    const int qp = qpos[i >> 1];
                    const bool hidden = key > qp || (window > 0 && key + window <= qp);
                    if (hidden) s = -INFINITY;
                }
                s_acc[j][i] = s;
                mx[i >> 1] = fmaxf(mx[i >> 1], s);
            }
        }
        float corr[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float base = (mx[r] == -INFINITY) ? 0.0f : mx[r];   // a row that has seen no key yet
            corr[r] = exp2f(m_run[r] - base);
            m_run[r] = mx[r];
            mx[r] = base;
        }
        uint32_t pf[4][4];                     // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = exp2f(s_acc[j][0] - mx[0]), p1 = exp2f(s_acc[j][1] - mx[0]);
            const float p2 = exp2f(s_acc[j][2] - mx[1]), p3 = exp2f(s_acc[j][3] - mx[1]);
            sum[0] += p0 + p1;
            sum[1] += p2 + p3;
            pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);          // rows g: a0 (keys lo) / a2 (keys hi)
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);      // rows g + 8: a1 / a3
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + sum[r];
#pragma unroll
        for (int j = 0; j < 2 * KD; ++j) {
            o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
            o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
        }

        // O += P V: k-steps over 16 keys, tiles of 8 head dimensions
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int j = 0; j < 2 * KD; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, vs + (8 * j + (lane & 7) + 8 * (lane >> 4)) * VP + 16 * kk + ((lane >> 3) & 1) * 8);
                mma_16816(o_acc[j], pf[kk], b[0], b[1]);
                mma_16816(o_acc[j + 1], pf[kk], b[2], b[3]);
            }
        }
        cp_async_wait<0>();
        group_sync(grp);
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // the second group hands its share over (its stages are free: its last group_sync is behind it)
    if (grp == 1) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = warp * 16 + g + 8 * r;
#pragma unroll
            for (int j = 0; j < 2 * KD; ++j)
                *reinterpret_cast<float2*>(merge_o + row * DH + 8 * j + 2 * t) =
                    make_float2(o_acc[j][2 * r], o_acc[j][2 * r + 1]);
            if (t == 0) *reinterpret_cast<float2*>(merge_ml + 2 * row) = make_float2(m_run[r], l_run[r]);
        }
    }
    __syncthreads();
    if (grp == 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = warp * 16 + g + 8 * r;
            if (row >= nq) continue;
            const float2 ml = *reinterpret_cast<const float2*>(merge_ml + 2 * row);
            const float m = fmaxf(m_run[r], ml.x);             // finite: the row sees at least its own key
            const float w0 = exp2f(m_run[r] - m), w1 = exp2f(ml.x - m);
            const float inv = 1.0f / (l_run[r] * w0 + ml.y * w1);
            __nv_bfloat16* dst = out + (long long)(flat0 + row) * ldo + h * DH;
#pragma unroll
            for (int j = 0; j < 2 * KD; ++j) {
                const float2 o1 = *reinterpret_cast<const float2*>(merge_o + row * DH + 8 * j + 2 * t);
                *reinterpret_cast<uint32_t*>(dst + 8 * j + 2 * t) =
                    pack_bf16((o_acc[j][2 * r] * w0 + o1.x * w1) * inv, (o_acc[j][2 * r + 1] * w0 + o1.y * w1) * inv);
            }
        }
    }
    __syncthreads();                               // shared memory and next_item are free again
    }
    // the last block to leave puts the counters back to zero for the next launch
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&counter[1], 1) == (int)gridDim.x - 1) {
            counter[0] = 0;
            counter[1] = 0;
        }
    }
}

template <int KD>
static int launch_prefill(const void* q, long long ldq, void* out, long long ldo, const void* kv,
                          const int* block_table, int max_pages, const int* tok_pos, const int* tok_seq,
                          const int* tiles, int n_tiles, int* counter, int n_heads, int n_kv_heads, float scale,
                          int window, cudaStream_t s) {
    constexpr int P = 16 * KD + 8;
    const size_t smem = ((size_t)FP_QT * P + 2 * ((size_t)2 * FP_KT * P + (size_t)2 * 16 * KD * (FP_KT + 8))) *
                        sizeof(__nv_bfloat16);
    auto kernel = attention_prefill_kernel<KD>;
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return MU_ERR_LAUNCH;
            raised = true;
        }
    }
    // as many blocks as the device holds at once (or as there are items)
    static int resident = 0;
    if (resident == 0) {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, FP_THREADS, smem) != cudaSuccess ||
            sms <= 0 || per_sm <= 0)
            return MU_ERR_LAUNCH;
        const int cap = 2;                          // two blocks per SM balance better than all that fit
        resident = sms * (per_sm < cap ? per_sm : cap);
    }
    const long long items = (long long)n_tiles * n_heads;
    if (items > 2147483647ll) return MU_ERR_UNSUPPORTED_SIZE;
    dim3 grid((unsigned)(items < resident ? items : resident));
    return launch_pdl(kernel, grid, dim3(FP_THREADS), smem, s, 1, (const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out,
                      ldo, (const __nv_bfloat16*)kv, block_table, max_pages, tok_pos, tok_seq, tiles, (int)items,
                      counter, n_heads, n_kv_heads, scale, window);
}

}  // namespace mu

// tiles: int32 [n_tiles][2] = (flat index of the tile's first query token, number of queries <= 64);
// a tile's queries belong to one sequence and follow one another.  bfloat16 only; pages of 64
// positions; head_dim 16..128 in steps of 16; q rows and the cache 16-byte aligned.  The blocks take
// (tile, head) items in the order of `tiles`, all heads of a tile together: list the tiles with the most
// keys first.  counter: two device ints that are zero between launches (the kernel leaves them zero).
MU_EXPORT int mu_attention_prefill(const void* q, long long ldq, void* out, long long ldo, const void* kv,
                                   const int* block_table, int max_pages, int page_tokens, const int* tok_pos,
                                   const int* tok_seq, const int* tiles, int n_tiles, int n_heads, int n_kv_heads,
                                   int head_dim, float scale, int window, int* counter, void* stream) {
    if (n_tiles <= 0) return MU_OK;
    if (!counter) return MU_ERR_BAD_ARGUMENT;
    if (page_tokens != mu::FP_KT) return MU_ERR_UNSUPPORTED_SIZE;
    if (head_dim < 16 || head_dim > 128 || head_dim % 16 != 0) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0 || n_heads > 65535)
        return MU_ERR_BAD_ARGUMENT;
    if (!q || !out || !kv || !block_table || !tok_pos || !tok_seq || !tiles) return MU_ERR_BAD_ARGUMENT;
    if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kv & 15) || ldo % 2 != 0 || ((uintptr_t)out & 3))
        return MU_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define MU_FP(KD)                                                                                              \
    case KD:                                                                                                   \
        return mu::launch_prefill<KD>(q, ldq, out, ldo, kv, block_table, max_pages, tok_pos, tok_seq, tiles,   \
                                      n_tiles, counter, n_heads, n_kv_heads, scale, window, s)
    switch (head_dim / 16) {
        MU_FP(1); MU_FP(2); MU_FP(3); MU_FP(4); MU_FP(5); MU_FP(6); MU_FP(7); MU_FP(8);
    }
#undef MU_FP
    return MU_ERR_UNSUPPORTED_SIZE;
}
