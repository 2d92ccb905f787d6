// Single-token attention over the paged cache on tensor cores (bfloat16).
//
// The CUDA-core kernel of attention_decode.cu spends its time issuing
// instructions: two thousand per warp and page, most of them widening
// bfloat16 and multiplying one pair at a time.  Here a warp does a page with
// some two hundred: both products of the page are mma.sync.m16n8k16, and the
// fragments are loaded straight from the cache in the layout the instruction
// wants, 16 bytes at a time, with no shuffles:
//   * S = Q K^T.  The 16 rows of the left operand are the query heads that
//     share one kv head (one row for plain multi-head attention; the rest are
//     zero).  A key is one contiguous row of the page; thread (g, t) of the
//     warp loads, for each of the 8 column tiles, dims [t*dh/4, (t+1)*dh/4) of
//     "its" key.  Which k slot of the instruction a dimension lands in does not
//     matter as long as Q uses the same assignment, and which key is column n
//     of tile j is our choice too: key(j, n) = 16 (n / 2) + 2 j + n % 2, chosen
//     so that the scores a thread ends up holding are 16 consecutive keys,
//     exactly the keys whose probabilities it must supply to the second product.
//   * O = P V.  Values lie dimension-major in the page (attention.cu), so thread
//     (g, t) loads for each tile of 8 dimensions the 16 consecutive positions
//     [16 t, 16 t + 16) of dimension row 8 j + g: again one 32-byte run.
// One block per (sequence, kv head), or with very few sequences a cluster of
// two or four; its warps share out the pages, fold several pages into a
// running (max, sum, output) when there are more pages than warps, and merge
// in shared memory in warp order (the blocks of a cluster then in rank order).  The step's own key and
// value are read from the step's projections and appended by the kernel, as in
// attention_decode.cu.  Softmax in float32; probabilities rounded to bfloat16
// for the second product, as in the prompt kernel.
//
// Formulas: include/ai/Kernels.hpp:132-161.  Head sizes 32, 64, 96 and 128; up
// to 16 query heads per kv head; pages of 64 positions.
#include "common.cuh"

#include <cooperative_groups.h>
#include <math.h>

namespace mu {

namespace cg = cooperative_groups;

constexpr int TD_PAGE = 64;

__device__ __forceinline__ void td_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t td_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Pages are staged in shared memory.  A key page and a value page of one kv head are each one
// contiguous run of the cache, so one thread brings a page in with two bulk copies (cp.async.bulk,
// completion counted by an mbarrier); every warp owns a ring of RING page buffers and keeps that many
// of its pages in flight while it works on the oldest.  The bytes in flight do not sit in registers,
// so several blocks fit on an SM and memory streams while the tensor cores work, and a block of few
// sequences can ask for all of its pages at once.  KD = head_dim / 16 (even), NW = warps per block.
// Fragments are read from shared memory with the addressing described above (rows of a page are
// 64 or 128 bytes apart, so the two rows that a quarter of a warp reads together collide on banks two
// ways at most).  Waits on a copy are bounded; a wait that runs out sets *status to 4 and the block
// writes nothing.
constexpr unsigned long long TD_WAIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t td_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool td_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = td_smem(bar);
    unsigned long long start = 0;
    for (unsigned int spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 1023u) == 1023u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > TD_WAIT_NS) return false;
        }
    }
}

// NG groups of SUB warps: a group owns a ring of RING page buffers and takes every NG-th page of the
// sequence; its SUB warps share each page, KPW = 64 / SUB keys a warp.  More warps on the same bytes in
// flight: a warp's work on a page is a chain of dependent steps (fragments in, scores, softmax, weighted
// values), and an SM hides one chain behind the others only if there are enough of them.
//
// CL blocks of a thread-block cluster (grid.y; 1, 2 or 4) may share a (sequence, kv head): with few sequences
// there are far fewer blocks than SMs, and one SM alone draws a sequence's pages more slowly than several do.
// The NG * CL groups of the cluster take the pages in turn; every block merges its own warps, the others hand
// their merged part (maximum, sum, weighted values) to block 0 through distributed shared memory, and block 0
// merges the parts in rank order and writes the result.
template <int KD, int NG, int SUB, int RING, int CL>
__global__ void __launch_bounds__(NG * SUB * 32)
attention_decode_ring_kernel(const __nv_bfloat16* __restrict__ q, long long ldq,
                             const __nv_bfloat16* __restrict__ k_new, long long ldk,
                             const __nv_bfloat16* __restrict__ v_new, long long ldv,
                             __nv_bfloat16* __restrict__ out, long long ldo, __nv_bfloat16* kv,
                             const int* __restrict__ block_table, int max_pages,
                             const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, int n_heads,
                             int n_kv_heads, float scale, int window, int* status) {
    constexpr int NW = NG * SUB;
    constexpr int DH = 16 * KD;
    constexpr int KV4 = KD / 2;                    // 16-byte pieces of a key row that a thread holds
    constexpr int KPW = TD_PAGE / SUB;             // keys of a page that one warp takes
    constexpr int TJ = KPW / 8;                    // score tiles of 8 keys
    constexpr int KT = KPW / 4;                    // consecutive keys whose scores one thread ends up holding
    constexpr int KK = KPW / 16;                   // steps of 16 positions in the second product
    constexpr int PAGE_ELEMS = TD_PAGE * DH;       // one kv head's keys (or values) of a page
    constexpr uint32_t PAGE_BYTES = PAGE_ELEMS * sizeof(__nv_bfloat16);
    static_assert(SUB == 1 || SUB == 2 || SUB == 4, "a warp takes 64, 32 or 16 keys of a page");
    extern __shared__ __align__(128) unsigned char ring_raw[];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(ring_raw);              // [NG][RING][2][PAGE_ELEMS]
    float* part_o = reinterpret_cast<float*>(ring_raw + (size_t)NG * RING * 2 * PAGE_BYTES);   // [NW][rows][DH + 1]
    __shared__ uint64_t full[NG][RING];            // a page has landed
    __shared__ uint64_t done[NG][RING];            // every warp of the group has read it
    __shared__ float part_m[NW][16], part_l[NW][16];
    __shared__ float weight[NW][16];
    __shared__ int failed;
    // with CL > 1: this block's merged maximum per row, and in block 0 what the other blocks hand over
    __shared__ float blk_m[16];
    __shared__ float peer_m[CL > 1 ? CL - 1 : 1][16], peer_l[CL > 1 ? CL - 1 : 1][16];
    __shared__ int cl_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / SUB, sub = warp % SUB;
    const int g = lane >> 2, t = lane & 3;
    const int tk = blockIdx.x / n_kv_heads, kvh = blockIdx.x % n_kv_heads;
    const int rows = n_heads / n_kv_heads;
    const int part = CL > 1 ? (int)blockIdx.y : 0;            // the cluster spans grid.y
    constexpr int LANES = NG * CL;                             // groups that share a sequence's pages
    pdl_trigger();
    if (threadIdx.x == 0) { failed = 0; cl_failed = 0; }
    if (lane == 0 && sub == 0) {
#pragma unroll
        for (int r = 0; r < RING; ++r) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(td_smem(&full[group][r])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(td_smem(&done[group][r])), "r"(SUB) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if constexpr (CL > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // set up; waited for before anything is handed over
    const int* pages = block_table + (long long)(tok_seq ? tok_seq[tk] : tk) * max_pages;
    const int pos = tok_pos[tk];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_page = first / TD_PAGE, last_page = pos / TD_PAGE;
    const long long head_stride = (long long)PAGE_ELEMS;
    const int my_first = first_page + group * CL + part;
    const int n_mine = my_first <= last_page ? (last_page - my_first) / LANES + 1 : 0;
    __nv_bfloat16* my_ring = ring + (size_t)group * RING * 2 * PAGE_ELEMS;
    const bool issuer = sub == 0 && lane == 0;

    // one lane asks for the group's i-th page: two contiguous runs of the cache, one barrier
    auto issue = [&](int i) {
        const int slot = i % RING;
        const long long page = pages[my_first + i * LANES];
        const __nv_bfloat16* ksrc = kv + (page * 2 * n_kv_heads + kvh) * head_stride;
        const __nv_bfloat16* vsrc = ksrc + (long long)n_kv_heads * head_stride;
        const uint32_t bar = td_smem(&full[group][slot]);
        const uint32_t dst = td_smem(my_ring + (size_t)slot * 2 * PAGE_ELEMS);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * PAGE_BYTES) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(ksrc), "r"(PAGE_BYTES), "r"(bar) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst + PAGE_BYTES), "l"(vsrc), "r"(PAGE_BYTES), "r"(bar) : "memory");
    };
    // rows written by earlier steps, which no kernel of this step touches, may be asked for at once
    int issued = 0;
    if (issuer)
        for (; issued < n_mine && issued < RING; ++issued) issue(issued);
    pdl_wait();                                    // this step's query, key and value from here on

    uint32_t qa[KD][4];
    {
        uint4 lo4[KV4], hi4[KV4];
#pragma unroll
        for (int c = 0; c < KV4; ++c) { lo4[c] = make_uint4(0, 0, 0, 0); hi4[c] = make_uint4(0, 0, 0, 0); }
        if (g < rows) {
            const uint4* src = reinterpret_cast<const uint4*>(q + (long long)tk * ldq + (long long)(kvh * rows + g) * DH + (DH / 4) * t);
#pragma unroll
            for (int c = 0; c < KV4; ++c) lo4[c] = src[c];
        }
        if (g + 8 < rows) {
            const uint4* src = reinterpret_cast<const uint4*>(q + (long long)tk * ldq + (long long)(kvh * rows + g + 8) * DH + (DH / 4) * t);
#pragma unroll
            for (int c = 0; c < KV4; ++c) hi4[c] = src[c];
        }
        const uint32_t* lw = reinterpret_cast<const uint32_t*>(lo4);
        const uint32_t* hw = reinterpret_cast<const uint32_t*>(hi4);
#pragma unroll
        for (int kk = 0; kk < KD; ++kk) {
            qa[kk][0] = lw[2 * kk]; qa[kk][1] = hw[2 * kk]; qa[kk][2] = lw[2 * kk + 1]; qa[kk][3] = hw[2 * kk + 1];
        }
    }
    const float c_log2 = scale * 1.4426950408889634f;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o_acc[2 * KD][4];
#pragma unroll
    for (int j = 0; j < 2 * KD; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[j][i] = 0.0f;

    bool ok = true;
    for (int i = 0; i < n_mine; ++i) {
        const int slot = i % RING;
        const int page_idx = my_first + i * LANES;
        if (!td_wait(&full[group][slot], (uint32_t)((i / RING) & 1))) { ok = false; break; }
        const __nv_bfloat16* ks = my_ring + (size_t)slot * 2 * PAGE_ELEMS;
        const __nv_bfloat16* vs = ks + PAGE_ELEMS;
        const int base = page_idx * TD_PAGE;
        // the keys of the page this warp takes: [key0, key0 + KPW); of those, [lo, hi) can be seen
        const int key0 = sub * KPW;
        const int lo = max(first - base, 0) - key0, hi = min(pos + 1 - base, TD_PAGE) - key0;      // relative to key0
        const bool in_page = (k_new != nullptr) && page_idx == last_page;
        const int new_key = pos - base - key0;                  // the step's own token, relative to key0
        const bool has_new = in_page && new_key >= 0 && new_key < KPW;
        const __nv_bfloat16* kn = has_new ? k_new + (long long)tk * ldk + kvh * DH : nullptr;
        const __nv_bfloat16* vn = has_new ? v_new + (long long)tk * ldv + kvh * DH : nullptr;
        if (has_new) {
            // append to the cache: this warp is the only one for this (sequence, kv head, key)
            const long long page = pages[page_idx];
            __nv_bfloat16* kpage = kv + (page * 2 * n_kv_heads + kvh) * head_stride;
            __nv_bfloat16* vpage = kpage + (long long)n_kv_heads * head_stride;
            for (int d = lane; d < DH; d += 32) {
                kpage[(long long)(key0 + new_key) * DH + d] = kn[d];
                vpage[(long long)d * TD_PAGE + key0 + new_key] = vn[d];
            }
        }
        if (hi > 0 && lo < KPW) {                               // some key of this warp's share can be seen
            const int jn = (new_key % KT) >> 1;
            const bool mine_new = has_new && (KT * (g >> 1) + 2 * jn + (g & 1) == new_key);

            // S = Q K^T: TJ tiles of 8 keys; which key is column n of tile j: KT (n / 2) + 2 j + n % 2, so that
            // a thread ends up with the scores of KT consecutive keys
            float s[TJ][4];
#pragma unroll
            for (int j = 0; j < TJ; ++j) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
                const int key = key0 + KT * (g >> 1) + 2 * j + (g & 1);
                uint4 kf[KV4];
                const uint4* src = (mine_new && j == jn) ? reinterpret_cast<const uint4*>(kn + (DH / 4) * t)
                                                         : reinterpret_cast<const uint4*>(ks + key * DH + (DH / 4) * t);
#pragma unroll
                for (int c = 0; c < KV4; ++c) kf[c] = src[c];
                const uint32_t* kw = reinterpret_cast<const uint32_t*>(kf);
#pragma unroll
                for (int kk = 0; kk < KD; ++kk) td_mma(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kw[2 * kk], kw[2 * kk + 1]);
            }
            float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int j = 0; j < TJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = KT * t + 2 * j + (e & 1);
                    const float v = (key >= lo && key < hi) ? s[j][e] * c_log2 : -INFINITY;
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float corr[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));      // finite: a key can be seen
                corr[r] = exp2f(m_run[r] - mx[r]);
                m_run[r] = mx[r];
            }
            // probabilities; the new key's is set aside (its value is not in the cache yet) and kept as w_new
            float w_new[2] = {0.0f, 0.0f};
            uint32_t pa[KK][4];
#pragma unroll
            for (int j = 0; j < TJ; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = exp2f(s[j][e] - mx[e >> 1]);
                    sum[e >> 1] += p[e];
                    if (has_new && KT * t + 2 * j + (e & 1) == new_key) { w_new[e >> 1] = p[e]; p[e] = 0.0f; }
                }
                pa[j >> 1][(j & 1) * 2] = td_pack(p[0], p[1]);
                pa[j >> 1][(j & 1) * 2 + 1] = td_pack(p[2], p[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + sum[r];
            // O = O * corr + P V: tiles of 8 dimensions, KK steps of 16 positions; a thread's KT positions of a
            // dimension row are one run of the page
#pragma unroll
            for (int j = 0; j < 2 * KD; ++j) {
                o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0]; o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
                const __nv_bfloat16* vrow = vs + (8 * j + g) * TD_PAGE + key0 + KT * t;
                uint32_t vw[2 * KK];
                if constexpr (KT == 16) {
                    const uint4 a4 = reinterpret_cast<const uint4*>(vrow)[0], b4 = reinterpret_cast<const uint4*>(vrow)[1];
                    vw[0] = a4.x; vw[1] = a4.y; vw[2] = a4.z; vw[3] = a4.w; vw[4] = b4.x; vw[5] = b4.y; vw[6] = b4.z; vw[7] = b4.w;
                } else if constexpr (KT == 8) {
                    const uint4 a4 = reinterpret_cast<const uint4*>(vrow)[0];
                    vw[0] = a4.x; vw[1] = a4.y; vw[2] = a4.z; vw[3] = a4.w;
                } else {
                    const uint2 a2 = reinterpret_cast<const uint2*>(vrow)[0];
                    vw[0] = a2.x; vw[1] = a2.y;
                }
#pragma unroll
                for (int kk = 0; kk < KK; ++kk)
                    td_mma(o_acc[j], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], vw[2 * kk], vw[2 * kk + 1]);
            }
            if (has_new) {
                // every thread of a row's group needs the new key's weight: it sits in the thread with t = new_key / KT
                const int src_lane = (lane & ~3) | ((new_key / KT) & 3);
                const float w0 = __shfl_sync(0xffffffffu, w_new[0], src_lane);
                const float w1 = __shfl_sync(0xffffffffu, w_new[1], src_lane);
#pragma unroll
                for (int j = 0; j < 2 * KD; ++j) {
                    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vn + 8 * j + 2 * t));
                    o_acc[j][0] = fmaf(w0, v.x, o_acc[j][0]); o_acc[j][1] = fmaf(w0, v.y, o_acc[j][1]);
                    o_acc[j][2] = fmaf(w1, v.x, o_acc[j][2]); o_acc[j][3] = fmaf(w1, v.y, o_acc[j][3]);
                }
            }
        }
        __syncwarp();                              // every lane has read the buffer
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(td_smem(&done[group][slot])) : "memory");
        if (issuer && issued < n_mine) {
            // the slot is filled again once every warp of the group has read it; if that never happens the
            // page is not asked for, and the warps that wait for it give up in their turn
            if (td_wait(&done[group][slot], (uint32_t)((i / RING) & 1))) issue(issued++);
            else atomicExch(status, 4);
        }
    }
    if (!ok) {
        // let the copies still under way land before the block goes away, then report
        if (issuer) {
            for (int i = 0; i < issued; ++i)
                if (i + RING >= issued) td_wait(&full[group][i % RING], (uint32_t)((i / RING) & 1));
        }
        if (lane == 0) {
            atomicExch(status, 4);
            failed = 1;
        }
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* mine = part_o + (long long)warp * rows * (DH + 1);
#pragma unroll
    for (int j = 0; j < 2 * KD; ++j) {
        if (g < rows) {
            mine[g * (DH + 1) + 8 * j + 2 * t] = o_acc[j][0];
            mine[g * (DH + 1) + 8 * j + 2 * t + 1] = o_acc[j][1];
        }
        if (g + 8 < rows) {
            mine[(g + 8) * (DH + 1) + 8 * j + 2 * t] = o_acc[j][2];
            mine[(g + 8) * (DH + 1) + 8 * j + 2 * t + 1] = o_acc[j][3];
        }
    }
    if (t == 0) {
        part_m[warp][g] = m_run[0]; part_m[warp][g + 8] = m_run[1];
        part_l[warp][g] = l_run[0]; part_l[warp][g + 8] = l_run[1];
    }
    __syncthreads();
    if (CL == 1 && failed) return;
    if (threadIdx.x < NW * 16) {
        const int w = threadIdx.x / 16, r = threadIdx.x % 16;
        float big = -INFINITY;
#pragma unroll
        for (int x = 0; x < NW; ++x) big = fmaxf(big, part_m[x][r]);
        weight[w][r] = part_m[w][r] == -INFINITY ? 0.0f : exp2f(part_m[w][r] - big);
        if (w == 0) blk_m[r] = big;
    }
    __syncthreads();
    if constexpr (CL == 1) {
        for (int idx = threadIdx.x; idx < rows * DH; idx += NW * 32) {
            const int r = idx / DH, d = idx % DH;
            float total = 0.0f, o = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                total = fmaf(part_l[w][r], weight[w][r], total);
                o = fmaf(part_o[(w * rows + r) * (DH + 1) + d], weight[w][r], o);
            }
            out[(long long)tk * ldo + (long long)(kvh * rows + r) * DH + d] = __float2bfloat16_rn(o / total);
        }
    } else {
        // this block's warps merged: (blk_m, total, o) per row, relative to blk_m.  Block 0 keeps its own in
        // place of warp 0's partials; the others write theirs into block 0's shared memory.
        float* peer_o = part_o + (size_t)NW * rows * (DH + 1);                  // [CL - 1][rows][DH], used in block 0
        cg::cluster_group cluster = cg::this_cluster();
        float* to_o = part == 0 ? nullptr : cluster.map_shared_rank(peer_o, 0) + (size_t)(part - 1) * rows * DH;
        float* to_m = part == 0 ? nullptr : cluster.map_shared_rank(&peer_m[0][0], 0) + (part - 1) * 16;
        float* to_l = part == 0 ? nullptr : cluster.map_shared_rank(&peer_l[0][0], 0) + (part - 1) * 16;
        float mine_o[(16 * DH + NW * 32 - 1) / (NW * 32)], mine_l[(16 * DH + NW * 32 - 1) / (NW * 32)];
        int n_held = 0;
        for (int idx = threadIdx.x; idx < rows * DH; idx += NW * 32, ++n_held) {
            const int r = idx / DH, d = idx % DH;
            float total = 0.0f, o = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                total = fmaf(part_l[w][r], weight[w][r], total);
                o = fmaf(part_o[(w * rows + r) * (DH + 1) + d], weight[w][r], o);
            }
            mine_o[n_held] = o;
            mine_l[n_held] = total;
        }
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");    // every block of the cluster is set up
        if (part != 0) {
            n_held = 0;
            for (int idx = threadIdx.x; idx < rows * DH; idx += NW * 32, ++n_held) {
                const int r = idx / DH, d = idx % DH;
                to_o[r * DH + d] = mine_o[n_held];
                if (d == 0) { to_l[r] = mine_l[n_held]; to_m[r] = blk_m[r]; }
            }
            if (failed && threadIdx.x == 0) *cluster.map_shared_rank(&cl_failed, 0) = 1;
        } else if (failed && threadIdx.x == 0) {
            cl_failed = 1;
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");    // the parts are in block 0
        if (part != 0 || cl_failed) return;
        n_held = 0;
        for (int idx = threadIdx.x; idx < rows * DH; idx += NW * 32, ++n_held) {
            const int r = idx / DH, d = idx % DH;
            float big = blk_m[r];
#pragma unroll
            for (int c = 0; c < CL - 1; ++c) big = fmaxf(big, peer_m[c][r]);
            float wgt = blk_m[r] == -INFINITY ? 0.0f : exp2f(blk_m[r] - big);
            float total = mine_l[n_held] * wgt, o = mine_o[n_held] * wgt;
#pragma unroll
            for (int c = 0; c < CL - 1; ++c) {                                  // in rank order
                wgt = peer_m[c][r] == -INFINITY ? 0.0f : exp2f(peer_m[c][r] - big);
                total = fmaf(peer_l[c][r], wgt, total);
                o = fmaf(peer_o[((size_t)c * rows + r) * DH + d], wgt, o);
            }
            out[(long long)tk * ldo + (long long)(kvh * rows + r) * DH + d] = __float2bfloat16_rn(o / total);
        }
    }
}

}  // namespace mu

// Arguments as mu_attention_decode (bfloat16 only).  n_warps: how the block is built, by how many blocks there
// are.  6: six groups of one warp, a block an SM (no more blocks than SMs: all pages of a sequence in flight at
// once); 12 or 24: two or four such blocks share each (sequence, kv head) as a cluster (blocks on at most
// half or a quarter of the SMs; head size 64).  3: three groups of two warps that share each page, two blocks
// an SM (up to twice as many blocks as SMs; head size 64).  2: two groups of two warps, three blocks an SM
// (more blocks than that).  Each group has a ring of pages.  `status` is a device word that is set to 4 if a
// wait for a copy runs out.
MU_EXPORT int mu_attention_decode_tc(const void* q, long long ldq, const void* k_new, long long ldk,
                                     const void* v_new, long long ldv, void* out, long long ldo, void* kv,
                                     const int* block_table, int max_pages, int page_tokens,
                                     const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, int n_warps,
                                     int* status, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (page_tokens != mu::TD_PAGE) return MU_ERR_UNSUPPORTED_SIZE;
    if (head_dim != 32 && head_dim != 64 && head_dim != 96 && head_dim != 128) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0) return MU_ERR_BAD_ARGUMENT;
    if (n_heads / n_kv_heads > 16) return MU_ERR_UNSUPPORTED_SIZE;
    if (!q || !out || !kv || !block_table || !tok_pos || !status) return MU_ERR_BAD_ARGUMENT;
    if ((k_new == nullptr) != (v_new == nullptr)) return MU_ERR_BAD_ARGUMENT;
    if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kv & 15)) return MU_ERR_ALIGNMENT;
    if (k_new && (ldk % 8 != 0 || ldv % 2 != 0 || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 3))) return MU_ERR_ALIGNMENT;
    const long long blocks = (long long)n_tokens * n_kv_heads;
    if (blocks > 2147483647ll) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    int rc = MU_ERR_UNSUPPORTED_SIZE;
    const int rows = n_heads / n_kv_heads;
#define MU_TR(KD, NG, SUB, CL)                                                                                 \
    do {                                                                                                       \
        auto kernel = mu::attention_decode_ring_kernel<KD, NG, SUB, 2, CL>;                                    \
        const size_t smem = (size_t)NG * 2 * 2 * mu::TD_PAGE * 16 * KD * sizeof(__nv_bfloat16) +               \
                            (size_t)NG * SUB * rows * (16 * KD + 1) * sizeof(float) +                          \
                            (size_t)(CL - 1) * rows * 16 * KD * sizeof(float);                                 \
        static bool raised = false;                                                                            \
        if (!raised) {                                                                                         \
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=       \
                cudaSuccess)                                                                                   \
                return MU_ERR_LAUNCH;                                                                          \
            raised = true;                                                                                     \
        }                                                                                                      \
        if (smem > 200 * 1024) return MU_ERR_UNSUPPORTED_SIZE;                                                 \
        rc = mu::launch_pdl(kernel, dim3((unsigned)blocks, CL), dim3(NG * SUB * 32), smem, s, CL,              \
            (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_new, ldk, (const __nv_bfloat16*)v_new, ldv,  \
            (__nv_bfloat16*)out, ldo, (__nv_bfloat16*)kv, block_table, max_pages, tok_pos, tok_seq, n_heads,   \
            n_kv_heads, scale, window, status);                                                                \
    } while (0)
    // six groups with their rings and many query heads per kv head may not fit: then two groups do it.  With
    // many blocks (two groups each, three blocks an SM) two warps share each page where the head is small
    // enough for the registers to allow it: more chains of work for the SM to switch between.  With few blocks
    // a warp per page is the shorter chain.  In between, three groups of two warps: a group walks over a
    // third of the pages instead of half of them, and two blocks still share an SM.  With very few blocks,
    // two or four of the large ones share each (sequence, kv head) as a cluster (head size 64).
    const size_t six = (size_t)6 * 2 * 2 * mu::TD_PAGE * head_dim * sizeof(__nv_bfloat16) +
                       (size_t)6 * rows * (head_dim + 1) * sizeof(float);
    const bool wide = n_warps >= 6 && six <= 200 * 1024;
    const int shared_by = !wide || head_dim != 64 ? 1 : n_warps >= 24 ? 4 : n_warps >= 12 ? 2 : 1;
    const bool fits = six + (size_t)(shared_by - 1) * rows * head_dim * sizeof(float) <= 200 * 1024;
    if (head_dim == 32) { if (wide) MU_TR(2, 6, 1, 1); else MU_TR(2, 2, 2, 1); }
    else if (head_dim == 64) {
        if (wide && shared_by == 4 && fits) MU_TR(4, 6, 1, 4);
        else if (wide && shared_by == 2 && fits) MU_TR(4, 6, 1, 2);
        else if (wide) MU_TR(4, 6, 1, 1);
        else if (n_warps >= 3) MU_TR(4, 3, 2, 1);
        else MU_TR(4, 2, 2, 1);
    }
    else if (head_dim == 96) MU_TR(6, 2, 1, 1);
    else MU_TR(8, 2, 1, 1);
#undef MU_TR
    return rc;
}
