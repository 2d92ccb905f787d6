// Single-token attention over the paged cache, one launch per layer.
//
// Each sequence brings one query token.  One block takes one (sequence, head);
// its warps share out the sequence's cache pages.  A page's 64 keys of that head
// are one contiguous block, so a lane computes two scores (16-byte loads along
// the head), the warp does the max-subtracted softmax of the page in float32,
// and the lanes, now spread over the head's dimensions, add up the weighted
// values, which were asked for before anything else so that they travel while
// the scores are computed.  A warp that has several pages folds them into one
// running (max, sum, values); the warps' results meet in shared memory and are
// merged in warp order, so the result does not depend on timing, and nothing
// goes through global scratch.
//
// The new token's own key and value need not be in the cache yet: given
// `k_new` / `v_new` (this step's projections) the kernel reads them from there,
// and the first query head of each kv head copies them into the page.  That
// folds the cache append and the merge of the split into the attention launch
// (3 launches -> 1).  Every load of a lane that does not depend on another is
// issued before the first use of any of them: the kernel is a short chain of
// round trips to memory, and each one saved shows.
//
// Formulas: include/ai/Kernels.hpp:132-161.  Split and merge after the idea of
// src/gpu/Kernels.metal:284-345 (128-key partitions there, 64-key pages here).
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int AD_PAGE = 64;

__device__ __forceinline__ float dot_head(const float* qs, const float* krow, int head_dim) {
    float s = 0.0f;
#pragma unroll 8
    for (int d = 0; d < head_dim; d += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(krow + d);
        s = fmaf(qs[d], kk.x, s);
        s = fmaf(qs[d + 1], kk.y, s);
        s = fmaf(qs[d + 2], kk.z, s);
        s = fmaf(qs[d + 3], kk.w, s);
    }
    return s;
}
__device__ __forceinline__ float dot_head(const float* qs, const __nv_bfloat16* krow, int head_dim) {
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll 8
    for (int d = 0; d < head_dim; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            s0 = fmaf(qs[d + 2 * i], f.x, s0);
            s1 = fmaf(qs[d + 2 * i + 1], f.y, s1);
        }
    }
    return s0 + s1;
}

// Two dot products at once: the loads of both rows are issued before either is used.
__device__ __forceinline__ void dot_head2(const float* qs, const float* ka, const float* kb, int head_dim,
                                          float& sa, float& sb) {
    float a = 0.0f, b = 0.0f;
#pragma unroll 4
    for (int d = 0; d < head_dim; d += 4) {
        const float4 x = *reinterpret_cast<const float4*>(ka + d);
        const float4 y = *reinterpret_cast<const float4*>(kb + d);
        a = fmaf(qs[d], x.x, a); a = fmaf(qs[d + 1], x.y, a); a = fmaf(qs[d + 2], x.z, a); a = fmaf(qs[d + 3], x.w, a);
        b = fmaf(qs[d], y.x, b); b = fmaf(qs[d + 1], y.y, b); b = fmaf(qs[d + 2], y.z, b); b = fmaf(qs[d + 3], y.w, b);
    }
    sa = a; sb = b;
}
__device__ __forceinline__ void dot_head2(const float* qs, const __nv_bfloat16* ka, const __nv_bfloat16* kb,
                                          int head_dim, float& sa, float& sb) {
    float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll 8
    for (int d = 0; d < head_dim; d += 8) {
        const uint4 ra = *reinterpret_cast<const uint4*>(ka + d);
        const uint4 rb = *reinterpret_cast<const uint4*>(kb + d);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
            a0 = fmaf(qs[d + 2 * i], fa.x, a0); a1 = fmaf(qs[d + 2 * i + 1], fa.y, a1);
            b0 = fmaf(qs[d + 2 * i], fb.x, b0); b1 = fmaf(qs[d + 2 * i + 1], fb.y, b1);
        }
    }
    sa = a0 + a1; sb = b0 + b1;
}

// DP: the head holds at most 64 * DP dimensions; a lane owns dims lane + 32 * i, i < 2 * DP.
// NW: warps per block.
template <typename TE, int DP, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_kernel(const TE* __restrict__ q, long long ldq, const TE* __restrict__ k_new, long long ldk,
                        const TE* __restrict__ v_new, long long ldv, TE* __restrict__ out, long long ldo,
                        TE* kv, const int* __restrict__ block_table, int max_pages,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, int n_heads,
                        int n_kv_heads, int head_dim, float scale, int window) {
    constexpr int D1 = 2 * DP;                                        // dimensions per lane
    constexpr int ES = (int)sizeof(TE);
    constexpr int VCK = 256 / (D1 * ES) > 64 ? 64 : 256 / (D1 * ES);  // keys fetched at once: 64 registers' worth
    constexpr int VQ = VCK * ES / 16;                                 // 16-byte pieces per dimension and fetch
    __shared__ float q_smem[DP * 64];
    __shared__ float part_o[NW][DP * 64];
    __shared__ float part_m[NW], part_l[NW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x / n_heads, h = blockIdx.x % n_heads;
    const int group = n_heads / n_kv_heads;
    const int kvh = h / group;
    pdl_trigger();
    // positions and page lists were set before this step began: they may be read at once
    const int* pages = block_table + (long long)(tok_seq ? tok_seq[t] : t) * max_pages;
    const int guess = pages[min(warp, max_pages - 1)];      // the warp's page if nothing is cut by a window
    const int pos = tok_pos[t];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_page = first / AD_PAGE, last_page = pos / AD_PAGE;
    const long long head_stride = (long long)AD_PAGE * head_dim;

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[D1];
#pragma unroll
    for (int i = 0; i < D1; ++i) acc[i] = 0.0f;

    // What a page needs: where it lies, which of its keys are visible, whether the new key is in it.
    struct PageView {
        TE* kpage; TE* vpage;                                  // keys [64][head_dim]; values [head_dim][64]
        int lo, hi, hi_cache;
        bool has_new;
    };
    auto view_of = [&](int page_idx) {
        PageView pv;
        const int page = (page_idx == warp) ? guess : pages[page_idx];
        pv.kpage = kv + ((long long)page * 2 * n_kv_heads + kvh) * head_stride;
        pv.vpage = pv.kpage + (long long)n_kv_heads * head_stride;
        const int base = page_idx * AD_PAGE;
        pv.lo = max(first - base, 0);                          // first visible key inside the page
        pv.hi = min(pos + 1 - base, AD_PAGE);                  // one past the last visible key
        pv.has_new = (k_new != nullptr) && page_idx == last_page;   // the query's own key lives here
        pv.hi_cache = pv.has_new ? pv.hi - 1 : pv.hi;          // keys to be read from the cache
        return pv;
    };
    // values of VCK positions from j0 on, for each of the lane's dimensions, as they lie in memory
    uint4 vraw[D1][VQ];
    auto fetch_values = [&](const PageView& pv, int j0) {
#pragma unroll
        for (int i = 0; i < D1; ++i) {
            const int d = lane + 32 * i;
            const uint4* src = reinterpret_cast<const uint4*>(pv.vpage + (long long)min(d, head_dim - 1) * AD_PAGE + j0);
#pragma unroll
            for (int c = 0; c < VQ; ++c) vraw[i][c] = src[c];
        }
    };

    // The warp's first page: its values are asked for before anything else (rows written by earlier
    // steps, untouched by the kernels ahead of this one), so that they travel during the wait.
    // Positions of the page that hold nothing yet are read too; their weights are zero.
    const int my_first = first_page + warp;
    PageView pv = {};
    if (my_first <= last_page) {
        pv = view_of(my_first);
        fetch_values(pv, (pv.lo / VCK) * VCK);
    }
    pdl_wait();                                                 // this step's query, key and value from here on
    for (int d = threadIdx.x; d < head_dim; d += NW * 32) q_smem[d] = to_float(q[(long long)t * ldq + h * head_dim + d]);
    __syncthreads();

    for (int page_idx = my_first; page_idx <= last_page; page_idx += NW) {
        if (page_idx != my_first) {
            pv = view_of(page_idx);
            fetch_values(pv, (pv.lo / VCK) * VCK);
        }
        TE* kpage = pv.kpage;
        TE* vpage = pv.vpage;
        const int lo = pv.lo, hi = pv.hi, hi_cache = pv.hi_cache;
        const bool has_new = pv.has_new;
        const int v_first = (lo / VCK) * VCK;                   // fetch that holds the first visible key
        const TE* kn = has_new ? k_new + (long long)t * ldk + kvh * head_dim : nullptr;
        const TE* vn = has_new ? v_new + (long long)t * ldv + kvh * head_dim : nullptr;
        if (has_new && h % group == 0) {
            // append: this step's key and value of the kv head go to their place in the page
            TE* kd = kpage + (long long)(hi - 1) * head_dim;
            for (int d = lane; d < head_dim; d += 32) {
                kd[d] = kn[d];
                vpage[(long long)d * AD_PAGE + hi - 1] = vn[d];
            }
        }

        // scores: lane -> keys lane and lane + 32 of the page
        float s0 = -INFINITY, s1 = -INFINITY;
        {
            const int j0 = lane, j1 = lane + 32;
            const bool in0 = j0 >= lo && j0 < hi_cache, in1 = j1 >= lo && j1 < hi_cache;
            const bool new0 = has_new && j0 == hi - 1, new1 = has_new && j1 == hi - 1;
            // a lane without a visible key reads the page's first visible row and drops the result
            const TE* safe = (hi_cache > lo) ? kpage + (long long)lo * head_dim : kn;
            const TE* k0 = in0 ? kpage + (long long)j0 * head_dim : (new0 ? kn : safe);
            const TE* k1 = in1 ? kpage + (long long)j1 * head_dim : (new1 ? kn : safe);
            float d0, d1;
            dot_head2(q_smem, k0, k1, head_dim, d0, d1);
            if (in0 || new0) s0 = d0 * scale;
            if (in1 || new1) s1 = d1 * scale;
        }
        const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));        // finite: the page has a visible key
        const float p_new = (has_new && (hi - 1) % 32 == lane) ? 1.0f : 0.0f;     // marks the lane that scored the new key
        float p0 = (s0 == -INFINITY) ? 0.0f : expf(s0 - m_new);
        float p1 = (s1 == -INFINITY) ? 0.0f : expf(s1 - m_new);
        const float corr = expf(m_run - m_new);                          // 0 for the warp's first page
        l_run = l_run * corr + warp_sum(p0 + p1);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < D1; ++i) acc[i] *= corr;
        // the new key's weight is taken out of the run over the cache and applied to v_new below
        const float w_new = has_new ? __shfl_sync(0xffffffffu, (hi - 1 < 32) ? p0 : p1, (hi - 1) & 31) : 0.0f;
        if (p_new != 0.0f) { if (hi - 1 < 32) p0 = 0.0f; else p1 = 0.0f; }

        for (int c0 = v_first; c0 < hi_cache; c0 += VCK) {
            if (c0 != v_first) fetch_values(pv, c0);
#pragma unroll
            for (int jj = 0; jj < VCK; ++jj) {
                const int j = c0 + jj;                           // positions outside [lo, hi_cache) carry p = 0
                const float pj = __shfl_sync(0xffffffffu, (j < 32) ? p0 : p1, j & 31);
#pragma unroll
                for (int i = 0; i < D1; ++i)
                    acc[i] = fmaf(pj, to_float(reinterpret_cast<const TE*>(&vraw[i][0])[jj]), acc[i]);
            }
        }
        if (has_new) {
#pragma unroll
            for (int i = 0; i < D1; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(w_new, to_float(vn[d]), acc[i]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < D1; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) part_o[warp][d] = acc[i];
    }
    if (lane == 0) { part_m[warp] = m_run; part_l[warp] = l_run; }
    __syncthreads();

    // merge in warp order; warps without a page carry max = -inf and weigh nothing.  The weights
    // exp(max_w - max) are computed once, by one thread each, not by every thread for itself.
    __shared__ float weight[NW];
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) big = fmaxf(big, part_m[w]);
    if (threadIdx.x < NW) weight[threadIdx.x] = part_m[threadIdx.x] == -INFINITY ? 0.0f : expf(part_m[threadIdx.x] - big);
    __syncthreads();
    if (threadIdx.x < head_dim) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) total = fmaf(part_l[w], weight[w], total);
        const float inv = 1.0f / total;
        for (int d = threadIdx.x; d < head_dim; d += NW * 32) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) o = fmaf(part_o[w][d], weight[w], o);
            out[(long long)t * ldo + h * head_dim + d] = from_float<TE>(o * inv);
        }
    }
}

}  // namespace mu

// One query token per sequence.  n_splits: warps per block, each taking every n_splits-th page of
// its sequence (1, 2, 4, 8 or 16; more pages than warps are folded by the warps in turn).
// tok_seq may be null when token t belongs to sequence t.  k_new / v_new: this step's keys and
// values ([n_tokens, n_kv_heads * head_dim] views) to be appended, or null if the cache holds them
// already.  The cache must have pages of 64 positions.
MU_EXPORT int mu_attention_decode(const void* q, long long ldq, const void* k_new, long long ldk,
                                  const void* v_new, long long ldv, void* out, long long ldo, void* kv,
                                  const int* block_table, int max_pages, int page_tokens,
                                  const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads,
                                  int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                  int max_warps, int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (page_tokens != mu::AD_PAGE) return MU_ERR_UNSUPPORTED_SIZE;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0) return MU_ERR_BAD_ARGUMENT;
    if (!q || !out || !kv || !block_table || !tok_pos) return MU_ERR_BAD_ARGUMENT;
    if ((k_new == nullptr) != (v_new == nullptr)) return MU_ERR_BAD_ARGUMENT;
    if (n_splits < 1) return MU_ERR_BAD_ARGUMENT;
    const long long items = (long long)n_tokens * n_heads;
    if (items > 2147483647ll) return MU_ERR_UNSUPPORTED_SIZE;
    dim3 grid((unsigned)items);
    cudaStream_t s = (cudaStream_t)stream;
    const int dp = (head_dim + 63) / 64;
    // a warp per page while the GPU has room for them; with many sequences fewer warps per block,
    // each folding several pages, so that several blocks share an SM and overlap their waits
    const int sms = mu::sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    long long room = ((long long)sms * 16 * 2) / items;
    if (room < 1) room = 1;
    const int want = n_splits < room ? n_splits : (int)room;
    int nw = want >= 16 ? 16 : want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;
    if (max_warps > 0)
        while (nw > 1 && nw > max_warps) nw /= 2;
    int rc = MU_OK;
#define MU_AD(TE, DP, NW)                                                                               \
    rc = mu::launch_pdl(mu::attention_decode_kernel<TE, DP, NW>, grid, dim3(NW * 32), 0, s, 1,          \
        (const TE*)q, ldq, (const TE*)k_new, ldk, (const TE*)v_new, ldv, (TE*)out, ldo, (TE*)kv,       \
        block_table, max_pages, tok_pos, tok_seq, n_heads, n_kv_heads, head_dim, scale, window)
#define MU_AD_W(TE, DP)                        \
    do {                                       \
        if (nw == 16) MU_AD(TE, DP, 16);       \
        else if (nw == 8) MU_AD(TE, DP, 8);    \
        else if (nw == 4) MU_AD(TE, DP, 4);    \
        else if (nw == 2) MU_AD(TE, DP, 2);    \
        else MU_AD(TE, DP, 1);                 \
    } while (0)
#define MU_AD_T(TE)                        \
    do {                                   \
        if (dp <= 1) MU_AD_W(TE, 1);       \
        else if (dp <= 2) MU_AD_W(TE, 2);  \
        else MU_AD_W(TE, 4);               \
    } while (0)
    if (is_bf16) MU_AD_T(__nv_bfloat16);
    else MU_AD_T(float);
#undef MU_AD_T
#undef MU_AD_W
#undef MU_AD
    return rc;
}
