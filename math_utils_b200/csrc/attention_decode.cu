// Single-token attention over the paged cache, one launch per layer.
//
// Each sequence brings one query token.  One warp takes one (sequence, head,
// cache page): the page's 64 keys of that head are one contiguous block, so a
// lane computes two scores (16-byte loads along the head), the warp does the
// max-subtracted softmax of the page in float32, and the lanes, now spread over
// the head's dimensions, add up the weighted values with the loads of a whole
// unrolled group in flight together.  The warp parks its partial (max, sum,
// unnormalised values) in scratch and takes a ticket; the warp that takes the
// last ticket of a (sequence, head) merges the pages in page order, so the
// result does not depend on which warp came last, and puts the ticket counter
// back to zero for the next launch.
//
// The new token's own key and value need not be in the cache yet: given
// `k_new` / `v_new` (this step's projections) the kernel reads them from there,
// and the first query head of each kv head copies them into the page.  That
// folds the cache append and the merge of the split into the attention launch
// (3 launches -> 1).
//
// Formulas: include/ai/Kernels.hpp:132-161.  Split and merge after the idea of
// src/gpu/Kernels.metal:284-345 (128-key partitions there, 64-key pages here).
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int AD_WARPS = 4;
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

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// Two neighbouring elements as they lie in memory, widened only when used.
template <typename TE> struct RawPair;
template <> struct RawPair<float> {
    float2 v;
    __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float2*>(p); }
    __device__ __forceinline__ void zero() { v = make_float2(0.0f, 0.0f); }
    __device__ __forceinline__ float2 get() const { return v; }
};
template <> struct RawPair<__nv_bfloat16> {
    __nv_bfloat162 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const __nv_bfloat162*>(p); }
    __device__ __forceinline__ void zero() { v = __floats2bfloat162_rn(0.0f, 0.0f); }
    __device__ __forceinline__ float2 get() const { return __bfloat1622float2(v); }
};

// DP: pairs of head dimensions per lane (lane owns dims 2*lane + 64*i, +1).
template <typename TE, int DP>
__global__ void __launch_bounds__(AD_WARPS * 32)
attention_decode_kernel(const TE* __restrict__ q, long long ldq, const TE* __restrict__ k_new, long long ldk,
                        const TE* __restrict__ v_new, long long ldv, TE* __restrict__ out, long long ldo,
                        TE* kv, const int* __restrict__ block_table, int max_pages,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, int n_tokens,
                        int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                        float* part_o, float* part_ml, int* tickets) {
    __shared__ float q_smem[AD_WARPS][DP * 64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * AD_WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int page_idx = blockIdx.y;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int group = n_heads / n_kv_heads;
    const int kvh = h / group;
    const int pos = tok_pos[t];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_page = first / AD_PAGE, last_page = pos / AD_PAGE;
    if (page_idx < first_page || page_idx > last_page) return;      // no key of this page is visible

    const int* pages = block_table + (long long)tok_seq[t] * max_pages;
    const long long head_stride = (long long)AD_PAGE * head_dim;
    TE* kpage = kv + ((long long)pages[page_idx] * 2 * n_kv_heads + kvh) * head_stride;
    TE* vpage = kpage + (long long)n_kv_heads * head_stride;
    const int base = page_idx * AD_PAGE;
    const int lo = max(first - base, 0);                       // first visible key inside the page
    const int hi = min(pos + 1 - base, AD_PAGE);               // one past the last visible key
    const bool has_new = (k_new != nullptr) && page_idx == last_page;   // the query's own key lives here
    const int hi_cache = has_new ? hi - 1 : hi;                // keys to be read from the cache
    const TE* kn = has_new ? k_new + (long long)t * ldk + kvh * head_dim : nullptr;
    const TE* vn = has_new ? v_new + (long long)t * ldv + kvh * head_dim : nullptr;

    // The values are asked for first, so that they travel while the scores are computed: VC keys
    // at a time (as many as fit 64 registers), each lane its own dimensions of every key.  These
    // rows were written by earlier steps, so they may be read before the kernels ahead have finished.
    pdl_trigger();
    constexpr int VC = 64 / (DP * (int)(sizeof(TE) / 2));
    RawPair<TE> vreg[VC][DP];
    auto fetch_values = [&](int j0) {
#pragma unroll
        for (int jj = 0; jj < VC; ++jj) {
            const int j = j0 + jj;
            const TE* vrow = vpage + (long long)j * head_dim;
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                const int d = 2 * lane + 64 * i;
                if (j >= lo && j < hi_cache && d < head_dim) vreg[jj][i].load(vrow + d);
                else vreg[jj][i].zero();
            }
        }
    };
    const int v_first = (lo / VC) * VC;                     // chunk that holds the first visible key
    fetch_values(v_first);
    pdl_wait();                                             // this step's query, key and value from here on

    float* qs = q_smem[warp];
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_float(q[(long long)t * ldq + h * head_dim + d]);
    if (has_new && h % group == 0) {
        // append: this step's key and value of the kv head go to their place in the page
        TE* kd = kpage + (long long)(hi - 1) * head_dim;
        TE* vd = vpage + (long long)(hi - 1) * head_dim;
        for (int d = lane; d < head_dim; d += 32) { kd[d] = kn[d]; vd[d] = vn[d]; }
    }
    __syncwarp();

    // scores: lane -> keys lane and lane + 32 of the page
    float s0 = -INFINITY, s1 = -INFINITY;
    {
        const int j0 = lane, j1 = lane + 32;
        const bool in0 = j0 >= lo && j0 < hi_cache, in1 = j1 >= lo && j1 < hi_cache;
        const bool new0 = has_new && j0 == hi - 1, new1 = has_new && j1 == hi - 1;
        const TE* k0 = in0 ? kpage + (long long)j0 * head_dim : kn;
        const TE* k1 = in1 ? kpage + (long long)j1 * head_dim : kn;
        if (in0 || new0) s0 = dot_head(qs, k0, head_dim) * scale;
        if (in1 || new1) s1 = dot_head(qs, k1, head_dim) * scale;
    }
    const float m = warp_max(fmaxf(s0, s1));
    const float p0 = (s0 == -INFINITY) ? 0.0f : expf(s0 - m);
    const float p1 = (s1 == -INFINITY) ? 0.0f : expf(s1 - m);
    const float l = warp_sum(p0 + p1);

    float2 acc[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) acc[i] = make_float2(0.0f, 0.0f);
    for (int c0 = v_first; c0 < hi_cache; c0 += VC) {
        if (c0 != v_first) fetch_values(c0);
#pragma unroll
        for (int jj = 0; jj < VC; ++jj) {
            const int j = c0 + jj;                           // keys outside [lo, hi_cache) carry p = 0 or v = 0
            const float pj = __shfl_sync(0xffffffffu, (j < 32) ? p0 : p1, j & 31);
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                const float2 v = vreg[jj][i].get();
                acc[i].x = fmaf(pj, v.x, acc[i].x);
                acc[i].y = fmaf(pj, v.y, acc[i].y);
            }
        }
    }
    if (has_new) {
        const int j = hi - 1;
        const float pj = (j < 32) ? __shfl_sync(0xffffffffu, p0, j) : __shfl_sync(0xffffffffu, p1, j - 32);
#pragma unroll
        for (int i = 0; i < DP; ++i) {
            const int d = 2 * lane + 64 * i;
            if (d < head_dim) {
                const float2 v = load2(vn + d);
                acc[i].x = fmaf(pj, v.x, acc[i].x);
                acc[i].y = fmaf(pj, v.y, acc[i].y);
            }
        }
    }

    const int n_visible = last_page - first_page + 1;
    if (n_visible == 1) {                                   // nothing to merge
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
            const int d = 2 * lane + 64 * i;
            if (d < head_dim) {
                TE* o = out + (long long)t * ldo + h * head_dim + d;
                o[0] = from_float<TE>(acc[i].x * inv);
                o[1] = from_float<TE>(acc[i].y * inv);
            }
        }
        return;
    }

    const long long unit = item * n_splits + page_idx;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < head_dim) *reinterpret_cast<float2*>(part_o + unit * head_dim + d) = acc[i];
    }
    if (lane == 0) {
        part_ml[unit * 2] = m;
        part_ml[unit * 2 + 1] = l;
    }
    __threadfence();                                        // the partial is out before the ticket is taken
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(&tickets[item], 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != n_visible - 1) return;
    __threadfence();                                        // the others' partials are visible from here on
    if (lane == 0) tickets[item] = 0;                       // ready for the next launch

    const float* ml = part_ml + item * n_splits * 2;
    float big = -INFINITY;
    for (int s = first_page; s <= last_page; ++s) big = fmaxf(big, __ldcg(ml + 2 * s));
    float total = 0.0f;
    float2 o[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) o[i] = make_float2(0.0f, 0.0f);
#pragma unroll 4
    for (int s = first_page; s <= last_page; ++s) {
        const float w = expf(__ldcg(ml + 2 * s) - big);
        total = fmaf(__ldcg(ml + 2 * s + 1), w, total);
        const float* po = part_o + (item * n_splits + s) * head_dim;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
            const int d = 2 * lane + 64 * i;
            if (d < head_dim) {
                const float2 v = __ldcg(reinterpret_cast<const float2*>(po + d));
                o[i].x = fmaf(v.x, w, o[i].x);
                o[i].y = fmaf(v.y, w, o[i].y);
            }
        }
    }
    const float inv = 1.0f / total;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < head_dim) {
            TE* dst = out + (long long)t * ldo + h * head_dim + d;
            dst[0] = from_float<TE>(o[i].x * inv);
            dst[1] = from_float<TE>(o[i].y * inv);
        }
    }
}

}  // namespace mu

// One query token per sequence.  n_splits = pages per sequence that the launch covers (at least
// max position / 64 + 1).  Scratch: part_o [n_tokens * n_heads * n_splits * head_dim] floats,
// part_ml [n_tokens * n_heads * n_splits * 2] floats, tickets [n_tokens * n_heads] ints that are
// zero before the first launch (each launch leaves them zero).  k_new / v_new: this step's keys
// and values ([n_tokens, n_kv_heads * head_dim] views) to be appended, or null if the cache holds
// them already.  The cache must have pages of 64 positions.
MU_EXPORT int mu_attention_decode(const void* q, long long ldq, const void* k_new, long long ldk,
                                  const void* v_new, long long ldv, void* out, long long ldo, void* kv,
                                  const int* block_table, int max_pages, int page_tokens,
                                  const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads,
                                  int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                  float* part_o, float* part_ml, int* tickets, int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (page_tokens != mu::AD_PAGE) return MU_ERR_UNSUPPORTED_SIZE;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return MU_ERR_UNSUPPORTED_SIZE;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0) return MU_ERR_BAD_ARGUMENT;
    if (!q || !out || !kv || !block_table || !tok_pos || !tok_seq) return MU_ERR_BAD_ARGUMENT;
    if ((k_new == nullptr) != (v_new == nullptr)) return MU_ERR_BAD_ARGUMENT;
    if (n_splits < 1 || n_splits > max_pages || n_splits > 65535) return MU_ERR_BAD_ARGUMENT;
    if (n_splits > 1 && (!part_o || !part_ml || !tickets)) return MU_ERR_BAD_ARGUMENT;
    const long long items = (long long)n_tokens * n_heads;
    dim3 grid((unsigned)((items + mu::AD_WARPS - 1) / mu::AD_WARPS), n_splits);
    cudaStream_t s = (cudaStream_t)stream;
    const int dp = (head_dim + 63) / 64;
#define MU_AD(TE, DP)                                                                                  \
    rc = mu::launch_pdl(mu::attention_decode_kernel<TE, DP>, grid, dim3(mu::AD_WARPS * 32), 0, s, 1,    \
        (const TE*)q, ldq, (const TE*)k_new, ldk, (const TE*)v_new, ldv, (TE*)out, ldo, (TE*)kv,       \
        block_table, max_pages, tok_pos, tok_seq, n_tokens, n_heads, n_kv_heads, head_dim, scale,      \
        window, n_splits, part_o, part_ml, tickets)
#define MU_AD_T(TE)                      \
    do {                                 \
        if (dp <= 1) MU_AD(TE, 1);       \
        else if (dp <= 2) MU_AD(TE, 2);  \
        else MU_AD(TE, 4);               \
    } while (0)
    int rc = MU_OK;
    if (is_bf16) MU_AD_T(__nv_bfloat16);
    else MU_AD_T(float);
#undef MU_AD_T
#undef MU_AD
    return rc;
}
