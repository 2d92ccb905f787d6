// Attention over the paged key/value cache, on CUDA cores, for any element type.
//
// Cache of one layer: pages of `page_tokens` positions,
//     keys    kv[page][0][kv_head][position in page][head_dim]
//     values  kv[page][1][kv_head][head_dim][position in page]     (transposed)
// Keys lie position-major, so a query's dot product with one key reads one contiguous row;
// values lie dimension-major, so the weighted sum over positions reads contiguous runs of
// positions for each output dimension, which is also the operand layout the tensor-core
// kernels want for both products.  A block table `block_table[s][i]` = page that holds positions
// [i * page_tokens, (i + 1) * page_tokens) of the s-th sequence of the step
// (`tok_seq[t]` says which sequence token t belongs to, `tok_pos[t]` where).
//
// mu_kv_append   copies this step's keys and values into their pages.
// mu_attention   one warp per (query token, head, key split): scores over the
//                keys first..position (a window cuts `first`), max-subtracted
//                softmax, weighted values; everything in float32 whatever the
//                storage type.  It serves whole prompts (each query sees the
//                keys the same step appended before it) and single-token
//                steps; with n_splits > 1 each warp takes a slice of the keys
//                and writes an unnormalised partial (max, sum, values) that
//                mu_attention_merge combines.
// The formulas are those of include/ai/Kernels.hpp:132-161; the split and merge
// follow the idea of src/gpu/Kernels.metal:284-345.
#include "common.cuh"

#include <math.h>

namespace mu {

template <typename TE>
__global__ void kv_append_kernel(const TE* __restrict__ k, long long ldk, const TE* __restrict__ v,
                                 long long ldv, const int* __restrict__ tok_pos,
                                 const int* __restrict__ tok_seq,
                                 const int* __restrict__ block_table, int max_pages, int page_tokens,
                                 int n_kv_heads, int head_dim, TE* __restrict__ kv) {
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const long long page = block_table[(long long)tok_seq[t] * max_pages + pos / page_tokens];
    const int off = pos % page_tokens;
    const int width = n_kv_heads * head_dim;
    const long long head_stride = (long long)page_tokens * head_dim;
    TE* kdst = kv + (page * 2 + 0) * n_kv_heads * head_stride + (long long)off * head_dim;
    TE* vdst = kv + (page * 2 + 1) * n_kv_heads * head_stride + off;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int h = i / head_dim, d = i % head_dim;
        kdst[h * head_stride + d] = k[(long long)t * ldk + i];
        vdst[h * head_stride + (long long)d * page_tokens] = v[(long long)t * ldv + i];
    }
}

// The same copy in 16-byte pieces, for rows and strides that allow it.  (WITH_V false: keys only.)
template <typename TE, bool WITH_V>
__global__ void kv_append_vec_kernel(const TE* __restrict__ k, long long ldk, const TE* __restrict__ v,
                                     long long ldv, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                     int max_pages, int page_tokens, int n_kv_heads, int head_dim,
                                     TE* __restrict__ kv) {
    constexpr int E = 16 / (int)sizeof(TE);               // elements per piece
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const long long page = block_table[(long long)tok_seq[t] * max_pages + pos / page_tokens];
    const int off = pos % page_tokens;
    const int pieces_per_head = head_dim / E, pieces = n_kv_heads * pieces_per_head;
    const long long head_stride = (long long)page_tokens * head_dim;
    TE* kdst = kv + (page * 2 + 0) * n_kv_heads * head_stride + (long long)off * head_dim;
    TE* vdst = kv + (page * 2 + 1) * n_kv_heads * head_stride + off;
#pragma unroll 2
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        const int h = i / pieces_per_head, d = (i % pieces_per_head) * E;
        const uint4 kk = *reinterpret_cast<const uint4*>(k + (long long)t * ldk + h * head_dim + d);
        *reinterpret_cast<uint4*>(kdst + h * head_stride + d) = kk;
        if (WITH_V) {
            // the value's elements go one by one to their dimension rows
            const uint4 vv = *reinterpret_cast<const uint4*>(v + (long long)t * ldv + h * head_dim + d);
            const TE* ve = reinterpret_cast<const TE*>(&vv);
#pragma unroll
            for (int e = 0; e < E; ++e) vdst[h * head_stride + (long long)(d + e) * page_tokens] = ve[e];
        }
    }
}

// Keys and values of a whole tile of prompt tokens (up to 64 consecutive tokens of one sequence) for
// one kv head.  Keys are copied row by row in 16-byte pieces.  Values are turned in shared memory so
// that each dimension row of the page is written as runs of consecutive positions: 16 bytes at a time
// where the tile starts at a position that allows it, element by element otherwise.
// tiles: int32 [n][2] = (first flat token, count).
template <typename TE>
__global__ void __launch_bounds__(256)
kv_append_tiles_kernel(const TE* __restrict__ k, long long ldk, const TE* __restrict__ v, long long ldv,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ block_table, int max_pages, int page_tokens,
                       const int* __restrict__ tiles, int n_kv_heads, int head_dim, TE* __restrict__ kv) {
    constexpr int E = 16 / (int)sizeof(TE);                      // elements per 16-byte piece
    constexpr int W = 4 / (int)sizeof(TE);                       // elements per 32-bit word
    extern __shared__ __align__(16) unsigned char vt_raw[];
    uint32_t* tile = reinterpret_cast<uint32_t*>(vt_raw);        // [64][pitch] words
    const int pitch = head_dim / W + 1;                          // an odd number of words per row
    pdl_trigger();
    pdl_wait();
    const int flat0 = tiles[2 * blockIdx.x], n = min(tiles[2 * blockIdx.x + 1], 64);   // the tile buffer holds 64 rows
    const int h = blockIdx.y;
    const int* pages = block_table + (long long)tok_seq[flat0] * max_pages;
    const int pos0 = tok_pos[flat0];
    const long long head_stride = (long long)page_tokens * head_dim;
    const int ppr = head_dim / E;                                // pieces per row
    for (int i = threadIdx.x; i < n * ppr; i += blockDim.x) {
        const int r = i / ppr, c = i % ppr, pos = pos0 + r;
        const long long src = (long long)(flat0 + r) * ldk + h * head_dim + c * E;
        TE* kdst = kv + ((long long)pages[pos / page_tokens] * 2 * n_kv_heads + h) * head_stride;
        *reinterpret_cast<uint4*>(kdst + (long long)(pos % page_tokens) * head_dim + c * E) =
            *reinterpret_cast<const uint4*>(k + src);
        const uint4 vv = *reinterpret_cast<const uint4*>(v + (long long)(flat0 + r) * ldv + h * head_dim + c * E);
        uint32_t* row = tile + r * pitch + c * 4;
        row[0] = vv.x; row[1] = vv.y; row[2] = vv.z; row[3] = vv.w;
    }
    __syncthreads();
    const TE* te = reinterpret_cast<const TE*>(tile);
    const int pitch_e = pitch * W;
    const int runs = (pos0 % E == 0) ? n / E : 0;                // whole 16-byte runs of positions
    // lanes along the runs of a dimension row (one row of the page is contiguous), then along dimensions
    const int rpd = 64 / E;                                      // runs a dimension row of a full tile has
    for (int i = threadIdx.x; i < head_dim * rpd; i += blockDim.x) {
        const int run = i % rpd, d = i / rpd;
        if (run >= runs) continue;
        const int pos = pos0 + run * E;
        __align__(16) TE piece[E];
#pragma unroll
        for (int e = 0; e < E; ++e) piece[e] = te[(run * E + e) * pitch_e + d];
        TE* vdst = kv + (((long long)pages[pos / page_tokens] * 2 + 1) * n_kv_heads + h) * head_stride;
        *reinterpret_cast<uint4*>(vdst + (long long)d * page_tokens + pos % page_tokens) =
            *reinterpret_cast<const uint4*>(piece);
    }
    const int rest0 = runs * E;                                  // what the runs left: one element at a time
    for (int i = threadIdx.x; i < (n - rest0) * head_dim; i += blockDim.x) {
        const int r = rest0 + i % (n - rest0), d = i / (n - rest0), pos = pos0 + r;
        TE* vdst = kv + (((long long)pages[pos / page_tokens] * 2 + 1) * n_kv_heads + h) * head_stride;
        vdst[(long long)d * page_tokens + pos % page_tokens] = te[r * pitch_e + d];
    }
}

__device__ __forceinline__ float dot_row(const float* qs, const float* krow, int head_dim) {
    float s = 0.0f;
    for (int d = 0; d < head_dim; d += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(krow + d);
        s = fmaf(qs[d], kk.x, s);
        s = fmaf(qs[d + 1], kk.y, s);
        s = fmaf(qs[d + 2], kk.z, s);
        s = fmaf(qs[d + 3], kk.w, s);
    }
    return s;
}
__device__ __forceinline__ float dot_row(const float* qs, const __nv_bfloat16* krow, int head_dim) {
    float s = 0.0f;
    for (int d = 0; d < head_dim; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            s = fmaf(qs[d + 2 * i], f.x, s);
            s = fmaf(qs[d + 2 * i + 1], f.y, s);
        }
    }
    return s;
}

// 32 consecutive values of one dimension row of a value page, widened.
__device__ __forceinline__ void load_run32(const float* p, float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 x = reinterpret_cast<const float4*>(p)[i];
        v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
    }
}
__device__ __forceinline__ void load_run32(const __nv_bfloat16* p, float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 raw = reinterpret_cast<const uint4*>(p)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y;
        }
    }
}

// The same for a head size whose rows are not whole 16-byte pieces: one element at a time.
template <typename TE>
__device__ __forceinline__ float dot_row_any(const float* qs, const TE* krow, int head_dim) {
    float s = 0.0f;
    for (int d = 0; d < head_dim; ++d) s = fmaf(qs[d], to_float(krow[d]), s);
    return s;
}

constexpr int ATT_WARPS = 4;

// DPL: dimensions per lane (head_dim <= 32 * DPL).  VEC: key rows are whole 16-byte pieces.
template <typename TE, int DPL, bool VEC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_kernel(const TE* __restrict__ q, long long ldq, TE* __restrict__ out, long long ldo,
                 const TE* __restrict__ kv, const int* __restrict__ block_table, int max_pages,
                 int page_tokens, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                 int n_tokens, int n_heads, int n_kv_heads,
                 int head_dim, float scale, int window, int n_splits, int split_keys,
                 float* __restrict__ part_o, float* __restrict__ part_ml) {
    __shared__ float q_smem[ATT_WARPS][DPL * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;          // whole warps leave together
    const int split = blockIdx.y;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = tok_pos[t];
    const int* pages = block_table + (long long)tok_seq[t] * max_pages;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    int lo = first, hi = pos + 1;
    if (n_splits > 1) {
        // the last split takes whatever the others leave, so no key is dropped when
        // n_splits * split_keys falls short of a sequence
        lo = max(first, split * split_keys);
        hi = split == n_splits - 1 ? pos + 1 : min(pos + 1, (split + 1) * split_keys);
    }
    float* qs = q_smem[warp];
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_float(q[(long long)t * ldq + h * head_dim + d]);
    __syncwarp();

    const long long head_stride = (long long)page_tokens * head_dim;
    const long long page_stride = 2ll * n_kv_heads * head_stride;
    const long long k_base = (long long)kvh * head_stride;
    const long long v_base = ((long long)n_kv_heads + kvh) * head_stride;

    float m = -INFINITY, l = 0.0f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;

    // keys in runs of 32 that start on multiples of 32, so that a run never crosses a page
    for (int base = lo & ~31; base < hi; base += 32) {
        const int j = base + lane;
        const bool valid = j >= lo && j < hi;
        const long long page_off = (long long)pages[base / page_tokens] * page_stride;
        float s = -INFINITY;
        if (valid) {
            const TE* krow = kv + page_off + k_base + (long long)(j % page_tokens) * head_dim;
            s = (VEC ? dot_row(qs, krow, head_dim) : dot_row_any(qs, krow, head_dim)) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.0f;   // the run holds at least one visible key
        const float corr = expf(m - m_new);               // 0 on the first run (m = -inf)
        l = l * corr + warp_sum(p);
        m = m_new;
        const TE* vhead = kv + page_off + v_base + (base % page_tokens);     // [head_dim][page_tokens], at this run
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            float v[32];
            if (d < head_dim) load_run32(vhead + (long long)d * page_tokens, v);
            float a = acc[i] * corr;
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);       // 0 for keys outside [lo, hi)
                if (d < head_dim) a = fmaf(pj, v[jj], a);
            }
            acc[i] = a;
        }
    }

    if (n_splits == 1) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) out[(long long)t * ldo + h * head_dim + d] = from_float<TE>(acc[i] * inv);
        }
    } else {
        const long long slot_idx = item * n_splits + split;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) part_o[slot_idx * head_dim + d] = acc[i];
        }
        if (lane == 0) {
            part_ml[slot_idx * 2] = m;
            part_ml[slot_idx * 2 + 1] = l;
        }
    }
}

template <typename TE>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       TE* __restrict__ out, long long ldo, int n_tokens, int n_heads,
                                       int head_dim, int n_splits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const float* ml = part_ml + item * n_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = ml[2 * s];
        if (ms != -INFINITY) l += ml[2 * s + 1] * expf(ms - m);
    }
    const float inv = 1.0f / l;
    for (int d = lane; d < head_dim; d += 32) {
        float o = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) o = fmaf(part_o[(item * n_splits + s) * head_dim + d], expf(ms - m), o);
        }
        out[(long long)t * ldo + h * head_dim + d] = from_float<TE>(o * inv);
    }
}

}  // namespace mu

static int check_paged(int page_tokens, int n_kv_heads, int head_dim, int max_pages) {
    if (page_tokens <= 0 || n_kv_heads <= 0 || max_pages <= 0) return MU_ERR_BAD_ARGUMENT;
    if (page_tokens % 32 != 0) return MU_ERR_UNSUPPORTED_SIZE;       // values are read in aligned runs of 32 positions
    if (head_dim <= 0 || head_dim > 256) return MU_ERR_UNSUPPORTED_SIZE;
    return MU_OK;
}

// tiles (optional): int32 [n_tiles][2] = (first flat token, count <= 64) covering all tokens, each tile
// within one sequence; with them the values are written a tile at a time, position runs together.
MU_EXPORT int mu_kv_append(const void* k, long long ldk, const void* v, long long ldv,
                           const int* tok_pos, const int* tok_seq,
                           const int* block_table, int max_pages, int page_tokens, int n_tokens,
                           int n_kv_heads, int head_dim, void* kv, int is_bf16, const int* tiles, int n_tiles,
                           void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (int e = check_paged(page_tokens, n_kv_heads, head_dim, max_pages)) return e;
    if (!k || !v || !kv || !tok_pos || !tok_seq || !block_table) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = n_kv_heads * head_dim >= 256 ? 256 : 128;
    const int e = is_bf16 ? 8 : 4;
    if (head_dim % e == 0 && ldk % e == 0 && ldv % e == 0 && !((uintptr_t)k & 15) && !((uintptr_t)v & 15) &&
        !((uintptr_t)kv & 15)) {
        const int vthreads = n_kv_heads * head_dim / e >= 128 ? 128 : 64;
        const bool tiled = tiles != nullptr && n_tiles > 0 && n_kv_heads <= 65535 && page_tokens % 8 == 0;
        if (tiled) {
            dim3 grid(n_tiles, n_kv_heads);
            const size_t smem = (size_t)64 * (head_dim * (is_bf16 ? 2 : 4) + 4);
            if (is_bf16) {
                mu::prefer_shared_memory(reinterpret_cast<const void*>(mu::kv_append_tiles_kernel<__nv_bfloat16>));   // a prompt-step kernel
                return mu::launch_pdl(mu::kv_append_tiles_kernel<__nv_bfloat16>, grid, dim3(256), smem, s, 1,
                                      (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, tok_pos, tok_seq,
                                      block_table, max_pages, page_tokens, tiles, n_kv_heads, head_dim,
                                      (__nv_bfloat16*)kv);
            } else {
                if (smem > 48 * 1024) {
                    static bool raised = false;
                    if (!raised && cudaFuncSetAttribute(mu::kv_append_tiles_kernel<float>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
                        return MU_ERR_LAUNCH;
                    raised = true;
                }
                return mu::launch_pdl(mu::kv_append_tiles_kernel<float>, grid, dim3(256), smem, s, 1, (const float*)k,
                                      ldk, (const float*)v, ldv, tok_pos, tok_seq, block_table, max_pages,
                                      page_tokens, tiles, n_kv_heads, head_dim, (float*)kv);
            }
            MU_CHECK_LAUNCH();
            return MU_OK;
        }
        if (is_bf16)
            mu::kv_append_vec_kernel<__nv_bfloat16, true><<<n_tokens, vthreads, 0, s>>>(
                (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, tok_pos, tok_seq, block_table,
                max_pages, page_tokens, n_kv_heads, head_dim, (__nv_bfloat16*)kv);
        else
            mu::kv_append_vec_kernel<float, true><<<n_tokens, vthreads, 0, s>>>(
                (const float*)k, ldk, (const float*)v, ldv, tok_pos, tok_seq, block_table, max_pages,
                page_tokens, n_kv_heads, head_dim, (float*)kv);
        MU_CHECK_LAUNCH();
        return MU_OK;
    }
    if (is_bf16)
        mu::kv_append_kernel<__nv_bfloat16><<<n_tokens, threads, 0, s>>>(
            (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, tok_pos, tok_seq,
            block_table, max_pages, page_tokens, n_kv_heads, head_dim, (__nv_bfloat16*)kv);
    else
        mu::kv_append_kernel<float><<<n_tokens, threads, 0, s>>>(
            (const float*)k, ldk, (const float*)v, ldv, tok_pos, tok_seq, block_table,
            max_pages, page_tokens, n_kv_heads, head_dim, (float*)kv);
    MU_CHECK_LAUNCH();
    return MU_OK;
}

// n_splits > 1 needs part_o [n_tokens * n_heads * n_splits * head_dim] and
// part_ml [n_tokens * n_heads * n_splits * 2] floats of scratch, and split s takes
// the keys [s * split_keys, (s + 1) * split_keys); the last split goes on to the
// token's own position.  Any head size up to 256.
MU_EXPORT int mu_attention(const void* q, long long ldq, void* out, long long ldo, const void* kv,
                           const int* block_table, int max_pages, int page_tokens,
                           const int* tok_pos, const int* tok_seq, int n_tokens,
                           int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                           int n_splits, int split_keys, float* part_o, float* part_ml,
                           int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (int e = check_paged(page_tokens, n_kv_heads, head_dim, max_pages)) return e;
    if (n_heads <= 0 || n_heads % n_kv_heads != 0 || window < 0) return MU_ERR_BAD_ARGUMENT;
    if (!q || !out || !kv || !tok_pos || !tok_seq || !block_table) return MU_ERR_BAD_ARGUMENT;
    if (n_splits < 1 || n_splits > 65535) return MU_ERR_BAD_ARGUMENT;
    if (n_splits > 1 && (!part_o || !part_ml || split_keys <= 0)) return MU_ERR_BAD_ARGUMENT;
    const long long items = (long long)n_tokens * n_heads;
    dim3 grid((unsigned)((items + mu::ATT_WARPS - 1) / mu::ATT_WARPS), n_splits);
    cudaStream_t s = (cudaStream_t)stream;
    const int dpl = (head_dim + 31) / 32;
    // key rows in 16-byte pieces where the head size and the cache's address allow it
    const bool vec = head_dim % (is_bf16 ? 8 : 4) == 0 && !((uintptr_t)kv & 15);
#define MU_ATT(TE, DPL, VEC)                                                                     \
    mu::attention_kernel<TE, DPL, VEC><<<grid, mu::ATT_WARPS * 32, 0, s>>>(                       \
        (const TE*)q, ldq, (TE*)out, ldo, (const TE*)kv, block_table, max_pages, page_tokens,    \
        tok_pos, tok_seq, n_tokens, n_heads, n_kv_heads, head_dim, scale, window,      \
        n_splits, split_keys, part_o, part_ml)
#define MU_ATT_T(TE)                                     \
    do {                                                 \
        if (!vec) {                                      \
            if (dpl <= 2) MU_ATT(TE, 2, false);          \
            else MU_ATT(TE, 8, false);                   \
        } else if (dpl <= 1) MU_ATT(TE, 1, true);        \
        else if (dpl <= 2) MU_ATT(TE, 2, true);          \
        else if (dpl <= 4) MU_ATT(TE, 4, true);          \
        else MU_ATT(TE, 8, true);                        \
    } while (0)
    if (is_bf16) MU_ATT_T(__nv_bfloat16);
    else MU_ATT_T(float);
#undef MU_ATT_T
#undef MU_ATT
    MU_CHECK_LAUNCH();
    if (n_splits > 1) {
        const int warps = 4;
        const unsigned blocks = (unsigned)((items + warps - 1) / warps);
        if (is_bf16)
            mu::attention_merge_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, s>>>(
                part_o, part_ml, (__nv_bfloat16*)out, ldo, n_tokens, n_heads, head_dim, n_splits);
        else
            mu::attention_merge_kernel<float><<<blocks, warps * 32, 0, s>>>(
                part_o, part_ml, (float*)out, ldo, n_tokens, n_heads, head_dim, n_splits);
        MU_CHECK_LAUNCH();
    }
    return MU_OK;
}

// ---------------------------------------------------------------------------
// The variant for callers that cannot allocate: see attention_static_scratch.h.
#include "attention_static_scratch.h"

#include <mutex>

// Scratch of the split attention, part of the loaded library on every device.
static __device__ __align__(256) float mu_static_scratch[MU_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MU_MAX_DEVICES = 64;
std::mutex static_scratch_mutex;
float* static_scratch_address[MU_MAX_DEVICES] = {};

// In host code `mu_static_scratch` is only a handle for the runtime, not an
// address a kernel could use: the device address is asked for once per device.
int static_scratch_for_current_device(float** ptr) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MU_MAX_DEVICES) return MU_ERR_SETUP;
    std::lock_guard<std::mutex> lock(static_scratch_mutex);
    if (!static_scratch_address[device]) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, mu_static_scratch) != cudaSuccess || !address) return MU_ERR_SETUP;
        static_scratch_address[device] = (float*)address;
    }
    *ptr = static_scratch_address[device];
    return MU_OK;
}
}  // namespace

MU_EXPORT int mu_attention_static_scratch(const void* q, long long ldq, void* out, long long ldo,
                                          const void* kv, const int* block_table, int max_pages,
                                          int page_tokens, const int* tok_pos, const int* tok_seq,
                                          int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                          float scale, int window, int n_splits, int split_keys,
                                          int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    // everything the size below is made of is checked first, so that the product cannot overflow
    if (int e = check_paged(page_tokens, n_kv_heads, head_dim, max_pages)) return e;
    if (n_heads <= 0 || n_heads > 65535 || n_splits < 1 || n_splits > 65535) return MU_ERR_BAD_ARGUMENT;
    if (n_splits > 1 && split_keys <= 0) return MU_ERR_BAD_ARGUMENT;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (n_splits > 1) {
        const long long per_token = (long long)n_heads * n_splits * (head_dim + 2);     // < 2^41 after the checks above
        if (per_token > (long long)MU_STATIC_SCRATCH_FLOATS ||
            (long long)n_tokens * per_token > (long long)MU_STATIC_SCRATCH_FLOATS)
            return MU_ERR_STATIC_SCRATCH;
        const long long units = (long long)n_tokens * n_heads * n_splits;
        float* base = nullptr;
        if (int e = static_scratch_for_current_device(&base)) return e;
        part_o = base;
        part_ml = base + units * head_dim;
    }
    return mu_attention(q, ldq, out, ldo, kv, block_table, max_pages, page_tokens, tok_pos, tok_seq,
                        n_tokens, n_heads, n_kv_heads, head_dim, scale, window, n_splits, split_keys,
                        part_o, part_ml, is_bf16, stream);
}
