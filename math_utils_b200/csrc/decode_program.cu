// A whole single-token step as ONE persistent kernel that runs a recorded program.
//
// The step of a small model is some sixty tiny kernels, each a short chain of
// round trips to memory behind a launch; their launches and drains, not their
// bytes, set the step's time.  Here the host records the step once as a list
// of operations (embedding, products with their epilogues, attention), and one
// cooperative kernel with a block per SM runs the list: every block takes its
// share of an operation's tiles, then all blocks meet at a barrier in global
// memory and go on to the next operation.  While it waits at the barrier a
// block already has the first weights of its next tile on the way (weights
// depend on nothing), so the memory system never idles across the barrier.
// The reference does the same on its Metal backend: it records one indirect
// command program per conversation and replays it per token
// (src/gpu/Metal.mm:194-396).
//
// Operations (the arithmetic is that of the stand-alone kernels):
//   EMBED      x[t] = table[id[t]] + pos_table[pos[t]]                    (elementwise.cu)
//   GEMM       C = act(A W^T + bias) (+ residual), A given or made as LayerNorm(x[rows]),
//              up to 16 rows; a tile is 16 weight rows, K split over the 8 warps of the
//              block and, for narrow outputs, over several blocks whose partial tiles are
//              added by the last one to arrive, in slice order               (gemm_skinny.cu)
//   ATTENTION  one token per sequence over the paged cache, a block per (sequence, head),
//              warps over pages, appends the step's key and value      (attention_decode.cu)
// The barrier is bounded: a block that waits longer than two seconds writes a code to
// `status` and every block leaves; nothing spins for ever.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int DP_THREADS = 256, DP_WARPS = 8;
constexpr int OP_EMBED = 1, OP_GEMM = 2, OP_ATTENTION = 3;
constexpr int DP_MAX_ROWS = 16;            // activation rows (sequences) a program may carry
constexpr int DP_PAGE = 64;

struct ProgramOp {
    int type, M, N, K;
    int act, out_bf16, has_ln, ksplit;
    // product
    const __nv_bfloat16* a; const __nv_bfloat16* w; const float* bias; const float* residual; void* c;
    const float* ln_x; const int* ln_rows; const float* ln_gamma; const float* ln_beta;
    long long lda, ldw, ldc, ldr, ln_ldx;
    float* part; int* tickets;              // partial tiles and arrival counters of a split over blocks
    float ln_eps, scale;
    // attention
    const __nv_bfloat16* q; const __nv_bfloat16* k_new; const __nv_bfloat16* v_new; __nv_bfloat16* out;
    __nv_bfloat16* kv; const int* block_table; const int* tok_pos;
    long long ldq, ldk, ldv, ldo;
    int max_pages, n_heads, n_kv_heads, head_dim, window, n_tokens;
    // embedding
    int hidden, table_bf16;
    const int* ids; const void* table; const void* pos_table; float* x;
};

struct BarrierState {
    unsigned int count;
    unsigned int generation;
};

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All blocks of the grid meet here.  Returns false (in every thread of the block) if the wait ran out.
__device__ __forceinline__ bool grid_barrier(BarrierState* bar, int* status) {
    __shared__ int ok_smem;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        const unsigned int gen = ld_acquire(&bar->generation);
        __threadfence();
        if (atomicAdd(&bar->count, 1u) == gridDim.x - 1) {
            bar->count = 0;
            __threadfence();
            atomicAdd(&bar->generation, 1u);
        } else {
            unsigned long long start = 0;
            for (unsigned int spin = 0; ld_acquire(&bar->generation) == gen; ++spin) {
                if ((spin & 1023u) == 1023u) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (start == 0) start = now;
                    else if (now - start > 2000000000ull) { ok = 0; atomicExch(status, 10); break; }
                }
            }
        }
        __threadfence();
        ok_smem = ok;
    }
    __syncthreads();
    return ok_smem != 0;
}

__device__ __forceinline__ void dp_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 dp_load_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int DP_UNROLL = 4;

// Which weight rows and which k-blocks a (unit, warp) pair works on.
struct GemmUnit {
    const __nv_bfloat16* w0; const __nv_bfloat16* w1;
    int tile, slice, kb0, kb1;
};
__device__ __forceinline__ GemmUnit gemm_unit(const ProgramOp& op, int unit, int warp, int lane) {
    GemmUnit u;
    u.tile = unit / op.ksplit;
    u.slice = unit % op.ksplit;
    const int g = lane >> 2, t = lane & 3;
    const int k_blocks = (op.K + 31) / 32;
    const int per = (k_blocks + op.ksplit * DP_WARPS - 1) / (op.ksplit * DP_WARPS);
    u.kb0 = (u.slice * DP_WARPS + warp) * per;
    u.kb1 = min(k_blocks, u.kb0 + per);
    const int r0 = min(u.tile * 16 + g, op.N - 1), r1 = min(u.tile * 16 + g + 8, op.N - 1);
    u.w0 = op.w + (long long)r0 * op.ldw + 8 * t;
    u.w1 = op.w + (long long)r1 * op.ldw + 8 * t;
    return u;
}
__device__ __forceinline__ void gemm_load(const ProgramOp& op, const GemmUnit& u, int kb, int lane, uint4* wa, uint4* wb) {
    const int t = lane & 3;
#pragma unroll
    for (int i = 0; i < DP_UNROLL; ++i) {
        const int k = (kb + i) * 32;
        const bool in = (kb + i) < u.kb1 && (k + 8 * t) < op.K;
        wa[i] = in ? dp_load_stream(u.w0 + k) : make_uint4(0, 0, 0, 0);
        wb[i] = in ? dp_load_stream(u.w1 + k) : make_uint4(0, 0, 0, 0);
    }
}

// MT: activation row tiles of 8 (1 or 2).
template <int MT>
__global__ void __launch_bounds__(DP_THREADS)
decode_program_kernel(const ProgramOp* __restrict__ ops, int n_ops, BarrierState* bar, int* status,
                      unsigned long long* trace) {
    constexpr int MP = 8 * MT;
    extern __shared__ __align__(16) unsigned char dp_dyn[];            // normed activations [MP][K + 8] bf16
    __shared__ float red[DP_WARPS][16][MP + 1];                        // per-warp partial tiles
    __shared__ float att_q[128];
    __shared__ float att_o[DP_WARPS][128];
    __shared__ float att_m[DP_WARPS], att_l[DP_WARPS], att_w[DP_WARPS];
    __shared__ int last_smem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint4 wa[DP_UNROLL], wb[DP_UNROLL];
    bool preloaded = false;

    for (int oi = 0; oi < n_ops; ++oi) {
        const ProgramOp op = ops[oi];
        if (trace && blockIdx.x == 0 && threadIdx.x == 0) {       // when block 0 began each operation
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            trace[2 * oi] = now;
        }
        if (op.type == OP_EMBED) {
            for (int row = blockIdx.x; row < op.n_tokens; row += gridDim.x) {
                const long long id = op.ids[row];
                const int pos = op.pos_table ? op.tok_pos[row] : 0;
                float* dst = op.x + (long long)row * op.hidden;
                for (int d = threadIdx.x; d < op.hidden; d += DP_THREADS) {
                    float v;
                    if (op.table_bf16) {
                        v = __bfloat162float(((const __nv_bfloat16*)op.table)[id * op.hidden + d]);
                        if (op.pos_table) v += __bfloat162float(((const __nv_bfloat16*)op.pos_table)[(long long)pos * op.hidden + d]);
                    } else {
                        v = ((const float*)op.table)[id * op.hidden + d];
                        if (op.pos_table) v += ((const float*)op.pos_table)[(long long)pos * op.hidden + d];
                    }
                    dst[d] = v;
                }
            }
        } else if (op.type == OP_GEMM) {
            const int n_tiles = (op.N + 15) / 16;
            const int n_units = n_tiles * op.ksplit;
            __nv_bfloat16* act_smem = reinterpret_cast<__nv_bfloat16*>(dp_dyn);
            const int act_ld = op.K + 8;
            if (op.has_ln && blockIdx.x < n_units) {
                // LayerNorm of the rows into shared memory, once per block (as in gemm_skinny.cu)
                constexpr int LNV = 16;
                const int n4 = op.K / 4;
                for (int m = warp; m < MP; m += DP_WARPS) {
                    __nv_bfloat16* dst = act_smem + (long long)m * act_ld;
                    if (m >= op.M) {
                        for (int k = lane * 8; k < op.K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
                        continue;
                    }
                    const float4* src4 = reinterpret_cast<const float4*>(
                        op.ln_x + (long long)(op.ln_rows ? op.ln_rows[m] : m) * op.ln_ldx);
                    float4 v[LNV];
#pragma unroll
                    for (int i = 0; i < LNV; ++i) {
                        const int idx = lane + 32 * i;
                        v[i] = idx < n4 ? src4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                    float sum = 0.0f;
#pragma unroll
                    for (int i = 0; i < LNV; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                    const float mean = warp_sum(sum) / (float)op.K;
                    float sq = 0.0f;
#pragma unroll
                    for (int i = 0; i < LNV; ++i) {
                        if (lane + 32 * i < n4) {
                            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                            sq += (a * a + b * b) + (c * c + d * d);
                        }
                    }
                    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)op.K + op.ln_eps);
                    const float4* g4 = reinterpret_cast<const float4*>(op.ln_gamma);
                    const float4* b4 = reinterpret_cast<const float4*>(op.ln_beta);
#pragma unroll
                    for (int i = 0; i < LNV; ++i) {
                        const int idx = lane + 32 * i;
                        if (idx < n4) {
                            const float4 gg = g4[idx];
                            const float4 bb = op.ln_beta ? b4[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
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
                }
                __syncthreads();
            }
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
                const GemmUnit u = gemm_unit(op, unit, warp, lane);
                if (!preloaded) gemm_load(op, u, u.kb0, lane, wa, wb);
                preloaded = false;
                const __nv_bfloat16* xrow[MT];
                bool xvalid[MT];
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    const int m = 8 * j + g;
                    xvalid[j] = op.has_ln || m < op.M;
                    xrow[j] = op.has_ln ? act_smem + (long long)m * act_ld + 8 * t
                                        : op.a + (long long)min(m, op.M - 1) * op.lda + 8 * t;
                }
                float acc[MT][4];
#pragma unroll
                for (int j = 0; j < MT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
                for (int kb = u.kb0; kb < u.kb1; kb += DP_UNROLL) {
                    if (kb != u.kb0) gemm_load(op, u, kb, lane, wa, wb);
#pragma unroll
                    for (int i = 0; i < DP_UNROLL; ++i) {
                        const int k = (kb + i) * 32;
                        const bool in = (kb + i) < u.kb1 && (k + 8 * t) < op.K;
#pragma unroll
                        for (int j = 0; j < MT; ++j) {
                            uint4 xb = make_uint4(0, 0, 0, 0);
                            if (in && xvalid[j]) xb = *reinterpret_cast<const uint4*>(xrow[j] + k);
                            dp_mma(acc[j], wa[i].x, wb[i].x, wa[i].y, wb[i].y, xb.x, xb.y);
                            dp_mma(acc[j], wa[i].z, wb[i].z, wa[i].w, wb[i].w, xb.z, xb.w);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    red[warp][g][8 * j + 2 * t] = acc[j][0];
                    red[warp][g][8 * j + 2 * t + 1] = acc[j][1];
                    red[warp][g + 8][8 * j + 2 * t] = acc[j][2];
                    red[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
                }
                __syncthreads();
                bool finish = true;
                if (op.ksplit > 1) {
                    // park the block's partial tile; the last slice to arrive adds them up in slice order
                    float* mine = op.part + ((long long)u.tile * op.ksplit + u.slice) * 16 * MP;
                    for (int idx = threadIdx.x; idx < 16 * MP; idx += DP_THREADS) {
                        const int r = idx / MP, m = idx % MP;
                        float v = 0.0f;
#pragma unroll
                        for (int s = 0; s < DP_WARPS; ++s) v += red[s][r][m];
                        mine[idx] = v;
                    }
                    __threadfence();
                    __syncthreads();
                    if (threadIdx.x == 0) {
                        const int ticket = atomicAdd(&op.tickets[u.tile], 1);
                        last_smem = ticket == op.ksplit - 1;
                        if (last_smem) op.tickets[u.tile] = 0;
                        __threadfence();
                    }
                    __syncthreads();
                    finish = last_smem != 0;
                }
                if (finish) {
                    const int col0 = u.tile * 16;
                    for (int idx = threadIdx.x; idx < 16 * op.M; idx += DP_THREADS) {
                        const int m = idx / 16, r = idx % 16;
                        const int n = col0 + r;
                        if (n >= op.N) continue;
                        float v = 0.0f;
                        if (op.ksplit > 1) {
                            const float* tile_part = op.part + (long long)u.tile * op.ksplit * 16 * MP;
                            for (int s = 0; s < op.ksplit; ++s) v += __ldcg(tile_part + s * 16 * MP + r * MP + m);
                        } else {
#pragma unroll
                            for (int s = 0; s < DP_WARPS; ++s) v += red[s][r][m];
                        }
                        if (op.bias) v += op.bias[n];
                        v = op.out_bf16 ? apply_act_bf16(v, op.act) : apply_act(v, op.act);
                        if (op.residual) v += op.residual[(long long)m * op.ldr + n];
                        if (op.out_bf16) ((__nv_bfloat16*)op.c)[(long long)m * op.ldc + n] = __float2bfloat16_rn(v);
                        else ((float*)op.c)[(long long)m * op.ldc + n] = v;
                    }
                }
                __syncthreads();
            }
        } else if (op.type == OP_ATTENTION) {
            const int items = op.n_tokens * op.n_heads;
            const int group = op.n_heads / op.n_kv_heads;
            const long long head_stride = (long long)DP_PAGE * op.head_dim;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int tk = item / op.n_heads, h = item % op.n_heads;
                const int kvh = h / group;
                const int pos = op.tok_pos[tk];
                const int* pages = op.block_table + (long long)tk * op.max_pages;
                const int first = (op.window > 0 && pos + 1 > op.window) ? pos + 1 - op.window : 0;
                const int first_page = first / DP_PAGE, last_page = pos / DP_PAGE;
                for (int d = threadIdx.x; d < op.head_dim; d += DP_THREADS)
                    att_q[d] = __bfloat162float(op.q[(long long)tk * op.ldq + h * op.head_dim + d]);
                __syncthreads();
                float m_run = -INFINITY, l_run = 0.0f;
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};                  // dims lane + 32 i
                for (int page_idx = first_page + warp; page_idx <= last_page; page_idx += DP_WARPS) {
                    __nv_bfloat16* kpage = op.kv + ((long long)pages[page_idx] * 2 * op.n_kv_heads + kvh) * head_stride;
                    __nv_bfloat16* vpage = kpage + (long long)op.n_kv_heads * head_stride;
                    const int base = page_idx * DP_PAGE;
                    const int lo = max(first - base, 0), hi = min(pos + 1 - base, DP_PAGE);
                    const bool has_new = (op.k_new != nullptr) && page_idx == last_page;
                    const int hi_cache = has_new ? hi - 1 : hi;
                    const __nv_bfloat16* kn = has_new ? op.k_new + (long long)tk * op.ldk + kvh * op.head_dim : nullptr;
                    const __nv_bfloat16* vn = has_new ? op.v_new + (long long)tk * op.ldv + kvh * op.head_dim : nullptr;
                    if (has_new && h % group == 0) {
                        __nv_bfloat16* kd = kpage + (long long)(hi - 1) * op.head_dim;
                        for (int d = lane; d < op.head_dim; d += 32) {
                            kd[d] = kn[d];
                            vpage[(long long)d * DP_PAGE + hi - 1] = vn[d];      // values lie dimension-major
                        }
                    }
                    float s0 = -INFINITY, s1 = -INFINITY;
                    {
                        const int j0 = lane, j1 = lane + 32;
                        const bool in0 = j0 >= lo && j0 < hi_cache, in1 = j1 >= lo && j1 < hi_cache;
                        const bool new0 = has_new && j0 == hi - 1, new1 = has_new && j1 == hi - 1;
                        const __nv_bfloat16* safe = (hi_cache > lo) ? kpage + (long long)lo * op.head_dim : kn;
                        const __nv_bfloat16* k0 = in0 ? kpage + (long long)j0 * op.head_dim : (new0 ? kn : safe);
                        const __nv_bfloat16* k1 = in1 ? kpage + (long long)j1 * op.head_dim : (new1 ? kn : safe);
                        float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll 8
                        for (int d = 0; d < op.head_dim; d += 8) {
                            const uint4 ra = *reinterpret_cast<const uint4*>(k0 + d);
                            const uint4 rb = *reinterpret_cast<const uint4*>(k1 + d);
                            const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
                            const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
                                a0 = fmaf(att_q[d + 2 * i], fa.x, a0); a1 = fmaf(att_q[d + 2 * i + 1], fa.y, a1);
                                b0 = fmaf(att_q[d + 2 * i], fb.x, b0); b1 = fmaf(att_q[d + 2 * i + 1], fb.y, b1);
                            }
                        }
                        if (in0 || new0) s0 = (a0 + a1) * op.scale;
                        if (in1 || new1) s1 = (b0 + b1) * op.scale;
                    }
                    const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
                    const float p0 = (s0 == -INFINITY) ? 0.0f : expf(s0 - m_new);
                    const float p1 = (s1 == -INFINITY) ? 0.0f : expf(s1 - m_new);
                    const float corr = expf(m_run - m_new);
                    l_run = l_run * corr + warp_sum(p0 + p1);
                    m_run = m_new;
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[i] *= corr;
                    // the new key's weight goes with v_new; in the runs over the cache it counts as zero
                    const float w_new = has_new ? __shfl_sync(0xffffffffu, (hi - 1 < 32) ? p0 : p1, (hi - 1) & 31) : 0.0f;
                    float r0 = p0, r1 = p1;
                    if (has_new && ((hi - 1) & 31) == lane) { if (hi - 1 < 32) r0 = 0.0f; else r1 = 0.0f; }
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (32 * half >= hi_cache || 32 * half + 32 <= lo) continue;      // no visible key in this run
                        const float pr = half ? r1 : r0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (32 * i >= op.head_dim) continue;                          // uniform over the warp
                            const int d = min(lane + 32 * i, op.head_dim - 1);          // idle lanes read a row that exists
                            const uint4* src = reinterpret_cast<const uint4*>(vpage + (long long)d * DP_PAGE + 32 * half);
                            uint4 raw[4];
#pragma unroll
                            for (int c = 0; c < 4; ++c) raw[c] = src[c];
                            const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(raw);
                            float a = acc[i];
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj)
                                a = fmaf(__shfl_sync(0xffffffffu, pr, jj), __bfloat162float(v[jj]), a);
                            acc[i] = a;
                        }
                    }
                    if (has_new) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int d = lane + 32 * i;
                            if (d < op.head_dim) acc[i] = fmaf(w_new, __bfloat162float(vn[d]), acc[i]);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int d = lane + 32 * i;
                    if (d < op.head_dim) att_o[warp][d] = acc[i];
                }
                if (lane == 0) { att_m[warp] = m_run; att_l[warp] = l_run; }
                __syncthreads();
                float big = -INFINITY;
#pragma unroll
                for (int w = 0; w < DP_WARPS; ++w) big = fmaxf(big, att_m[w]);
                if (threadIdx.x < DP_WARPS)
                    att_w[threadIdx.x] = att_m[threadIdx.x] == -INFINITY ? 0.0f : expf(att_m[threadIdx.x] - big);
                __syncthreads();
                if (threadIdx.x < op.head_dim) {
                    float total = 0.0f;
#pragma unroll
                    for (int w = 0; w < DP_WARPS; ++w) total = fmaf(att_l[w], att_w[w], total);
                    float o = 0.0f;
#pragma unroll
                    for (int w = 0; w < DP_WARPS; ++w) o = fmaf(att_o[w][threadIdx.x], att_w[w], o);
                    op.out[(long long)tk * op.ldo + h * op.head_dim + threadIdx.x] = __float2bfloat16_rn(o / total);
                }
                __syncthreads();
            }
        }
        if (trace && blockIdx.x == 0 && threadIdx.x == 0) {       // ... and when it had done its share of it
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            trace[2 * oi + 1] = now;
        }
        if (oi + 1 < n_ops) {
            // the first weights of this block's next tile set off before the barrier: they depend on nothing
            const ProgramOp next = ops[oi + 1];
            if (next.type == OP_GEMM && (int)blockIdx.x < ((next.N + 15) / 16) * next.ksplit) {
                const GemmUnit u = gemm_unit(next, blockIdx.x, warp, lane);
                gemm_load(next, u, u.kb0, lane, wa, wb);
                preloaded = true;
            }
            if (!grid_barrier(bar, status)) return;
        }
    }
}

}  // namespace mu

// ops: n_ops ProgramOp records in device memory; barrier: 8 zeroed bytes that stay with the program;
// status: a device word that stays 0 unless a barrier wait ran out (code 10).  max_rows: the largest
// M of the program (<= 16); dyn_smem: bytes for the normed activations, 16 * (largest normed K + 8) * 2.
// trace: optional 2 * n_ops 64-bit words; block 0 notes the time (ns) at which it began and ended its
// share of each operation.
MU_EXPORT int mu_decode_program(const void* ops, int n_ops, int max_rows, int dyn_smem, void* barrier,
                                int* status, unsigned long long* trace, void* stream) {
    if (n_ops <= 0) return MU_OK;
    if (!ops || !barrier || !status || max_rows < 1 || max_rows > mu::DP_MAX_ROWS) return MU_ERR_BAD_ARGUMENT;
    if (dyn_smem < 0 || dyn_smem > 160 * 1024) return MU_ERR_UNSUPPORTED_SIZE;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        return MU_ERR_LAUNCH;
    auto run = [&](auto kernel) -> int {
        static bool raised = false;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
                return MU_ERR_LAUNCH;
            raised = true;
        }
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, mu::DP_THREADS, dyn_smem) != cudaSuccess ||
            per_sm < 1)
            return MU_ERR_UNSUPPORTED_SIZE;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms);                     // one block per SM, all resident at once
        cfg.blockDim = dim3(mu::DP_THREADS);
        cfg.dynamicSmemBytes = dyn_smem;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, kernel, (const mu::ProgramOp*)ops, n_ops, (mu::BarrierState*)barrier,
                                  status, trace) == cudaSuccess ? MU_OK : MU_ERR_LAUNCH;
    };
    if (max_rows <= 8) return run(mu::decode_program_kernel<1>);
    return run(mu::decode_program_kernel<2>);
}

// Size of one ProgramOp record, so that the host can check its own layout against this one.
MU_EXPORT int mu_decode_program_op_size() { return (int)sizeof(mu::ProgramOp); }
