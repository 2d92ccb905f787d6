// Host side of the tensor-core product (the kernel: gemm_tc_kernel.cuh): tensor maps, the choice of the
// tile width and of a cut along K, and the library's entry points.  The kernels of cut products are
// compiled in gemm_tc_split.cu.
#include "gemm_tc_kernel.cuh"

#include <mutex>

namespace mu {

SplitWorkspace g_split;

// the variants for products cut along K (gemm_tc_split.cu); bn: 64, 128 or 256
int launch_tc_split(int bn, const void* A, const void* W, const float* bias, const float* residual, void* C, int M,
                    int N, int K, long long lda, long long ldw, long long ldc, long long ldr, int act, int out_bf16,
                    int* status, int splits, cudaStream_t s);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// Descriptors are pure functions of (address, shape, stride, box): the last few hundred are kept, since a
// model asks for the same ones step after step (weights always, activations whenever the allocator hands
// the same buffer back).
struct MapKey {
    const void* base; long long rows; int cols, box_rows; long long ld; int kind;      // kind 0: operand tiles
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && ld == o.ld && kind == o.kind;
    }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
static MapSlot map_cache[512];
static std::mutex map_mutex;

static bool make_map_uncached(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows);

bool tensor_map_bf16(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    const MapKey key = {base, rows, cols, box_rows, ld, 0};
    const size_t h = ((uintptr_t)base >> 8) * 0x9E3779B97F4A7C15ull + (size_t)rows * 31 + (size_t)cols * 131 + box_rows;
    MapSlot& slot = map_cache[(h >> 20) & 511];
    std::lock_guard<std::mutex> lock(map_mutex);
    if (slot.used && slot.key == key) { *map = slot.map; return true; }
    if (!make_map_uncached(map, base, rows, cols, ld, box_rows)) return false;
    slot.key = key; slot.map = *map; slot.used = true;
    return true;
}

// An output matrix [rows, cols] of bfloat16 or float32 with `ld` elements between rows, cut into boxes of
// 32 x 32 that lie row after row in shared memory (no swizzle): what the epilogue's bulk stores write.
bool tensor_map_out(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int is_bf16) {
    const MapKey key = {base, rows, cols, 32, ld, is_bf16 ? 1 : 2};
    const size_t h = ((uintptr_t)base >> 8) * 0x9E3779B97F4A7C15ull + (size_t)rows * 37 + (size_t)cols * 113 + key.kind;
    MapSlot& slot = map_cache[(h >> 20) & 511];
    std::lock_guard<std::mutex> lock(map_mutex);
    if (slot.used && slot.key == key) { *map = slot.map; return true; }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const size_t elem_bytes = is_bf16 ? 2 : 4;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims,
           strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    slot.key = key; slot.map = *map; slot.used = true;
    return true;
}

// A [rows, cols] bfloat16 matrix with `ld` elements between rows, cut into boxes of box_rows x 64.
static bool make_map_uncached(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace mu

// Gives the product kernel room for products that are cut along K (few tiles of C, long K): `parts` takes
// the partial tiles (float32, 16-byte aligned), `tickets` n_tickets counters that are zero now and are left
// zero by every launch.  Without it, or where it is too small, such products run uncut.
MU_EXPORT int mu_gemm_tc_split_workspace(void* parts, long long parts_bytes, int* tickets, int n_tickets) {
    if (((uintptr_t)parts & 15) || parts_bytes < 0 || n_tickets < 0) return MU_ERR_BAD_ARGUMENT;
    mu::g_split.parts = (float*)parts;
    mu::g_split.parts_bytes = parts ? parts_bytes : 0;
    mu::g_split.tickets = tickets;
    mu::g_split.n_tickets = tickets ? n_tickets : 0;
    return MU_OK;
}

// bfloat16 A [M, K] (lda) and W [N, K] (ldw): K, lda, ldw multiples of 8, bases 16-byte aligned.
// C bfloat16 or float32 (ldc); residual float32 (ldr), may be C itself.  `status` is a device word
// that stays 0 unless a wait inside the kernel ran out (1 producer, 2 tensor-core issuer, 3 epilogue).
// tile: width of the tiles of C (64, 128 or 256; 0: chosen here).  splits: parts that K is cut into
// (-1: chosen here; 0 or 1: never cut; n: n parts wherever K allows).
MU_EXPORT int mu_gemm_tc(const void* A, const void* W, const float* bias, const float* residual, void* C,
                         int M, int N, int K, long long lda, long long ldw, long long ldc, long long ldr,
                         int act, int out_bf16, int tile, int want_splits, int* status, void* stream) {
    if (M <= 0 || N <= 0) return MU_OK;
    if (K <= 0 || !A || !W || !C || !status) return MU_ERR_BAD_ARGUMENT;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return MU_ERR_ALIGNMENT;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return MU_ERR_ALIGNMENT;
    if (lda < K || ldw < K || ldc < N || (residual && ldr < N)) return MU_ERR_BAD_ARGUMENT;
    if ((M + mu::TC_BM - 1) / mu::TC_BM > 65535) return MU_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    // Tile width: wider tiles do more products per byte loaded, but the tiles must also fill whole
    // rounds of the SMs; take the width with the best (fill of the last round) x (worth of the width).
    const int sms = mu::sm_count();
    if (sms <= 0) return MU_ERR_LAUNCH;
    if (tile != 0 && tile != 64 && tile != 128 && tile != 256) return MU_ERR_BAD_ARGUMENT;
    const long long m_tiles = (M + mu::TC_BM - 1) / mu::TC_BM;
    int best_bn = 64;
    double best = -1.0;
    const int widths[3] = {64, 128, 256};
    const double worth[3] = {0.6, 0.85, 1.0};
    for (int i = 0; i < 3; ++i) {
        if (widths[i] > 64 && N <= widths[i] / 2) continue;
        const long long tiles = m_tiles * ((N + widths[i] - 1) / widths[i]);
        const long long rounds = (tiles + sms - 1) / sms;
        const double score = (double)tiles / (double)(rounds * sms) * worth[i];
        if (score > best) { best = score; best_bn = widths[i]; }
    }
#define MU_TC(BN, ST, KS)                                                                                       \
    (out_bf16 ? mu::launch_tc<BN, ST, KS, __nv_bfloat16, false>(A, W, bias, residual, (__nv_bfloat16*)C, M, N, K, \
                                                                lda, ldw, ldc, ldr, act, status, 1, s)           \
              : mu::launch_tc<BN, ST, KS, float, false>(A, W, bias, residual, (float*)C, M, N, K, lda, ldw, ldc,   \
                                                        ldr, act, status, 1, s))
    if (tile) best_bn = tile;
    // Few tiles and a long K can be cut along K so that (tiles x parts) fill the SMs.  Handing the parts over
    // (stores, a fence, a ticket, the sum) costs some microseconds, as much as a dozen 64-deep stages of
    // products, so the rule here cuts a K of 2,048 or more into parts of six stages or more.
    int splits = 1;
    {
        const long long tiles = m_tiles * ((N + best_bn - 1) / best_bn);
        const int kb64 = (K + 63) / 64;
        if (want_splits >= 0) {
            splits = want_splits <= 1 ? 1 : (want_splits < kb64 ? want_splits : kb64);
        } else if (tiles * 2 <= sms && kb64 >= 32) {
            long long want = sms / tiles;
            if (want > kb64 / 6) want = kb64 / 6;
            if (want > 8) want = 8;
            splits = (int)want;
        }
        // the workspace must hold a partial tile per (tile, part) and a ticket per tile
        if (!mu::g_split.parts || tiles > mu::g_split.n_tickets ||
            tiles * splits * (long long)(mu::TC_BM * best_bn * sizeof(float)) > mu::g_split.parts_bytes)
            splits = 1;
    }
    if (splits > 1)
        return mu::launch_tc_split(best_bn, A, W, bias, residual, C, M, N, K, lda, ldw, ldc, ldr, act, out_bf16, status,
                                   splits, s);
    // narrow tiles: 128-deep stages (issuing, not multiplying, sets their pace); K of a single 64 keeps 64
    if (best_bn == 64) return K > 64 ? MU_TC(64, 4, 2) : MU_TC(64, 6, 1);
    if (best_bn == 128) return K > 64 ? MU_TC(128, 3, 2) : MU_TC(128, 5, 1);
    return MU_TC(256, 4, 1);
#undef MU_TC
}

extern "C" int mu_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* y,
                            int n_rows, int hidden, float eps, int out_bf16, void* stream);

// LayerNorm of float32 rows of x (contiguous, K wide; optionally the rows that `rows` picks) into the
// bfloat16 buffer `normed` [M, K], then the product of it: two launches from one call, for the prompt
// step, whose host side would otherwise spend as long on the two calls as the device on the kernels.
MU_EXPORT int mu_layernorm_gemm_tc(const float* x, const int* rows, const float* gamma, const float* beta,
                                   float eps, void* normed, const void* W, const float* bias,
                                   const float* residual, void* C, int M, int N, int K, long long ldw,
                                   long long ldc, long long ldr, int act, int out_bf16, int* status,
                                   void* stream) {
    if (!normed) return MU_ERR_BAD_ARGUMENT;
    if (int e = mu_layernorm(x, rows, gamma, beta, normed, M, K, eps, 1, stream)) return e;
    return mu_gemm_tc(normed, W, bias, residual, C, M, N, K, K, ldw, ldc, ldr, act, out_bf16, 0, -1, status, stream);
}
