// One layer of a prompt step from one call into the library.
//
// A pre-norm layer of LayerNorm, causal attention over the paged cache and a two-matrix feed-forward is, for a
// prompt of some hundred tokens, seven launches of a few microseconds each; issued one by one from Python the
// host needs longer for them than the device.  mu_prompt_layer takes everything the layer needs in one
// structure and issues the launches itself, through the same entry points the single calls use (so the
// kernels, their checks and their choices are the same ones):
//     normed = LayerNorm(x);  qkv = normed . Wqkv^T + b            mu_layernorm_gemm_tc
//     append this step's keys and values; attention over the cache mu_attention_prefill_tc
//     x += attn . Wout^T + b                                        mu_gemm_tc (added in place)
//     normed = LayerNorm(x);  hidden = act(normed . Wup^T + b)      mu_layernorm_gemm_tc
//     x += hidden . Wdown^T + b                                     mu_gemm_tc (added in place)
// (include/ai/LocalModel.hpp:3705-3782 for the order.)  bfloat16 weights, head size 64, pages of 64, no
// rotation of queries and keys: what the Python side checks before it takes this path.
#include "common.cuh"

extern "C" int mu_layernorm_gemm_tc(const float* x, const int* rows, const float* gamma, const float* beta, float eps,
                                    void* normed, const void* W, const float* bias, const float* residual, void* C,
                                    int M, int N, int K, long long ldw, long long ldc, long long ldr, int act,
                                    int out_bf16, int* status, void* stream);
extern "C" int mu_gemm_tc(const void* A, const void* W, const float* bias, const float* residual, void* C, int M, int N,
                          int K, long long lda, long long ldw, long long ldc, long long ldr, int act, int out_bf16,
                          int tile, int want_splits, int* status, void* stream);
extern "C" int mu_attention_prefill_tc(const void* q, long long ldq, int n_tokens, void* out, long long ldo, void* kv,
                                       long long n_cache_pages, const int* block_table, int max_pages, int page_tokens,
                                       const int* tok_pos, const int* tok_seq, const int* tiles, int n_tiles, int n_heads,
                                       int n_kv_heads, int head_dim, float scale, int window, const void* k_new,
                                       long long ldk, const void* v_new, long long ldv, const int* append_tiles,
                                       int n_append_tiles, int* status, void* stream);

// The Python side mirrors this layout field by field (ops.PromptLayerArgs).
struct MuPromptLayerArgs {
    // the step
    float* x;                       // residual stream [n_tokens, hidden], float32, updated in place
    void* normed;                   // scratch [n_tokens, hidden] bfloat16
    void* qkv;                      // scratch [n_tokens, q_width + 2 kv_width] bfloat16
    void* attn;                     // scratch [n_tokens, q_width] bfloat16
    void* inner_buf;                // scratch [n_tokens, inner] bfloat16
    const int* tok_pos;
    const int* tok_seq;
    const int* block_table;
    const int* tiles_wide;          // query tiles of up to 128 tokens, longest first
    const int* tiles;               // tiles of up to 64 tokens (the cache append)
    int* status;
    void* stream;
    // the layer
    void* kv_pages;
    const float* ln1_gamma; const float* ln1_beta;
    const void* qkv_weight; const float* qkv_bias;
    const void* out_weight; const float* out_bias;
    const float* ln2_gamma; const float* ln2_beta;
    const void* up_weight; const float* up_bias;
    const void* down_weight; const float* down_bias;
    long long n_cache_pages, ld_qkv_weight, ld_out_weight, ld_up_weight, ld_down_weight;
    float eps1, eps2, scale;
    int n_tokens, hidden, inner, n_heads, n_kv_heads, head_dim, window, act;
    int max_pages, page_tokens, n_tiles_wide, n_tiles, owns_cache;
};

MU_EXPORT int mu_prompt_layer_args_size() { return (int)sizeof(MuPromptLayerArgs); }

// Returns 0, or 100 * (the failing launch, 1-5) + its error code.
MU_EXPORT int mu_prompt_layer(const MuPromptLayerArgs* a) {
    if (!a || a->n_tokens <= 0) return MU_ERR_BAD_ARGUMENT;
    const int T = a->n_tokens, D = a->hidden;
    const int qw = a->n_heads * a->head_dim, kw = a->n_kv_heads * a->head_dim;
    const int width = qw + 2 * kw;
    __nv_bfloat16* qkv = (__nv_bfloat16*)a->qkv;
    if (int e = mu_layernorm_gemm_tc(a->x, nullptr, a->ln1_gamma, a->ln1_beta, a->eps1, a->normed, a->qkv_weight,
                                     a->qkv_bias, nullptr, qkv, T, width, D, a->ld_qkv_weight, width, 0, 0, 1, a->status,
                                     a->stream))
        return 100 + e;
    const void* k_new = a->owns_cache ? (const void*)(qkv + qw) : nullptr;
    const void* v_new = a->owns_cache ? (const void*)(qkv + qw + kw) : nullptr;
    if (int e = mu_attention_prefill_tc(qkv, width, T, a->attn, qw, a->kv_pages, a->n_cache_pages, a->block_table,
                                        a->max_pages, a->page_tokens, a->tok_pos, a->tok_seq, a->tiles_wide,
                                        a->n_tiles_wide, a->n_heads, a->n_kv_heads, a->head_dim, a->scale, a->window,
                                        k_new, width, v_new, width, a->tiles, a->n_tiles, a->status, a->stream))
        return 200 + e;
    if (int e = mu_gemm_tc(a->attn, a->out_weight, a->out_bias, a->x, a->x, T, D, qw, qw, a->ld_out_weight, D, D, 0, 0, 0,
                           -1, a->status, a->stream))
        return 300 + e;
    if (int e = mu_layernorm_gemm_tc(a->x, nullptr, a->ln2_gamma, a->ln2_beta, a->eps2, a->normed, a->up_weight,
                                     a->up_bias, nullptr, a->inner_buf, T, a->inner, D, a->ld_up_weight, a->inner, 0,
                                     a->act, 1, a->status, a->stream))
        return 400 + e;
    if (int e = mu_gemm_tc(a->inner_buf, a->down_weight, a->down_bias, a->x, a->x, T, D, a->inner, a->inner,
                           a->ld_down_weight, D, D, 0, 0, 0, -1, a->status, a->stream))
        return 500 + e;
    return MU_OK;
}
