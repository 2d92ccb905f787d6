/* mu_attention_static_scratch: split-key attention for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference project; it exists for
 * users of this library only.
 *
 * Who needs it: code that runs where device memory may not be allocated or
 * freed -- a plug-in loaded into a host application that owns the memory pool,
 * a real-time loop that must not enter the allocator, a process that runs
 * under a fixed memory budget handed out at start-up.  Single-token attention
 * splits each head's keys over several warps and has to park the partial
 * results somewhere until they are merged.  The ordinary entry point,
 * mu_attention, takes that scratch from the caller (part_o, part_ml); a caller
 * of the kind above has nowhere to get it from.  This variant keeps the
 * scratch inside the library instead: a fixed array in device memory that comes
 * with the loaded library (MU_STATIC_SCRATCH_FLOATS floats = 4 MiB on every GPU
 * that uses the library, held until the process exits).  It calls no
 * cudaMalloc, cudaFree or any other allocating routine.  Inputs and outputs
 * are still the caller's.
 *
 * Arguments are those of mu_attention without part_o and part_ml.  Split s of
 * n_splits takes the keys [s * split_keys, (s + 1) * split_keys) of every
 * sequence, and the last split goes on to the query's own position, so a
 * split_keys that falls short of a long sequence loses no key (it only makes
 * the last split longer).  At most 65535 heads and 65535 splits.
 *
 * Limit: n_tokens * n_heads * n_splits * (head_dim + 2) must not exceed
 * MU_STATIC_SCRATCH_FLOATS; a larger request returns MU_ERR_STATIC_SCRATCH (6)
 * and launches nothing.  n_splits == 1 needs no scratch and is accepted too.
 *
 * First call on a device: looks up the array's device address (once per
 * device, with that device current) and keeps it; if that lookup fails the
 * call returns MU_ERR_SETUP (5).  Make this first call before any stream
 * capture begins.
 *
 * Sharing: every call on a device uses the same array, and the array keeps
 * whatever the last call left in it.  Nothing in it needs to start at zero:
 * each call writes every partial result it later reads.  Two calls that may
 * run on the GPU at the same time (different streams, different threads)
 * race on the array; order them, for instance by issuing them into one stream.
 *
 * Returns 0 or an MU_ERR_* code of common.cuh, as mu_attention does.
 */
#pragma once

#define MU_STATIC_SCRATCH_FLOATS (1 << 20)
#define MU_ERR_SETUP 5
#define MU_ERR_STATIC_SCRATCH 6

#ifdef __cplusplus
extern "C"
#endif
int mu_attention_static_scratch(const void* q, long long ldq, void* out, long long ldo, const void* kv,
                                const int* block_table, int max_pages, int page_tokens,
                                const int* tok_pos, const int* tok_seq, int n_tokens, int n_heads,
                                int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                int split_keys, int is_bf16, void* stream);
