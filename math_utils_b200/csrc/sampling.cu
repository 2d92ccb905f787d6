// Sampling on the device: greedy, and temperature with an optional top-k.
//
// The rule is the reference's sampleTopK (include/ai/LocalModel.hpp:3809-3841):
// greedy when temperature <= 0 or top_k == 1 (first maximum wins); otherwise
// keep the top_k largest logits (0 keeps all), p_i = exp(l_i / T - best / T),
// pick = u * sum p, and walk the kept tokens in descending order of logit
// (ties: lower index first) until the running sum passes pick.
//
// No sort is needed for that walk.  Logits map to 32-bit keys that order like
// the floats; an 8-bit radix descent over the keys (4 passes) finds the k-th
// largest key, and a second descent, over histograms of probability mass
// instead of counts, finds the key at which the running mass passes pick.
// Masses are summed as 64-bit fixed point (2^-40 units) with integer atomics,
// so the sums do not depend on the order threads arrive in and a (seed,
// request, draw index) always gives the same token.
//
// How the passes over a row are kept short (sample_kernel):
//   * eight logits are asked for before any is used (for_each_logit);
//   * the first pass of a descent, whose bins are the keys' sign and exponent,
//     adds into a histogram per warp, in 32-bit words (zero_private / fold_private);
//   * the total mass is the sum of the first mass histogram, not a pass of its own;
//   * a top_k of up to SAMPLE_CANDIDATES: the kept tokens are gathered into shared
//     memory once the threshold is known, and the second descent and the pick walk
//     that list;
//   * up to eight blocks (a thread-block cluster, fewer as the rows grow) share a
//     row's passes: each counts its share, every block adds the shares up through
//     distributed shared memory in rank order and selects the same bin.
//
// u comes from a counter-based stream per request: key = splitmix64(seed ^
// request * 0x9E3779B97F4A7C15), x = splitmix64(key + n * 0xD1B54A32D192ED03),
// u = (x >> 11) * 2^-53 (splitmix64 and the 53-bit mantissa rule as in
// include/math/Random.hpp:27,79-84), n = how many tokens the request has drawn.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace mu {

constexpr int SAMPLE_THREADS = 1024;
constexpr double FIXED_ONE = 1099511627776.0;  // 2^40

__device__ __forceinline__ unsigned int float_key(float v) {
    const unsigned int b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__host__ __device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    unsigned long long z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ double uniform_draw(unsigned long long seed, unsigned long long request,
                                               unsigned long long n) {
    const unsigned long long key = splitmix64(seed ^ (request * 0x9E3779B97F4A7C15ull));
    const unsigned long long x = splitmix64(key + n * 0xD1B54A32D192ED03ull);
    return (double)(x >> 11) * (1.0 / 9007199254740992.0);
}

// The kernels' status word handed on with the tokens: row 0's writer copies it to status_out (the word behind
// the tokens of a recorded step, which one copy then brings to the host).  Every kernel before this one has
// finished with the word by then.
struct StatusCopy {
    const int* status;          // null: nothing to copy
    int* status_out;
    __device__ __forceinline__ void write(int r) const {
        if (status && r == 0) *status_out = *reinterpret_cast<const volatile int*>(status);
    }
};

// The vocabulary of a row is cut over ARGMAX_PARTS blocks.  Each folds (key, ~index) pairs into one
// 64-bit maximum in global memory; the block that takes the row's last ticket writes the token and
// puts the workspace back to zero for the next launch.
constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_PARTS = 16;

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out,
              unsigned long long* __restrict__ best_ws, unsigned int* __restrict__ ticket_ws,
              int* __restrict__ feed_ids, int* __restrict__ feed_pos, int last_pos, StatusCopy status_copy) {
    __shared__ unsigned long long best_smem[ARGMAX_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (long long)r * ld;
    const int per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const int begin = blockIdx.y * per, end = min(vocab, begin + per);
    unsigned long long best = 0;
    constexpr int BATCH = 8;                    // loads of a batch are issued before any is compared
    for (int i0 = begin + threadIdx.x; i0 < end; i0 += BATCH * ARGMAX_THREADS) {
        float vals[BATCH];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int i = i0 + b * ARGMAX_THREADS;
            vals[b] = i < end ? row[i] : -INFINITY;
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int i = i0 + b * ARGMAX_THREADS;
            if (i < end) {
                // larger logit wins; among equals the lower index (larger ~index) wins
                const unsigned long long cand =
                    ((unsigned long long)float_key(vals[b]) << 32) | (unsigned int)(0xFFFFFFFFu - (unsigned)i);
                best = cand > best ? cand : best;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) best_smem[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ARGMAX_THREADS / 32; ++w) best = best_smem[w] > best ? best_smem[w] : best;
        atomicMax(&best_ws[r], best);
        __threadfence();
        const unsigned int ticket = atomicAdd(&ticket_ws[r], 1u);
        if (ticket == ARGMAX_PARTS - 1) {
            __threadfence();
            const unsigned long long all = atomicExch(&best_ws[r], 0ull);
            ticket_ws[r] = 0;
            const int token = (int)(0xFFFFFFFFu - (unsigned int)(all & 0xFFFFFFFFull));
            out[r] = token;
            if (feed_ids) feed_ids[r] = token;  // hand the token to the next single-token step
            if (feed_pos) {
                const int p = feed_pos[r] + 1;
                feed_pos[r] = p < last_pos ? p : last_pos;
            }
            status_copy.write(r);
        }
    }
}

// Among 256 bins taken from the highest down, finds the first whose running
// total exceeds `target`.  Called by warp 0; returns through shared memory
// (sel[0] = bin, sel[1] = total of the bins above it).
__device__ __forceinline__ void select_bin(const unsigned long long* hist, unsigned long long target,
                                           unsigned long long* sel) {
    const int lane = threadIdx.x & 31;
    unsigned long long local = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) local += hist[255 - (lane * 8 + i)];
    unsigned long long incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const unsigned long long before = incl - local;
    if (before <= target && target < incl) {
        unsigned long long run = before;
        for (int i = 0; i < 8; ++i) {
            const int bin = 255 - (lane * 8 + i);
            const unsigned long long h = hist[bin];
            if (target < run + h) {
                sel[0] = (unsigned long long)bin;
                sel[1] = run;
                break;
            }
            run += h;
        }
    }
}

// The first byte of the keys (sign and exponent) takes a handful of values whatever the logits are, so in the
// first pass of a descent every token would queue on a few shared-memory words.  There the warps add into
// `groups` histograms (one a warp), in 32-bit words
// that native shared-memory atomics serve: a count, or a mass (at most 2^40) cut into two limbs of 20 bits.  A
// group sees at most vocab / groups + 32 tokens, so a limb's sum stays below 2^32 up to 4,000 tokens a group
// (a vocabulary of 128,000 with a group a warp); beyond that the block's one histogram is used as in the
// later passes.  fold_private() adds the groups' histograms up into the block's 64-bit one.
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;
constexpr int SAMPLE_CANDIDATES = 1024;
constexpr int LIMBS = 2, LIMB_BITS = 20;
constexpr size_t sample_private_bytes(int groups) { return (size_t)groups * 256 * LIMBS * sizeof(unsigned int); }

__device__ __forceinline__ void zero_private(unsigned int* priv, int groups) {
    for (int i = threadIdx.x; i < groups * 256 * LIMBS; i += SAMPLE_THREADS) priv[i] = 0u;
}
__device__ __forceinline__ void fold_private(const unsigned int* priv, int groups, unsigned long long* hist) {
    if (threadIdx.x < 256) {
        unsigned long long limb[LIMBS] = {0, 0};
        for (int g = 0; g < groups; ++g)
#pragma unroll
            for (int k = 0; k < LIMBS; ++k) limb[k] += priv[(g * 256 + threadIdx.x) * LIMBS + k];
        hist[threadIdx.x] = limb[0] + (limb[1] << LIMB_BITS);
    }
}

// f(i, logit) for every token i of this thread, in rising order: the tokens tid + SAMPLE_THREADS * (part + parts * k),
// k = 0, 1, ... (`parts` blocks share a row, block `part` takes every parts-th run of SAMPLE_THREADS tokens).
// Eight logits are asked for before any is used: a pass over the row is a chain of trips to the L2 otherwise.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* row, int vocab, F f, int part = 0, int parts = 1) {
    constexpr int U = 8;
    const int step = parts * SAMPLE_THREADS;
    for (int i0 = part * SAMPLE_THREADS + threadIdx.x; i0 < vocab; i0 += step * U) {
        float l[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            l[u] = i < vocab ? row[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            if (i < vocab) f(i, l[u]);
        }
    }
}

struct RowView {
    const float* row;
    int vocab;
    float temperature, best;       // best = max logit / temperature
    unsigned int thr_key;          // kept: key > thr_key, or key == thr_key and index <= idx_cut
    int idx_cut;
    __device__ __forceinline__ bool kept(unsigned int key, int i) const {
        return key > thr_key || (key == thr_key && i <= idx_cut);
    }
    __device__ __forceinline__ unsigned long long mass(float logit) const {
        // (a float times 2^40 is exact, and so is the float's way to the integer: the same number as through double)
        return __float2ull_rz(expf(logit / temperature - best) * (float)FIXED_ONE);
    }
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int vocab, float temperature, int top_k,
              unsigned long long seed, const long long* __restrict__ request_ids,
              int* __restrict__ draw_index, int* __restrict__ out, int* __restrict__ feed_ids,
              int* __restrict__ feed_pos, int last_pos, StatusCopy status_copy, int staged, int groups, int parts) {
    // `parts` > 1: that many blocks (a thread-block cluster along grid.y) share a row for the passes over the
    // whole row: each counts its share into a histogram of its own, every block adds the shares up through
    // distributed shared memory (the same sums in the same order: every block selects the same bin), and the
    // kept tokens of a gathered top_k (see below) are collected in block 0, which then finishes alone.
    __shared__ unsigned long long hist[256];
    __shared__ float max_share;
    __shared__ unsigned long long hist_share[2][256];    // this block's share; two, used in turn, so that a block
                                                         // may start its next pass while others still read this one
    // dynamic shared memory: with `staged` the row's logits (every pass reads them there instead of going to the
    // L2 a dozen times), then the groups' histograms of the first pass of a descent (see above)
    extern __shared__ __align__(16) unsigned char sample_dyn[];
    float* row_smem = reinterpret_cast<float*>(sample_dyn);
    unsigned int* priv = reinterpret_cast<unsigned int*>(sample_dyn + (staged ? ((size_t)vocab * 4 + 15) / 16 * 16 : 0));
    const bool private_ok = vocab / groups + 32 < (1 << (32 - LIMB_BITS));   // else a limb could overflow
    __shared__ unsigned long long sel[2];
    __shared__ float red[32];
    __shared__ unsigned long long total_smem;
    __shared__ int found_idx;
    // With a top_k of at most SAMPLE_CANDIDATES the kept tokens are gathered here once the threshold is known,
    // and everything after that (the largest logit, the masses, the second descent, the pick) walks this list
    // instead of the row.
    __shared__ float cand_logit[SAMPLE_CANDIDATES];
    __shared__ int cand_idx[SAMPLE_CANDIDATES];
    __shared__ int n_cand;
    const bool gather = top_k > 0 && top_k < vocab && top_k <= SAMPLE_CANDIDATES;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, r = blockIdx.x;
    const int part = parts > 1 ? (int)blockIdx.y : 0;
    cg::cluster_group cluster = cg::this_cluster();
    if (tid == 0) n_cand = 0;                          // (block 0's is the one the cluster fills)
    RowView v;
    v.row = logits + (long long)r * ld;
    v.vocab = vocab;
    v.temperature = temperature;
    v.thr_key = 0;
    v.idx_cut = vocab;
    if (staged) {
        for_each_logit(v.row, vocab, [&](int i, float l) { row_smem[i] = l; });
        __syncthreads();
        v.row = row_smem;
    }

    // maximum logit (of the row; with a gathered top_k it is the largest of the list, found below)
    auto block_max = [&](float mx) {
        mx = warp_max(mx);
        __syncthreads();                               // (red may still be read from an earlier call)
        if ((tid & 31) == 0) red[tid >> 5] = mx;
        __syncthreads();
        mx = red[0];
        for (int w = 1; w < SAMPLE_WARPS; ++w) mx = fmaxf(mx, red[w]);
        return mx;
    };
    if (!gather) {
        float mx = -INFINITY;
        for_each_logit(v.row, vocab, [&](int, float l) { mx = fmaxf(mx, l); }, part, parts);
        mx = block_max(mx);
        if (parts > 1) {
            if (tid == 0) max_share = mx;
            cluster.sync();
            for (int c = 0; c < parts; ++c) mx = fmaxf(mx, *cluster.map_shared_rank(&max_share, c));
        }
        v.best = mx / temperature;
    }

    // the k-th largest key, when top_k cuts anything
    if (top_k > 0 && top_k < vocab) {
        unsigned int prefix = 0, mask = 0;
        unsigned long long need = (unsigned long long)top_k - 1;   // first bin whose running count exceeds this
        for (int shift = 24; shift >= 0; shift -= 8) {
            unsigned long long* share = parts > 1 ? hist_share[(shift >> 3) & 1] : hist;
            if (tid < 256) share[tid] = 0;
            __syncthreads();
            if (shift == 24 && private_ok) {
                // every token takes part and the bins are few: a histogram per warp
                zero_private(priv, groups);
                __syncthreads();
                unsigned int* mine = priv + (size_t)((tid >> 5) * groups / SAMPLE_WARPS) * 256 * LIMBS;
                for_each_logit(v.row, vocab, [&](int, float l) { atomicAdd(&mine[(float_key(l) >> 24) * LIMBS], 1u); },
                               part, parts);
                __syncthreads();
                fold_private(priv, groups, share);
            } else {
                // few tokens are left, spread over the bins; a thread adds up a run of one bin before it
                // touches shared memory
                int cur = -1;
                unsigned long long run = 0;
                for_each_logit(v.row, vocab, [&](int, float l) {
                    const unsigned int key = float_key(l);
                    if ((key & mask) != prefix) return;
                    const int bin = (int)((key >> shift) & 255u);
                    if (bin == cur) { ++run; return; }
                    if (cur >= 0) atomicAdd(&share[cur], run);
                    cur = bin;
                    run = 1;
                }, part, parts);
                if (cur >= 0) atomicAdd(&share[cur], run);
            }
            if (parts > 1) {
                cluster.sync();                        // every block's share is complete
                if (tid < 256) {
                    unsigned long long sum = 0;
                    for (int c = 0; c < parts; ++c) sum += *cluster.map_shared_rank(&share[tid], c);
                    hist[tid] = sum;
                }
            }
            __syncthreads();
            if (tid < 32) select_bin(hist, need, sel);
            __syncthreads();
            prefix |= (unsigned int)sel[0] << shift;
            mask |= 0xFFu << shift;
            need -= sel[1];
            __syncthreads();
        }
        v.thr_key = prefix;
        // `need` + 1 of the tokens equal to the threshold are kept; cut by index if there are more
        if (tid == 0) found_idx = vocab;
        __syncthreads();
        const unsigned long long equal_total = hist[prefix & 255u];
        if (equal_total > need + 1) {
            if (tid == 0) {
                unsigned long long seen = 0;
                for (int i = 0; i < vocab; ++i)
                    if (float_key(v.row[i]) == prefix && ++seen == need + 1) { found_idx = i; break; }
            }
            __syncthreads();
        }
        v.idx_cut = found_idx;
        __syncthreads();
    }
    if (gather) {
        // (n_cand was set to zero at the start, and every block has passed a barrier of the block, and of the
        // cluster if there is one, since)
        int* count = parts > 1 ? cluster.map_shared_rank(&n_cand, 0) : &n_cand;
        float* list_logit = parts > 1 ? cluster.map_shared_rank(cand_logit, 0) : cand_logit;
        int* list_idx = parts > 1 ? cluster.map_shared_rank(cand_idx, 0) : cand_idx;
        for_each_logit(v.row, vocab, [&](int i, float l) {
            if (v.kept(float_key(l), i)) {
                const int at = atomicAdd(count, 1);        // top_k of them at most: the order does not matter
                if (at < SAMPLE_CANDIDATES) { list_logit[at] = l; list_idx[at] = i; }
            }
        }, part, parts);
        if (parts > 1) {
            cluster.sync();                            // the list is complete; block 0 goes on alone, reading
            if (part != 0) return;                     // nothing of the others any more
        }
        __syncthreads();
        float mx = -INFINITY;
        for (int c = tid; c < n_cand; c += SAMPLE_THREADS) mx = fmaxf(mx, cand_logit[c]);
        v.best = block_max(mx) / temperature;
    }
    // f(i, logit) for every kept token of this thread: from the list, or from the row (f checks `kept` itself)
    const int sharing = gather ? 1 : parts;         // blocks that share what follows (after a gather: block 0 alone)
    auto each_kept = [&](auto f) {
        if (gather) {
            for (int c = tid; c < n_cand; c += SAMPLE_THREADS) f(cand_idx[c], cand_logit[c]);
        } else {
            for_each_logit(v.row, vocab, f, part, parts);
        }
    };

    const long long request = request_ids ? request_ids[r] : r;
    const double u = uniform_draw(seed, (unsigned long long)request, (unsigned long long)draw_index[r]);
    unsigned long long target = 0;                 // u * (total mass of the kept tokens), known after the first pass

    // the key at which the running mass, taken from the largest logit down, passes target
    unsigned int prefix = 0, mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        unsigned long long* share = sharing > 1 ? hist_share[(shift >> 3) & 1] : hist;
        if (tid < 256) share[tid] = 0;
        __syncthreads();
        if (shift == 24 && private_ok) {
            zero_private(priv, groups);
            __syncthreads();
            unsigned int* mine = priv + (size_t)((tid >> 5) * groups / SAMPLE_WARPS) * 256 * LIMBS;
            each_kept([&](int i, float l) {
                const unsigned int key = float_key(l);
                if (!v.kept(key, i)) return;
                const unsigned long long w = v.mass(l);             // at most 2^40
                unsigned int* word = &mine[(key >> 24) * LIMBS];
                atomicAdd(word, (unsigned int)(w & ((1u << LIMB_BITS) - 1)));
                atomicAdd(word + 1, (unsigned int)(w >> LIMB_BITS));
            });
            __syncthreads();
            fold_private(priv, groups, share);
        } else {
            int cur = -1;
            unsigned long long run = 0;
            each_kept([&](int i, float l) {
                const unsigned int key = float_key(l);
                if ((key & mask) != prefix || !v.kept(key, i)) return;
                const int bin = (int)((key >> shift) & 255u);
                const unsigned long long w = v.mass(l);
                if (bin == cur) { run += w; return; }
                if (cur >= 0) atomicAdd(&share[cur], run);
                cur = bin;
                run = w;
            });
            if (cur >= 0) atomicAdd(&share[cur], run);
        }
        if (sharing > 1) {
            cluster.sync();                            // every block's share is complete
            if (tid < 256) {
                unsigned long long sum = 0;
                for (int c = 0; c < sharing; ++c) sum += *cluster.map_shared_rank(&share[tid], c);
                hist[tid] = sum;
            }
        }
        __syncthreads();
        if (shift == 24) {
            // the first histogram holds every kept token: its sum is the total mass the draw is scaled by
            if (tid == 0) total_smem = 0;
            __syncthreads();
            if (tid < 256) {
                unsigned long long part = hist[tid];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if ((tid & 31) == 0) atomicAdd(&total_smem, part);
            }
            __syncthreads();
            const unsigned long long total = total_smem;
            target = (unsigned long long)(u * (double)total);
            if (target >= total) target = total - 1;
        }
        if (tid < 32) select_bin(hist, target, sel);
        __syncthreads();
        prefix |= (unsigned int)sel[0] << shift;
        mask |= 0xFFu << shift;
        target -= sel[1];
        __syncthreads();
    }
    // tokens with exactly this key share one mass; the (target / mass)-th of them by index
    if (tid == 0) found_idx = vocab;
    __syncthreads();
    const unsigned long long group_mass = hist[prefix & 255u];
    float group_logit = 0.0f;
    {
        // recover the logit from the key
        const unsigned int b = (prefix & 0x80000000u) ? (prefix & 0x7FFFFFFFu) : ~prefix;
        group_logit = __uint_as_float(b);
    }
    const unsigned long long one = v.mass(group_logit);
    const unsigned long long nth = one ? target / one : 0;
    if (nth == 0) {
        each_kept([&](int i, float l) {
            if (float_key(l) == prefix && v.kept(prefix, i)) atomicMin(&found_idx, i);
        });
    } else if (tid == 0) {
        unsigned long long seen = 0;
        if (gather) {
            // the list is in no order: the next larger index among the equal ones, nth + 1 times
            int last = -1;
            for (;;) {
                int next = vocab;
                for (int c = 0; c < n_cand; ++c)
                    if (float_key(cand_logit[c]) == prefix && cand_idx[c] > last && cand_idx[c] < next) next = cand_idx[c];
                if (next == vocab) break;
                found_idx = last = next;             // the last one stands if fewer than nth + 1 exist
                if (seen++ == nth) break;
            }
        } else {
            for (int i = 0; i < vocab; ++i)
                if (float_key(v.row[i]) == prefix && v.kept(prefix, i)) {
                    found_idx = i;                   // the last one stands if fewer than nth + 1 exist
                    if (seen++ == nth) break;
                }
        }
    }
    (void)group_mass;
    __syncthreads();
    int picked = found_idx;
    if (sharing > 1) {
        cluster.sync();                                // every block's smallest index is in place
        if (nth == 0)
            for (int c = 0; c < sharing; ++c) picked = min(picked, *cluster.map_shared_rank(&found_idx, c));
        cluster.sync();                                // nobody leaves while another may read its shared memory
        if (part != 0) return;
    }
    if (tid == 0) {
        const int token = picked < vocab ? picked : 0;
        out[r] = token;
        draw_index[r] += 1;
        if (feed_ids) feed_ids[r] = token;
        if (feed_pos) {
            const int p = feed_pos[r] + 1;
            feed_pos[r] = p < last_pos ? p : last_pos;
        }
        status_copy.write(r);
    }
}

}  // namespace mu

// logits [n_rows, ld] float32 -> out[n_rows] token ids.  workspace: 2 * n_rows 64-bit words that are
// zero before the first launch (each launch leaves them zero).  With feed_ids the tokens are also written
// there, and with feed_pos those positions move on by one, up to last_pos: what mu_advance does, without
// its launch.  With status (and status_out) the word there is copied to status_out.
MU_EXPORT int mu_argmax(const float* logits, long long ld, int n_rows, int vocab, int* out,
                        unsigned long long* workspace, int* feed_ids, int* feed_pos, int last_pos,
                        const int* status, int* status_out, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (!logits || !out || !workspace || vocab <= 0 || ld < vocab) return MU_ERR_BAD_ARGUMENT;
    if (feed_pos && !feed_ids) return MU_ERR_BAD_ARGUMENT;
    if ((status == nullptr) != (status_out == nullptr)) return MU_ERR_BAD_ARGUMENT;
    const mu::StatusCopy status_copy{status, status_out};
    dim3 grid(n_rows, mu::ARGMAX_PARTS);
    return mu::launch_pdl(mu::argmax_kernel, grid, dim3(mu::ARGMAX_THREADS), 0, (cudaStream_t)stream, 1, logits, ld,
                          vocab, out, workspace, reinterpret_cast<unsigned int*>(workspace + n_rows), feed_ids,
                          feed_pos, last_pos, status_copy);
}

// request_ids [n_rows] int64 (null: the row index), draw_index [n_rows] int32 is read and
// then incremented.  temperature must be > 0; the caller routes greedy to mu_argmax.
MU_EXPORT int mu_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature,
                        int top_k, unsigned long long seed, const long long* request_ids,
                        int* draw_index, int* out, int* feed_ids, int* feed_pos, int last_pos,
                        const int* status, int* status_out, void* stream) {
    if (n_rows <= 0) return MU_OK;
    if (!logits || !out || !draw_index || vocab <= 0 || ld < vocab) return MU_ERR_BAD_ARGUMENT;
    if (!(temperature > 0.0f) || top_k < 0) return MU_ERR_BAD_ARGUMENT;
    if ((status == nullptr) != (status_out == nullptr)) return MU_ERR_BAD_ARGUMENT;
    const mu::StatusCopy status_copy{status, status_out};
    // the row in shared memory if it fits beside a histogram per warp (vocabularies up to some 32,000); else it
    // is read from the L2 in every pass (fewer histograms to make room cost more than the staging gains)
    const size_t limit = 208 * 1024;             // (the kernel has some 15 KB of static shared memory of its own)
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(mu::sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit) !=
            cudaSuccess)
            return MU_ERR_LAUNCH;
        raised = true;
    }
    const size_t row_bytes = ((size_t)vocab * 4 + 15) / 16 * 16;
    // a long row: up to eight blocks share the passes over it
    // (a block of this kernel has an SM to itself; clusters of eight find their place only while a third of the
    // SMs stay free)
    const int sms = mu::sm_count();
    int parts = 1;
    if (vocab >= 16 * mu::SAMPLE_THREADS && sms > 0)
        parts = n_rows * 8 <= sms * 2 / 3 ? 8 : n_rows * 4 <= sms * 9 / 10 ? 4 : n_rows * 2 <= sms ? 2 : 1;
    int staged = 0, groups = mu::SAMPLE_WARPS;
    size_t dyn = mu::sample_private_bytes(groups);
    if (parts == 1 && row_bytes + mu::sample_private_bytes(groups) <= limit) {
        staged = 1;
        dyn += row_bytes;
    }
    return mu::launch_pdl(mu::sample_kernel, dim3(n_rows, parts), dim3(mu::SAMPLE_THREADS), dyn, (cudaStream_t)stream, parts,
                          logits, ld, vocab, temperature, top_k, seed, request_ids, draw_index, out, feed_ids,
                          feed_pos, last_pos, status_copy, staged, groups, parts);
}
