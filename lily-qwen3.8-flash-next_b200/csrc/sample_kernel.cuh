// The sampling kernel: one launch draws every row of a batch.
//
// Grid (n_slices, rows), 512 threads. A thread block owns one slice of one
// row's vocabulary and makes ONE pass over it:
//
//   A. history ids -> a "seen" bitmap in shared memory (and, when the
//      frequency penalty needs multiplicities, a count table in global
//      scratch that the block clears again before it exits);
//   B. the few ids with a logit bias or a ban are adjusted one by one and
//      put into the candidate buffer up front;
//   C. the slice streams through a shared-memory ring filled by cp.async
//      (16 bytes per thread per round of 4096 logits, several rounds in
//      flight). A logit is looked at only if it beats a threshold that is
//      exact in the raw (unscaled) domain: the largest float c whose scaled
//      value does not beat a key that at least k untouched logits seen so
//      far reach. The first threshold comes from a fine histogram of the
//      first round; it is tightened from a small histogram of the keys
//      pushed since. Survivors go into the candidate buffer as raw bits;
//   D. the buffered candidates are adjusted all at once (bias and bans were
//      done in B; here the penalties, the division by the temperature and
//      the monotone key), the best k are selected exactly by (key
//      descending, id ascending), and go to global scratch; the last block
//      of the row to arrive (an atomic ticket, nobody waits) merges the
//      slices, sorts the k survivors and runs the softmax prefix / top-p /
//      min-p cut / draw exactly in the order the reference's CPU sampler
//      does (tests/unit/kernels/sample.rs:8-54).
//
// With one slice per row (large batches) step D ends in the same block.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lily_sampler.h"
#include "lily_math.cuh"

namespace lily {

constexpr int NT = 512;                 // threads per block
constexpr uint32_t FRAG_BYTES = 32;     // logit bytes per thread per round
constexpr uint32_t KCAP = LILY_K_CAP;
constexpr uint32_t CAP = 4096;          // candidate buffer entries
constexpr int STAGES = 2;               // rounds in flight in the cp.async ring
constexpr uint32_t RING_BYTES = STAGES * NT * FRAG_BYTES;
constexpr uint32_t SP_SMEM = 256;       // bias + ban entries staged in shared memory
constexpr uint32_t BLOOM_WORDS = 128;   // 4096-bit filter over the low 12 bits of a bias / ban id
constexpr uint32_t MAX_SLICES = LILY_MAX_SLICES;
constexpr uint32_t MIN_SLICE = 32768;   // shorter slices cost more in merging than they save (measured)
constexpr uint32_t H0_SHIFT = 19;       // first-round histogram: raw key >> 19, 8192 bins
constexpr uint32_t H0_BINS = 1u << (32 - H0_SHIFT);
constexpr uint32_t TH_BINS = 1024;      // tightening histogram: raw key >> 16 above a base
constexpr uint32_t RANKSORT_MAX = 384;  // candidate counts up to this are rank-sorted
constexpr uint32_t LCAP = 1024;         // candidates of a row in stream_rows_kernel, whose ring borrows key and id

// Per logit type: 16 bf16 or 8 f32 per thread per round.
template <typename T>
struct Geo {
    static constexpr uint32_t GROUP = FRAG_BYTES / sizeof(T);
    static constexpr uint32_t ROUND = NT * GROUP;
    static constexpr uint32_t RGROUP = 32u / GROUP;  // rounds between block-wide checks
};

// Row status bits OR-ed into the handle's status word.
constexpr uint32_t ROW_INTERNAL = 8;  // candidate buffer overflow: a bug, never expected

// What one vocabulary shard tells the others about a row: its best candidates
// in order (monotone key of the adjusted logit, vocabulary id; unused entries
// have id 0xFFFFFFFF), the largest adjusted logit of the shard and the sum of
// exp(adjusted - that) over the whole shard. 520 bytes.
struct ShardRecord {
    uint2 cand[LILY_SHARD_CANDIDATES];
    float max_adj;
    float sum_exp;
};
static_assert(sizeof(ShardRecord) == LILY_SHARD_RECORD_BYTES, "record layout is part of the ABI");

struct SpecArgs {
    const uint32_t *draft_ids;  // [n_spec]
    const float *q_dense;       // [n_spec, q_ld] or null
    uint64_t q_ld;
    const uint32_t *q_ids;      // [n_spec, KCAP] or null
    const float *q_probs;
    const uint32_t *q_n;
    const float *u_resid;       // [n_spec] or null (then from seed/step)
    uint32_t n_spec;            // rows below this index draw speculatively
};

struct KArgs {
    const void *logits;
    uint64_t logits_ld;
    uint32_t vocab;
    uint32_t rows;
    const lily_sampling_params_t *params;  // device [rows] (null with force_greedy)
    const float *uniforms;
    const uint32_t *steps;
    const uint32_t *history_ids;
    const uint32_t *history_len;
    uint64_t history_ld;
    const uint32_t *extra_ids;  // ids appended to every row's history (earlier draws of a step)
    uint32_t extra_len;
    uint32_t force_greedy;      // ignore params: exact argmax rows
    uint32_t max_history;       // history_len[row] above this (or above history_ld) refuses the row
    uint32_t max_list;          // likewise bias_len[row] and ban_len[row]
    const uint32_t *bias_ids;
    const float *bias_vals;
    const uint32_t *bias_len;
    uint64_t bias_ld;
    const uint32_t *ban_ids;
    const uint32_t *ban_len;
    uint64_t ban_ld;
    const int32_t *forced_ids;
    const uint32_t *count_slots;   // device [rows] or null
    uint32_t *counts_table;        // [slots, vocab]
    uint32_t *seen_table;          // [slots, seen_words]
    uint32_t seen_words;           // words per slot bitmap = ceil(vocab / 32)
    uint32_t row0;                 // first row of this launch (grid.y rows follow it)
    uint32_t *counts_scratch;      // [max_rows, vocab], all zero between launches
    uint32_t *out_ids;
    uint32_t *out_status;
    uint32_t *kept_n;
    uint32_t *kept_ids;
    float *kept_probs;
    uint64_t kept_ld;
    uint32_t n_slices;             // grid.x: the most slices a row may be cut into
    uint2 *part;                   // [max_rows, CAP] (key, id): slice s at s * k
    uint32_t *part_n;              // [max_rows, MAX_SLICES]
    uint32_t *tickets;             // [max_rows], zero between launches
    uint32_t *status_word;
    long long *phase_clocks;       // optional [max_rows, MAX_SLICES, LILY_PHASES] SM clock stamps
    // Vocabulary shards. A shard launch (cand_out set) keeps each row's best
    // shard_k candidates and writes them, sorted, as a ShardRecord instead of
    // drawing; the merge kernel draws from the records of all shards.
    uint32_t shard_k;              // candidates a sampled row keeps per shard (greedy rows keep 1)
    uint32_t id_offset;            // vocabulary id of this shard's logit 0
    ShardRecord *cand_out;         // [rows]
    uint32_t shard_sums;           // stream_rows_kernel: sum_exp of the record too, in the same pass
    const ShardRecord *merge_in;   // [merge_shards, merge_stride >= rows]
    uint32_t merge_shards;
    uint64_t merge_stride;         // records between two shards
    // The merge of a step whose records travel over peer memory (n == 0: not so):
    // a row's block first writes this rank's record of the row into every rank's
    // buffer and raises the row's flag there, then waits for the row's flags of
    // all ranks in its own buffer.
    struct PeerLink {
        void *buffers[16];         // rank r's exchange buffer as this process sees it
        const void *own;           // this rank's records of the step (null: already published)
        unsigned long long wait_ns;
        uint32_t n, rank, max_rows, step;
    } peer;
    float *out_lse;                // optional [rows]: log of the sum over the vocabulary of exp(adjusted)
    SpecArgs spec;
};

struct RowCtx {
    float T, rep, presence, frequency, top_p, min_p;
    uint32_t k;
    bool use_pen, need_counts, argmax_mode, monotone, has_special;
    uint32_t lo, hi;
    const uint32_t *seen;    // shared-memory bitmap of [lo, hi)
    const uint32_t *counts;  // global count table of this row (null unless need_counts)
    const uint32_t *bias_ids;
    const float *bias_vals;
    uint32_t bias_len;
    const uint32_t *ban_ids;
    uint32_t ban_len;
    bool sp_in_smem;
};

struct alignas(16) SmemFixed {
    uint32_t key[CAP];    // candidates: adjusted keys below n_adj, raw logit bits above;
    uint32_t id[CAP];     //   during the first round key+id hold the 8192-bin histogram
    uint32_t tkey[KCAP];  // select's histogram / staging; later the candidates' p
    uint32_t tid[KCAP];   // select's histogram / staging; later the prefix sums
    uint32_t thist[TH_BINS];
    uint32_t warp_sums[NT / 32];
    alignas(16) uint32_t sp_ids[SP_SMEM + 4];  // padded to a multiple of four with an id no logit has
    float sp_vals[SP_SMEM];
    uint32_t n;      // buffered candidates
    uint32_t n_adj;  // the first n_adj hold adjusted keys, the rest raw logit bits
    uint32_t cnt;
    uint32_t sel_digit;
    uint32_t sel_before;
    uint32_t sel_count;
    uint32_t sel_min;
    uint32_t sel_max;
    uint32_t tau_key;   // exact k-th key of the last selection
    uint32_t kstar;     // a logit is looked at iff its plain key is above this
    float c_raw;        // ... iff it is above this (NaN: no threshold yet)
    uint32_t th_base;   // key >> 16 of the tightening histogram's bin 0
    uint32_t th_new;    // pushes counted since the threshold was last tightened
    uint32_t overflow;  // a push found the buffer full
    uint32_t err;
    uint32_t is_last;
    uint32_t n_keep;
    uint32_t chosen;
    float p_d;
    float q_d;
    uint32_t bloom[BLOOM_WORDS];
    // Where pushes go: key / id (CAP entries), or lkey / lid (LCAP) while the
    // cp.async ring borrows key and id as its third and fourth stage.
    uint32_t *ckey;
    uint32_t *cid;
    uint32_t ccap;
    float u_draw;         // the row's uniform, fetched (or derived) when the block starts
    uint32_t lean_abort;  // stream_rows_kernel: a thread saw a NaN before the threshold was taken
    alignas(8) unsigned long long mbar[2];  // stream_rows_kernel: history marked; thread maxima written
    uint32_t lkey[LCAP];
    uint32_t lid[LCAP];
    RowCtx ctx;  // the row's parameters, for the out-of-line helpers
};

static_assert(2 * CAP >= H0_BINS, "the first-round histogram aliases the candidate buffer");
static_assert(CAP >= KCAP + NT, "a selection must leave room for one push per thread");

__device__ __forceinline__ float neg_inf() { return __uint_as_float(0xFF800000u); }

// Nanoseconds of the GPU's global timer: one time base for every block of a launch.
__device__ __forceinline__ long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return (long long)t;
}

// Warp-aggregated append to the candidate buffer. A full buffer refuses the
// entry and raises the overflow flag; the caller remembers the element and
// offers it again after the next selection has made room.
__device__ __forceinline__ bool push(SmemFixed *sm, uint32_t key, uint32_t id) {
    const unsigned act = __activemask();
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(act) - 1;
    uint32_t base = 0;
    if (lane == leader) {
        base = atomicAdd(&sm->n, (uint32_t)__popc(act));
    }
    base = __shfl_sync(act, base, leader);
    const uint32_t slot = base + __popc(act & ((1u << lane) - 1u));
    if (slot < sm->ccap) {
        sm->ckey[slot] = key;
        sm->cid[slot] = id;
        return true;
    }
    sm->overflow = 1;
    return false;
}

// The key of a logit that neither history nor bias nor ban touches.
__device__ __forceinline__ uint32_t plain_key(float l, float T, bool argmax_mode) {
    float q = __fdiv_rn(l, T);
    if (argmax_mode) {
        // The exact-argmax route compares floats: NaN never wins and the two
        // zeros tie (src/kernels/metal/elementwise.metal:145-150).
        q = q != q ? neg_inf() : __fadd_rn(q, 0.0f);
    }
    return key_of(q);
}

__device__ __forceinline__ bool seen_bit(const RowCtx &c, uint32_t id) {
    const uint32_t off = id - c.lo;
    return (c.seen[off >> 5] >> (off & 31u)) & 1u;
}

// Whether `id` is on the row's bias or ban list.
__device__ __forceinline__ bool is_special(const SmemFixed *sm, const RowCtx &c, uint32_t id) {
    if (!((sm->bloom[(id >> 5) & (BLOOM_WORDS - 1u)] >> (id & 31u)) & 1u)) {
        return false;
    }
    const uint32_t n = c.bias_len + c.ban_len;
    if (c.sp_in_smem) {
        // Four staged ids per load; the padding never matches.
        const uint4 *v = reinterpret_cast<const uint4 *>(sm->sp_ids);
        bool hit = false;
        for (uint32_t j = 0; j < n; j += 4u) {
            const uint4 e = v[j >> 2];
            hit = hit || e.x == id || e.y == id || e.z == id || e.w == id;
        }
        return hit;
    }
    for (uint32_t j = 0; j < n; ++j) {
        const uint32_t e = j < c.bias_len ? c.bias_ids[j] : c.ban_ids[j - c.bias_len];
        if (e == id) {
            return true;
        }
    }
    return false;
}

// The adjusted key of logit `l` of id `id`: bias (list order), penalties,
// ban, division by the temperature, monotone key. `special`: the id is on
// the bias / ban list (the up-front pass only; the stream skips those ids).
// A NaN marks the row as failed.
__device__ __noinline__ uint32_t adjusted_key(SmemFixed *sm, uint32_t id, float l, bool special) {
    const RowCtx &c = sm->ctx;
    float x = l;
    bool banned = false;
    if (special) {
        for (uint32_t j = 0; j < c.bias_len; ++j) {
            const uint32_t e = c.sp_in_smem ? sm->sp_ids[j] : c.bias_ids[j];
            if (e == id) {
                x = __fadd_rn(x, c.sp_in_smem ? sm->sp_vals[j] : c.bias_vals[j]);
            }
        }
        for (uint32_t j = 0; j < c.ban_len; ++j) {
            const uint32_t e = c.sp_in_smem ? sm->sp_ids[c.bias_len + j] : c.ban_ids[j];
            banned = banned || e == id;
        }
    }
    if (c.use_pen && seen_bit(c, id)) {
        float cnt = 1.0f;
        if (c.need_counts) {
            cnt = (float)__ldcg(c.counts + id);
        }
        x = x > 0.0f ? __fdiv_rn(x, c.rep) : __fmul_rn(x, c.rep);
        x = __fsub_rn(x, __fadd_rn(c.presence, __fmul_rn(c.frequency, cnt)));
    }
    if (banned) {
        x = neg_inf();
    }
    float q = __fdiv_rn(x, c.T);
    if (c.argmax_mode) {
        q = q != q ? neg_inf() : __fadd_rn(q, 0.0f);
    } else if (q != q) {
        sm->err = LILY_ROW_NAN;
        return 0u;
    }
    return key_of(q);
}

// The stream pushes raw logits; before a selection looks at the buffer, the
// entries pushed since the last one, [n_adj, n), become adjusted keys, all
// threads at once.
__device__ __noinline__ void adjust_pending(SmemFixed *sm) {
    const uint32_t n = min(sm->n, CAP);
    const uint32_t from = sm->n_adj;
    for (uint32_t i = from + threadIdx.x; i < n; i += NT) {
        sm->key[i] = adjusted_key(sm, sm->id[i], __uint_as_float(sm->key[i]), false);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        sm->n_adj = n;
    }
    __syncthreads();
}

// End of the stream: adjusts what is still raw and keeps only the entries
// whose key reaches the threshold (at least k of them do), compacted to the
// front in chunks so that no entry is overwritten before it is read.
__device__ __noinline__ void filter_adjust(SmemFixed *sm) {
    const uint32_t tid = threadIdx.x;
    const uint32_t n = min(sm->n, sm->ccap);
    const uint32_t from = sm->n_adj;
    const uint32_t kstar = sm->kstar;
    const uint32_t *src_key = sm->ckey, *src_id = sm->cid;
    if (tid == 0) {
        sm->cnt = 0;
    }
    __syncthreads();
    for (uint32_t c0 = 0; c0 < n; c0 += NT) {
        const uint32_t i = c0 + tid;
        bool alive = false;
        uint32_t key = 0, id = 0;
        if (i < n) {
            id = src_id[i];
            key = src_key[i];
            if (i >= from) {
                key = adjusted_key(sm, id, __uint_as_float(key), false);
            }
            alive = key >= kstar;
        }
        __syncthreads();  // the chunk is read: survivors may now land in it
        if (alive) {
            const unsigned act = __activemask();
            const int lane = tid & 31;
            const int leader = __ffs(act) - 1;
            uint32_t base = 0;
            if (lane == leader) {
                base = atomicAdd(&sm->cnt, (uint32_t)__popc(act));
            }
            base = __shfl_sync(act, base, leader);
            const uint32_t pos = base + __popc(act & ((1u << lane) - 1u));
            sm->key[pos] = key;
            sm->id[pos] = id;
        }
    }
    __syncthreads();
    if (tid == 0) {
        sm->n = sm->cnt;
        sm->n_adj = sm->cnt;
        sm->ckey = sm->key;  // from here on the candidates live in key / id
        sm->cid = sm->id;
        sm->ccap = CAP;
    }
    __syncthreads();
}

constexpr uint32_t SEL_BITS = 11;
constexpr uint32_t SEL_BINS = 1u << SEL_BITS;  // the select's histogram aliases tkey + tid

// All threads: finds the bin of hist[0, nbins), nbins <= BPT * 512, in which the running count,
// taken from the top bin down when `descending` and from bin 0 up otherwise,
// reaches `remaining`. Results in sm->sel_digit / sel_before / sel_count.
template <int BPT>
__device__ __forceinline__ void find_bin(SmemFixed *sm, const uint32_t *hist, uint32_t nbins,
                                         uint32_t remaining, bool descending) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t c[BPT];
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < BPT; ++j) {
        const uint32_t pos = tid * (uint32_t)BPT + j;
        uint32_t v = 0;
        if (pos < nbins) {
            v = hist[descending ? nbins - 1u - pos : pos];
        }
        c[j] = v;
        sum += v;
    }
    uint32_t incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (lane >= (uint32_t)off) {
            incl += t;
        }
    }
    if (lane == 31u) {
        sm->warp_sums[warp] = incl;
    }
    __syncthreads();
    uint32_t before = 0;
    for (uint32_t w = 0; w < warp; ++w) {
        before += sm->warp_sums[w];
    }
    const uint32_t excl = before + incl - sum;
    if (excl < remaining && remaining <= excl + sum) {
        uint32_t cum = excl;
#pragma unroll
        for (int j = 0; j < BPT; ++j) {
            if (cum + c[j] >= remaining) {
                const uint32_t pos = tid * (uint32_t)BPT + j;
                sm->sel_digit = descending ? nbins - 1u - pos : pos;
                sm->sel_before = cum;
                sm->sel_count = c[j];
                break;
            }
            cum += c[j];
        }
    }
    __syncthreads();
}

// Range-adaptive radix select over the buffered candidates [0, n).
//   BY_ID = false: the `remaining`-th largest key.
//   BY_ID = true:  the `remaining`-th smallest id among entries whose key is kstar.
// Every pass buckets the live value range [lo, hi] into at most 2048 bins
// (so that candidates, whose float keys share their high bits, still spread
// over the histogram), keeps the bin that holds the wanted rank and narrows
// the range to it; three passes at most. Returns the value; *remaining_out
// is the rank wanted inside that value's ties, *count_eq_out how many
// entries hold the value.
template <bool BY_ID>
__device__ __noinline__ uint32_t adaptive_select(SmemFixed *sm, uint32_t n, uint32_t remaining, uint32_t kstar,
                                    uint32_t *remaining_out, uint32_t *count_eq_out) {
    const uint32_t tid = threadIdx.x;
    uint32_t *hist = sm->tkey;  // SEL_BINS words: tkey and tid are adjacent
    if (tid == 0) {
        sm->sel_min = 0xFFFFFFFFu;
        sm->sel_max = 0u;
    }
    __syncthreads();
    uint32_t mn = 0xFFFFFFFFu, mx = 0u;
    for (uint32_t i = tid; i < n; i += NT) {
        if (!BY_ID || sm->key[i] == kstar) {
            const uint32_t v = BY_ID ? sm->id[i] : sm->key[i];
            mn = min(mn, v);
            mx = max(mx, v);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, off));
        mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    }
    if ((tid & 31u) == 0u) {
        atomicMin(&sm->sel_min, mn);
        atomicMax(&sm->sel_max, mx);
    }
    __syncthreads();
    uint32_t lo = sm->sel_min, hi = sm->sel_max;
    uint32_t count_eq = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const uint32_t range = hi - lo;
        const uint32_t bits = 32u - (uint32_t)__clz((int)range);  // 0 when range == 0
        const uint32_t shift = bits > SEL_BITS ? bits - SEL_BITS : 0u;
        const uint32_t nbins = (range >> shift) + 1u;
        for (uint32_t b = tid; b < nbins; b += NT) {
            hist[b] = 0;
        }
        __syncthreads();
        for (uint32_t i0 = 0; i0 < n; i0 += NT) {
            const uint32_t i = i0 + tid;
            bool ok = i < n;
            uint32_t bin = 0;
            if (ok) {
                ok = !BY_ID || sm->key[i] == kstar;
                const uint32_t v = BY_ID ? sm->id[i] : sm->key[i];
                ok = ok && v >= lo && v <= hi;
                bin = (v - lo) >> shift;
            }
            // Candidates crowd into few bins: one atomic per distinct bin of the warp.
            const unsigned live = __ballot_sync(0xFFFFFFFFu, ok);
            if (ok) {
                const unsigned peers = __match_any_sync(live, bin);
                if ((tid & 31u) == (uint32_t)(__ffs(peers) - 1)) {
                    atomicAdd(&hist[bin], (uint32_t)__popc(peers));
                }
            }
        }
        __syncthreads();
        find_bin<SEL_BINS / NT>(sm, hist, nbins, remaining, !BY_ID);
        remaining -= sm->sel_before;
        count_eq = sm->sel_count;
        const uint32_t new_lo = lo + (sm->sel_digit << shift);
        const uint32_t width = shift == 0u ? 0u : (1u << shift) - 1u;
        hi = min(hi, new_lo + width);
        lo = new_lo;
        __syncthreads();
        if (shift == 0u) {
            break;
        }
    }
    *remaining_out = remaining;
    *count_eq_out = count_eq;
    return lo;
}

// Keeps the best k of the n buffered candidates (n > k), by key descending
// then id ascending, in slots [0, k) in any order; records the k-th key.
__device__ __noinline__ void select_topk(SmemFixed *sm, uint32_t n, uint32_t k) {
    const uint32_t tid = threadIdx.x;
    uint32_t remaining = 0, count_eq = 0;
    const uint32_t kstar = adaptive_select<false>(sm, n, k, 0u, &remaining, &count_eq);
    uint32_t istar = 0xFFFFFFFFu;
    if (count_eq > remaining) {
        // More candidates share the k-th key than fit: the lowest ids win.
        uint32_t r2 = 0, c2 = 0;
        istar = adaptive_select<true>(sm, n, remaining, kstar, &r2, &c2);
    }
    if (tid == 0) {
        sm->cnt = 0;
    }
    __syncthreads();
    // The survivors go to the front of the id array's upper half first (the
    // histogram's storage doubles as staging and is free again by now).
    for (uint32_t i0 = 0; i0 < n; i0 += NT) {
        const uint32_t i = i0 + tid;
        if (i < n) {
            const uint32_t key = sm->key[i];
            const uint32_t id = sm->id[i];
            if (key > kstar || (key == kstar && id <= istar)) {
                const unsigned act = __activemask();
                const int lane = tid & 31;
                const int leader = __ffs(act) - 1;
                uint32_t base = 0;
                if (lane == leader) {
                    base = atomicAdd(&sm->cnt, (uint32_t)__popc(act));
                }
                base = __shfl_sync(act, base, leader);
                const uint32_t slot = base + __popc(act & ((1u << lane) - 1u));
                if (slot < KCAP) {
                    sm->tkey[slot] = key;
                    sm->tid[slot] = id;
                }
            }
        }
    }
    __syncthreads();
    for (uint32_t i = tid; i < k; i += NT) {
        sm->key[i] = sm->tkey[i];
        sm->id[i] = sm->tid[i];
    }
    if (tid == 0) {
        if (sm->cnt != k) {
            sm->err = ROW_INTERNAL;
        }
        sm->n = k;
        sm->n_adj = k;
        sm->tau_key = kstar;
    }
    __syncthreads();
}

// The largest raw logit c whose plain key does not beat kstar: an untouched
// logit l beats the k-th candidate exactly when l > c. Thread 0 only.
__device__ __noinline__ float raw_threshold(uint32_t kstar, float T, bool argmax_mode) {
    const float tq = float_of_key(kstar);
    if (tq != tq) {
        return tq;
    }
    if (tq == neg_inf() || tq == -neg_inf()) {
        return tq;
    }
    uint32_t ck = key_of(__fmul_rn(tq, T));
    int it = 0;
    while (plain_key(float_of_key(ck), T, argmax_mode) > kstar && it < 64) {
        --ck;
        ++it;
    }
    while (plain_key(float_of_key(ck + 1u), T, argmax_mode) <= kstar && it < 64) {
        ++ck;
        ++it;
    }
    if (it >= 64) {
        return neg_inf();  // conservative: every finite logit is looked at
    }
    float c = float_of_key(ck);
    if (c == 0.0f) {
        // The float compare cannot tell the zeros apart; let both through.
        c = __uint_as_float(0x80000001u);
    }
    return c;
}

// The steps after the selection run on k candidates. For k <= 64 (the
// common case) one warp does them with warp barriers only; larger k uses the
// whole block. `Team` abstracts the two.
template <bool SMALL>
struct Team {
    static __device__ __forceinline__ uint32_t size() { return SMALL ? 32u : (uint32_t)NT; }
    static __device__ __forceinline__ uint32_t rank() {
        return SMALL ? (threadIdx.x & 31u) : threadIdx.x;
    }
    static __device__ __forceinline__ void sync() {
        if (SMALL) {
            __syncwarp();
        } else {
            __syncthreads();
        }
    }
};

// Bitonic sort of slots [0, n) by (key descending, id ascending).
template <bool SMALL>
__device__ __noinline__ void sort_candidates(SmemFixed *sm, uint32_t n) {
    const uint32_t me = Team<SMALL>::rank(), team = Team<SMALL>::size();
    uint32_t P = 1;
    while (P < n) {
        P <<= 1;
    }
    for (uint32_t i = n + me; i < P; i += team) {
        sm->key[i] = 0u;
        sm->id[i] = 0xFFFFFFFFu;
    }
    Team<SMALL>::sync();
    for (uint32_t size = 2; size <= P; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            for (uint32_t t = me; t < (P >> 1); t += team) {
                const uint32_t i = ((t / stride) * stride << 1) + (t % stride);
                const uint32_t j = i + stride;
                const uint32_t ka = sm->key[i], kb = sm->key[j];
                const uint32_t ia = sm->id[i], ib = sm->id[j];
                const bool a_first = ka > kb || (ka == kb && ia < ib);
                const bool forward = (i & size) == 0;
                if (forward != a_first) {
                    sm->key[i] = kb;
                    sm->key[j] = ka;
                    sm->id[i] = ib;
                    sm->id[j] = ia;
                }
            }
            Team<SMALL>::sync();
        }
    }
}

// Whole-block sort of slots [0, n), n <= SORT2K, by (key descending, id
// ascending): a bitonic network over 2048 packed (key, ~id) words, four per
// thread in registers. Partners fewer than 32 slots apart sit in the same warp
// and trade by shuffle; only the wider strides go through shared memory (the
// key and id arrays, overlaid as 64-bit words, one barrier per stage).
constexpr uint32_t SORT2K = 2048;
static_assert(SORT2K == 4 * NT && 2 * SORT2K <= 2 * CAP, "four slots per thread; the overlay fits key + id");

__device__ __forceinline__ unsigned long long sort_exchange(unsigned long long v, unsigned long long other,
                                                            bool keep_first) {
    return keep_first ? (v > other ? v : other) : (v < other ? v : other);
}

__device__ __noinline__ void sort_block_2k(SmemFixed *sm, uint32_t n) {
    const uint32_t t = threadIdx.x;
    unsigned long long *buf = reinterpret_cast<unsigned long long *>(sm->key);
    unsigned long long v[4];
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
        const uint32_t idx = t + NT * r;
        v[r] = idx < n ? ((unsigned long long)sm->key[idx] << 32) | (uint32_t)~sm->id[idx] : 0ull;
    }
    __syncthreads();  // every slot is in a register: the arrays may be overlaid
    // Stages of one network level whose partners are in the same warp.
    auto warp_stages = [&](uint32_t size, uint32_t from_stride) {
        for (uint32_t stride = from_stride; stride > 0u; stride >>= 1) {
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r) {
                const uint32_t idx = t + NT * r;
                const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, v[r], stride);
                const bool forward = (idx & size) == 0u, lower = (idx & stride) == 0u;
                v[r] = sort_exchange(v[r], other, forward == lower);
            }
        }
    };
    for (uint32_t size = 2u; size <= 32u; size <<= 1) {
        warp_stages(size, size >> 1);
    }
    for (uint32_t size = 64u; size <= SORT2K; size <<= 1) {
#pragma unroll
        for (uint32_t r = 0; r < 4u; ++r) {
            buf[t + NT * r] = v[r];
        }
        __syncthreads();
        for (uint32_t stride = size >> 1; stride >= 32u; stride >>= 1) {
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                const uint32_t pr = t + NT * h;  // one of the 1024 pairs
                const uint32_t i = ((pr / stride) * stride << 1) + (pr % stride);
                const uint32_t j = i + stride;
                const unsigned long long x = buf[i], y = buf[j];
                const bool forward = (i & size) == 0u;
                if ((x < y) == forward) {
                    buf[i] = y;
                    buf[j] = x;
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (uint32_t r = 0; r < 4u; ++r) {
            v[r] = buf[t + NT * r];
        }
        warp_stages(size, 16u);
    }
    __syncthreads();  // the overlay has been read for the last time
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
        const uint32_t idx = t + NT * r;
        if (idx < n) {
            sm->key[idx] = (uint32_t)(v[r] >> 32);
            sm->id[idx] = ~(uint32_t)v[r];
        }
    }
    __syncthreads();
}

// First slot of [0, n) whose prefix sum exceeds target, else the last slot
// (tests/unit/kernels/sample.rs:48-52). Result in sm->chosen.
template <bool SMALL>
__device__ __forceinline__ void pick(SmemFixed *sm, const float *cum, uint32_t n, float target) {
    const uint32_t me = Team<SMALL>::rank(), team = Team<SMALL>::size();
    if (me == 0) {
        sm->chosen = n - 1u;
    }
    Team<SMALL>::sync();
    for (uint32_t i = me; i < n; i += team) {
        if (target < cum[i]) {
            atomicMin(&sm->chosen, i);
        }
    }
    Team<SMALL>::sync();
}

// Steps 6-8 on the sorted candidates [0, n): softmax weights, sequential
// prefix, cut, draw (plain or speculative), outputs.
template <bool SMALL>
__device__ __noinline__ void finalize(SmemFixed *sm, const KArgs &a, uint32_t row, uint32_t n,
                                      uint64_t seed) {
    const RowCtx &c = sm->ctx;
    const uint32_t me = Team<SMALL>::rank(), team = Team<SMALL>::size();
    const uint32_t out_row = row;
    float *p = reinterpret_cast<float *>(sm->tkey);
    float *cum = reinterpret_cast<float *>(sm->tid);
    const float top = float_of_key(sm->key[0]);
    uint32_t err = sm->err;
    if (!c.argmax_mode && err == 0 && (top == neg_inf() || top == -neg_inf())) {
        err = LILY_ROW_NONFINITE;
    }
    if (err != 0) {
        if (me == 0) {
            a.out_ids[out_row] = 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[out_row] = err;
            }
            if (a.kept_n) {
                a.kept_n[out_row] = 0;
            }
            atomicOr(a.status_word, 1u << (err & 31u));
        }
        return;
    }
    if (c.argmax_mode) {
        if (me == 0) {
            a.out_ids[out_row] = sm->id[0];
            if (a.out_status) {
                a.out_status[out_row] = LILY_ROW_OK;
            }
            if (a.kept_n) {
                a.kept_n[out_row] = 1;
                a.kept_ids[(uint64_t)out_row * a.kept_ld] = sm->id[0];
                a.kept_probs[(uint64_t)out_row * a.kept_ld] = 1.0f;
            }
        }
        return;
    }
    // The uniform is fetched early: its latency hides behind the prefix sums.
    float u;
    uint32_t step = 0;
    if (a.uniforms) {
        u = a.uniforms[row];
    } else {
        step = a.steps ? a.steps[row] : 0u;
        u = uniform_for(seed, step);
    }
    for (uint32_t i = me; i < n; i += team) {
        p[i] = exp_f32(__fsub_rn(float_of_key(sm->key[i]), top));
    }
    Team<SMALL>::sync();
    if (me == 0) {
        // One thread, rank order, one rounding per add (for n <= 64 too: a
        // chain of dependent adds is shorter than a chain of shuffles).
        const float *__restrict__ pr = p;
        float *__restrict__ cw = cum;
        float s = 0.0f;
        for (uint32_t i = 0; i < n; ++i) {
            s = __fadd_rn(s, pr[i]);
            cw[i] = s;
        }
        sm->n_keep = n;
    }
    Team<SMALL>::sync();
    const float limit = __fmul_rn(c.top_p, cum[n - 1u]);
    for (uint32_t i = me + 1u; i < n; i += team) {
        if (!(cum[i - 1u] < limit && p[i] >= c.min_p)) {
            atomicMin(&sm->n_keep, i);
        }
    }
    Team<SMALL>::sync();
    const uint32_t n_keep = sm->n_keep;
    const float mass = cum[n_keep - 1u];

    if (a.kept_n) {
        for (uint32_t i = me; i < n_keep; i += team) {
            a.kept_ids[(uint64_t)out_row * a.kept_ld + i] = sm->id[i];
            a.kept_probs[(uint64_t)out_row * a.kept_ld + i] = __fdiv_rn(p[i], mass);
        }
        if (me == 0) {
            a.kept_n[out_row] = n_keep;
        }
    }

    uint32_t chosen_id;
    if (row < a.spec.n_spec) {
        // Speculative draw against proposal `row` (tests/unit/kernels/
        // sample.rs:264-283; src/kernels/metal/sample.metal:597-658).
        const uint32_t d = a.spec.draft_ids[row];
        if (me == 0) {
            sm->p_d = 0.0f;
            float qd = 0.0f;
            if (a.spec.q_dense) {
                qd = d < a.vocab ? a.spec.q_dense[(uint64_t)row * a.spec.q_ld + d] : 0.0f;
            }
            sm->q_d = qd;
        }
        Team<SMALL>::sync();
        const uint32_t qn = a.spec.q_dense ? 0u : min(a.spec.q_n[row], KCAP);
        const uint32_t *qi = a.spec.q_ids + (uint64_t)row * KCAP;
        const float *qp = a.spec.q_probs + (uint64_t)row * KCAP;
        for (uint32_t i = me; i < n_keep; i += team) {
            if (sm->id[i] == d) {
                sm->p_d = __fdiv_rn(p[i], mass);
            }
        }
        for (uint32_t j = me; j < qn; j += team) {
            if (qi[j] == d) {
                sm->q_d = qp[j];
            }
        }
        Team<SMALL>::sync();
        if (__fmul_rn(u, sm->q_d) < sm->p_d) {
            chosen_id = d;
        } else {
            // Residual max(0, p - q) over the kept set, rank order.
            float *r = reinterpret_cast<float *>(sm->key + KCAP);
            float *rcum = reinterpret_cast<float *>(sm->id + KCAP);
            for (uint32_t i = me; i < n_keep; i += team) {
                const uint32_t id = sm->id[i];
                float q = 0.0f;
                if (a.spec.q_dense) {
                    q = a.spec.q_dense[(uint64_t)row * a.spec.q_ld + id];
                } else {
                    for (uint32_t j = 0; j < qn; ++j) {
                        if (qi[j] == id) {
                            q = qp[j];
                            break;
                        }
                    }
                }
                const float x = __fsub_rn(__fdiv_rn(p[i], mass), q);
                r[i] = x > 0.0f ? x : 0.0f;
            }
            Team<SMALL>::sync();
            if (me == 0) {
                float s = 0.0f;
                for (uint32_t i = 0; i < n_keep; ++i) {
                    s = __fadd_rn(s, r[i]);
                    rcum[i] = s;
                }
            }
            Team<SMALL>::sync();
            const float r_total = rcum[n_keep - 1u];
            float u2;
            if (a.spec.u_resid) {
                u2 = a.spec.u_resid[row];
            } else {
                u2 = uniform_for(seed, step | 0x80000000u);
            }
            if (r_total > 0.0f) {
                pick<SMALL>(sm, rcum, n_keep, __fmul_rn(u2, r_total));
            } else {
                pick<SMALL>(sm, cum, n_keep, __fmul_rn(u2, mass));
            }
            chosen_id = sm->id[sm->chosen];
        }
    } else {
        pick<SMALL>(sm, cum, n_keep, __fmul_rn(u, mass));
        chosen_id = sm->id[sm->chosen];
    }
    if (me == 0) {
        a.out_ids[out_row] = chosen_id;
        if (a.out_status) {
            a.out_status[out_row] = LILY_ROW_OK;
        }
        if (c.use_pen && a.count_slots) {
            // src/kernels/metal/sample.metal:509-511: the draw is counted.
            const uint32_t slot = a.count_slots[row];
            if (chosen_id < a.vocab) {
                atomicAdd(a.counts_table + (uint64_t)slot * a.vocab + chosen_id, 1u);
                atomicOr(a.seen_table + (uint64_t)slot * a.seen_words + (chosen_id >> 5),
                         1u << (chosen_id & 31u));
            }
        }
    }
}

// finalize for at most 64 sorted candidates and a plain (not speculative)
// draw, one warp, everything in registers: lane i holds candidates i and
// i + 32. The prefix sums are the sequential rank-order sums of the
// reference (tests/unit/kernels/sample.rs:37-46): every lane runs the same
// chain of adds over values handed round by shuffles, which do not sit on the
// chain.
__device__ __noinline__ void finalize_warp(SmemFixed *sm, const KArgs &a, uint32_t row, uint32_t n,
                                           uint64_t seed) {
    const RowCtx &c = sm->ctx;
    const uint32_t lane = threadIdx.x & 31u;
    constexpr unsigned FULL = 0xFFFFFFFFu;
    const uint32_t k0 = lane < n ? sm->key[lane] : 0u, k1 = lane + 32u < n ? sm->key[lane + 32u] : 0u;
    const uint32_t i0 = lane < n ? sm->id[lane] : 0xFFFFFFFFu, i1 = lane + 32u < n ? sm->id[lane + 32u] : 0xFFFFFFFFu;
    const float top = float_of_key(__shfl_sync(FULL, k0, 0));
    uint32_t err = sm->err;
    if (!c.argmax_mode && err == 0 && (top == neg_inf() || top == -neg_inf())) {
        err = LILY_ROW_NONFINITE;
    }
    if (err != 0) {
        if (lane == 0) {
            a.out_ids[row] = 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[row] = err;
            }
            if (a.kept_n) {
                a.kept_n[row] = 0;
            }
            atomicOr(a.status_word, 1u << (err & 31u));
        }
        return;
    }
    if (c.argmax_mode) {
        if (lane == 0) {
            a.out_ids[row] = i0;
            if (a.out_status) {
                a.out_status[row] = LILY_ROW_OK;
            }
            if (a.kept_n) {
                a.kept_n[row] = 1;
                a.kept_ids[(uint64_t)row * a.kept_ld] = i0;
                a.kept_probs[(uint64_t)row * a.kept_ld] = 1.0f;
            }
        }
        return;
    }
    const float u = sm->u_draw;
    const float p0 = lane < n ? exp_f32(__fsub_rn(float_of_key(k0), top)) : 0.0f;
    const float p1 = lane + 32u < n ? exp_f32(__fsub_rn(float_of_key(k1), top)) : 0.0f;
    // The running sum in rank order, one add after the other as the reference's
    // CPU sampler does it. Unrolled over all 32 lanes: the shuffles do not depend
    // on the sum and go out back to back, the chain is the adds alone; ranks past
    // n weigh 0, and s + 0 is s (s is never -0).
    float s = 0.0f, c0 = 0.0f, c1 = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < 32u; ++i) {
        s = __fadd_rn(s, __shfl_sync(FULL, p0, (int)i));
        c0 = lane == i ? s : c0;
    }
    if (n > 32u) {
#pragma unroll
        for (uint32_t i = 0; i < 32u; ++i) {
            s = __fadd_rn(s, __shfl_sync(FULL, p1, (int)i));
            c1 = lane == i ? s : c1;
        }
    }
    // Keep rank i >= 1 while the mass before it is below top_p of the total and
    // its weight reaches min_p; the first rank that fails ends the kept set.
    const float limit = __fmul_rn(c.top_p, s);
    const float up0 = __shfl_up_sync(FULL, c0, 1);
    const float up1 = __shfl_up_sync(FULL, c1, 1);
    const float last0 = __shfl_sync(FULL, c0, 31);
    const float before0 = up0, before1 = lane == 0u ? last0 : up1;
    uint32_t stop = n;
    if (lane + 32u < n && !(before1 < limit && p1 >= c.min_p)) {
        stop = lane + 32u;
    }
    if (lane >= 1u && lane < n && !(before0 < limit && p0 >= c.min_p)) {
        stop = lane;
    }
    const uint32_t n_keep = __reduce_min_sync(FULL, stop);
    const uint32_t last = n_keep - 1u;
    const float mass = last < 32u ? __shfl_sync(FULL, c0, (int)last) : __shfl_sync(FULL, c1, (int)(last - 32u));
    if (a.kept_n) {
        if (lane < n_keep) {
            a.kept_ids[(uint64_t)row * a.kept_ld + lane] = i0;
            a.kept_probs[(uint64_t)row * a.kept_ld + lane] = __fdiv_rn(p0, mass);
        }
        if (lane + 32u < n_keep) {
            a.kept_ids[(uint64_t)row * a.kept_ld + lane + 32u] = i1;
            a.kept_probs[(uint64_t)row * a.kept_ld + lane + 32u] = __fdiv_rn(p1, mass);
        }
        if (lane == 0) {
            a.kept_n[row] = n_keep;
        }
    }
    // First kept rank whose prefix sum exceeds the target, else the last one
    // (tests/unit/kernels/sample.rs:48-52).
    const float target = __fmul_rn(u, mass);
    uint32_t hit = last;
    if (lane + 32u < n_keep && target < c1) {
        hit = lane + 32u;
    }
    if (lane < n_keep && target < c0) {
        hit = lane;
    }
    const uint32_t chosen = __reduce_min_sync(FULL, hit);
    const uint32_t chosen_id = chosen < 32u ? __shfl_sync(FULL, i0, (int)chosen) : __shfl_sync(FULL, i1, (int)(chosen - 32u));
    if (lane == 0) {
        a.out_ids[row] = chosen_id;
        if (a.out_status) {
            a.out_status[row] = LILY_ROW_OK;
        }
        if (c.use_pen && a.count_slots) {
            // src/kernels/metal/sample.metal:509-511: the draw is counted.
            const uint32_t slot = a.count_slots[row];
            if (chosen_id < a.vocab) {
                atomicAdd(a.counts_table + (uint64_t)slot * a.vocab + chosen_id, 1u);
                atomicOr(a.seen_table + (uint64_t)slot * a.seen_words + (chosen_id >> 5),
                         1u << (chosen_id & 31u));
            }
        }
    }
}


// Raises the raw threshold to `c` (pass iff l > c) and the adjusted-key
// threshold to `kstar` (survivors have key >= kstar). Any single thread;
// concurrent callers only ever store valid thresholds.
__device__ __forceinline__ void raise_threshold(SmemFixed *sm, float c, uint32_t kstar) {
    if (c == c && !(c <= sm->c_raw)) {
        sm->c_raw = c;
    }
    if (kstar > sm->kstar) {
        sm->kstar = kstar;
    }
}

// After an exact selection: the k-th key is the new threshold.
__device__ __forceinline__ void set_exact_threshold(SmemFixed *sm, uint32_t kth_key) {
    const RowCtx &c = sm->ctx;
    raise_threshold(sm, raw_threshold(kth_key, c.T, c.argmax_mode), kth_key);
}

// At least k untouched logits have a raw key of `edge_key` or more: no logit
// below that value can be among the best k (scaling keeps the order).
__device__ __forceinline__ void set_raw_edge(SmemFixed *sm, uint32_t edge_key) {
    const RowCtx &c = sm->ctx;
    if (edge_key == 0u) {
        return;
    }
    float below = float_of_key(edge_key - 1u);
    if (below == 0.0f) {
        below = __uint_as_float(0x80000001u);  // the float compare cannot tell the zeros apart
    }
    const uint32_t pk = plain_key(float_of_key(edge_key), c.T, c.argmax_mode);
    raise_threshold(sm, below, pk > 0u ? pk - 1u : 0u);
}

// One warp tightens the threshold from the histogram of the raw keys pushed
// so far: the highest bin edge that at least k counted (untouched) logits
// reach. Only the bins at and above the current threshold can matter.
__device__ __noinline__ void tighten(SmemFixed *sm) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t k = sm->ctx.k;
    const uint32_t base = sm->th_base;
    const uint32_t cur16 = key_of(sm->c_raw) >> 16;  // a NaN threshold maps above every bin
    const uint32_t lo_bin = (sm->c_raw == sm->c_raw && cur16 > base)
                                ? min(cur16 - base, TH_BINS - 1u)
                                : 0u;
    const uint32_t per = (TH_BINS - lo_bin + 31u) / 32u;  // bins per lane, from the top down
    uint32_t sum = 0;
    for (uint32_t j = 0; j < per; ++j) {
        const uint32_t pos = lane * per + j;
        if (pos < TH_BINS - lo_bin) {
            sum += sm->thist[TH_BINS - 1u - pos];
        }
    }
    uint32_t incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (lane >= (uint32_t)off) {
            incl += t;
        }
    }
    const uint32_t excl = incl - sum;
    if (excl < k && k <= incl) {
        uint32_t cum = excl;
        for (uint32_t j = 0; j < per; ++j) {
            const uint32_t pos = lane * per + j;
            if (pos >= TH_BINS - lo_bin) {
                break;
            }
            const uint32_t bin = TH_BINS - 1u - pos;
            cum += sm->thist[bin];
            if (cum >= k) {
                // (The top bin also holds everything above it; its lower
                // edge is as valid a bound.)
                if (base + bin <= 0xFFFFu) {
                    set_raw_edge(sm, (base + bin) << 16);
                }
                break;
            }
        }
    }
    if (lane == 0) {
        sm->th_new = 0;
    }
}

// Exact best-k of n <= RANKSORT_MAX buffered candidates by counting, for
// each, how many others come before it: the best k land sorted in [0, k).
__device__ __noinline__ void rank_sort(SmemFixed *sm, uint32_t n, uint32_t k) {
    const uint32_t tid = threadIdx.x;
    uint32_t rank = 0xFFFFFFFFu, mk = 0, mi = 0;
    if (tid < n) {
        mk = sm->key[tid];
        mi = sm->id[tid];
        rank = 0;
        for (uint32_t j = 0; j < n; ++j) {
            const uint32_t kj = sm->key[j], ij = sm->id[j];
            rank += (kj > mk || (kj == mk && ij < mi)) ? 1u : 0u;
        }
    }
    __syncthreads();
    if (rank < k) {
        sm->key[rank] = mk;
        sm->id[rank] = mi;
    }
    if (tid == 0) {
        sm->n = min(n, k);
        sm->n_adj = min(n, k);
    }
    __syncthreads();
}

// cp.async: 16 bytes global -> shared, `bytes` of them read, the rest zero.
__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gsrc, uint32_t bytes) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gsrc),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// One thread's logits of a round: 32 bytes, 16 bf16 or 8 f32.
struct Frag {
    uint4 v[2];
};

template <typename T>
__device__ __forceinline__ float frag_get(const Frag &f, int e);

template <>
__device__ __forceinline__ float frag_get<float>(const Frag &f, int e) {
    const uint4 &q = f.v[e >> 2];
    const uint32_t w = (e & 3) == 0 ? q.x : (e & 3) == 1 ? q.y : (e & 3) == 2 ? q.z : q.w;
    return __uint_as_float(w);
}

template <>
__device__ __forceinline__ float frag_get<__nv_bfloat16>(const Frag &f, int e) {
    const uint4 &q = f.v[e >> 3];
    const int i = (e >> 1) & 3;
    const uint32_t w = i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w;
    return (e & 1) ? bf16_hi(w) : bf16_lo(w);
}

// Element e of a fragment, e not known at compile time.
template <typename T>
__device__ __forceinline__ float frag_pick(const Frag &f, uint32_t e);

template <>
__device__ __forceinline__ float frag_pick<float>(const Frag &f, uint32_t e) {
    const uint4 q = e < 4u ? f.v[0] : f.v[1];
    const uint32_t i = e & 3u;
    return __uint_as_float(i == 0u ? q.x : i == 1u ? q.y : i == 2u ? q.z : q.w);
}

template <>
__device__ __forceinline__ float frag_pick<__nv_bfloat16>(const Frag &f, uint32_t e) {
    const uint4 q = e < 8u ? f.v[0] : f.v[1];
    const uint32_t i = (e >> 1) & 3u;
    const uint32_t w = i == 0u ? q.x : i == 1u ? q.y : i == 2u ? q.z : q.w;
    return (e & 1u) ? bf16_hi(w) : bf16_lo(w);
}

// The NaN-propagating maximum of the fragment's logits.
template <typename T>
__device__ __forceinline__ float frag_max(const Frag &f);

template <>
__device__ __forceinline__ float frag_max<float>(const Frag &f) {
    const float a = max_nan_f32(__uint_as_float(f.v[0].x), __uint_as_float(f.v[0].y));
    const float b = max_nan_f32(__uint_as_float(f.v[0].z), __uint_as_float(f.v[0].w));
    const float c = max_nan_f32(__uint_as_float(f.v[1].x), __uint_as_float(f.v[1].y));
    const float d = max_nan_f32(__uint_as_float(f.v[1].z), __uint_as_float(f.v[1].w));
    return max_nan_f32(max_nan_f32(a, b), max_nan_f32(c, d));
}

template <>
__device__ __forceinline__ float frag_max<__nv_bfloat16>(const Frag &f) {
    const uint32_t a = max_nan_bf16x2(f.v[0].x, f.v[0].y);
    const uint32_t b = max_nan_bf16x2(f.v[0].z, f.v[0].w);
    const uint32_t c = max_nan_bf16x2(f.v[1].x, f.v[1].y);
    const uint32_t d = max_nan_bf16x2(f.v[1].z, f.v[1].w);
    const uint32_t m = max_nan_bf16x2(max_nan_bf16x2(a, b), max_nan_bf16x2(c, d));
    return max_nan_f32(bf16_lo(m), bf16_hi(m));
}

__device__ __forceinline__ float widen(float x) { return x; }
__device__ __forceinline__ float widen(__nv_bfloat16 x) { return __bfloat162float(x); }

// Plain loads (any alignment) of the logits [base, base + GROUP) of a row;
// slots at or past `hi` zero.
template <typename T>
__device__ __forceinline__ void load_frag_scalar(Frag &f, const T *row, uint32_t base,
                                                 uint32_t hi) {
    constexpr int G = (int)Geo<T>::GROUP;
    f.v[0] = make_uint4(0, 0, 0, 0);
    f.v[1] = make_uint4(0, 0, 0, 0);
    uint32_t *words = reinterpret_cast<uint32_t *>(&f);
    if (sizeof(T) == 4) {
#pragma unroll
        for (int e = 0; e < G; ++e) {
            if (base + e < hi) {
                words[e] = __float_as_uint(widen(row[base + e]));
            }
        }
    } else {
        const uint16_t *r16 = reinterpret_cast<const uint16_t *>(row);
#pragma unroll
        for (int e = 0; e < G; ++e) {
            if (base + e < hi) {
                const uint32_t b = r16[base + e];
                words[e >> 1] |= (e & 1) ? (b << 16) : b;
            }
        }
    }
}

// Which of a fragment's logits beat the raw threshold (a NaN always does).
template <typename T>
__device__ __forceinline__ uint32_t pass_mask(const Frag &f, float c_raw);

template <>
__device__ __forceinline__ uint32_t pass_mask<float>(const Frag &f, float c_raw) {
    uint32_t m = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        m |= (!(frag_get<float>(f, e) <= c_raw) ? 1u : 0u) << e;
    }
    return m;
}

template <>
__device__ __forceinline__ uint32_t pass_mask<__nv_bfloat16>(const Frag &f, float c_raw) {
    // For a bf16 logit l: l > c  <=>  l > (the largest bf16 not above c), so
    // two logits are tested at a time against that value, unordered-greater
    // (a NaN on either side passes).
    uint32_t cb = __float_as_uint(c_raw);
    if (c_raw == c_raw) {
        const uint32_t low = cb & 0xFFFFu;
        cb &= 0xFFFF0000u;
        if ((cb >> 31) && low != 0u) {
            cb += 0x10000u;  // negative: truncation went up, step down
        }
    }
    const uint32_t c2 = (cb >> 16) | (cb & 0xFFFF0000u);
    const uint32_t w[8] = {f.v[0].x, f.v[0].y, f.v[0].z, f.v[0].w,
                           f.v[1].x, f.v[1].y, f.v[1].z, f.v[1].w};
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t d;
        asm("set.gtu.u32.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(w[i]), "r"(c2));
        m |= ((d & 1u) | ((d >> 15) & 2u)) << (2 * i);
    }
    return m;
}

// Pushes the logits of `pass` as raw bits; ids on the bias / ban list were
// handled up front and are skipped. Untouched logits also count in the
// tightening histogram. Returns the mask of elements the full buffer refused.
template <typename T>
__device__ __forceinline__ uint32_t push_masked(SmemFixed *sm, const RowCtx &c, const Frag &cur,
                                                const T *in_smem, uint32_t base, uint32_t pass) {
    uint32_t failed = 0;
    while (pass != 0u) {
        const uint32_t e = (uint32_t)__ffs(pass) - 1u;
        pass &= pass - 1u;
        // The fragment still sits in the thread's ring slot: one load picks
        // element e (without it: a chain of selects over the registers).
        const float l = in_smem != nullptr ? widen(in_smem[e]) : frag_pick<T>(cur, e);
        const uint32_t id = base + e;
        if (c.has_special && is_special(sm, c, id)) {
            continue;
        }
        if (!push(sm, __float_as_uint(l), id)) {
            failed |= 1u << e;
            continue;
        }
        // An untouched logit counts towards the next threshold. (A NaN never
        // does: its raw key is the highest, its adjusted key is not.)
        if (!(c.use_pen && seen_bit(c, id)) && l == l) {
            const uint32_t k16 = key_of(l) >> 16;
            const uint32_t b16 = sm->th_base;
            if (k16 >= b16) {
                atomicAdd(&sm->thist[min(k16 - b16, TH_BINS - 1u)], 1u);
                sm->th_new = 1;
            }
        }
    }
    return failed;
}

// One thread's logits of a round: those in `mask` that beat the raw
// threshold (or, when penalties may raise a logit, are in the history) are
// pushed. Returns the mask of elements the full buffer refused.
template <typename T>
__device__ __forceinline__ uint32_t process_frag(SmemFixed *sm, const RowCtx &c, const Frag &cur,
                                                 const T *in_smem, uint32_t base, uint32_t mask,
                                                 float c_raw, bool always_seen) {
    constexpr int G = (int)Geo<T>::GROUP;
    uint32_t pass = pass_mask<T>(cur, c_raw);
    if (always_seen) {
        const uint32_t off = base - c.lo;  // a multiple of GROUP: the bits sit in one word
        pass |= (c.seen[off >> 5] >> (off & 31u)) & ((1u << G) - 1u);
    }
    return push_masked<T>(sm, c, cur, in_smem, base, pass & mask);
}

// Block-wide: adjusts what the stream pushed, keeps the exact best k and
// raises the threshold to the k-th key.
__device__ __noinline__ void compact(SmemFixed *sm) {
    adjust_pending(sm);
    const uint32_t n = min(sm->n, CAP);
    const uint32_t k = sm->ctx.k;
    if (n > k) {
        select_topk(sm, n, k);
        if (threadIdx.x == 0) {
            set_exact_threshold(sm, sm->tau_key);
        }
    }
    if (threadIdx.x == 0) {
        sm->overflow = 0;
    }
    __syncthreads();
}

// ---- The two lean passes of the small-k route, out of line: each gets a
// register allocation of its own instead of sharing the big kernel's.

constexpr uint32_t ROUND_BYTES = NT * FRAG_BYTES;  // one round of logits, either type

struct Pass1 {
    float best;        // the thread's largest logit over its full rounds
    uint32_t best_r;   // the round it came from (0xFFFFFFFF: no full round)
    uint32_t saw_nan;
};

__device__ __forceinline__ void lean_copy_round(uint32_t dst, const char *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + 16u), "l"(src + 16) : "memory");
}

__device__ __forceinline__ void lean_read_slot(uint32_t at, Frag &f) {
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(f.v[0].x), "=r"(f.v[0].y), "=r"(f.v[0].z), "=r"(f.v[0].w)
                 : "r"(at));
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(f.v[1].x), "=r"(f.v[1].y), "=r"(f.v[1].z), "=r"(f.v[1].w)
                 : "r"(at + 16u));
}

__device__ __forceinline__ void lean_write_slot(uint32_t at, const Frag &f) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(f.v[0].x), "r"(f.v[0].y),
                 "r"(f.v[0].z), "r"(f.v[0].w)
                 : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at + 16u), "r"(f.v[1].x), "r"(f.v[1].y),
                 "r"(f.v[1].z), "r"(f.v[1].w)
                 : "memory");
}

// Pass 1 over the full rounds of a 16-byte aligned row: four rounds in
// flight (stages 0, 1 at slot_a, 2, 3 at slot_b; rounds 0..2 are already on
// their way), and (fused4 != 0) four history ids per thread and round marked
// in the seen bitmap of [lo, lo + width).
//
// Per thread it keeps the fragment with the largest logit (left in the
// thread's stage-1 slot at the end), the rounds and maxima of the second and
// third best fragments and the maximum over all the others (left at `tab`:
// m2, m3, m4, r2 | r3 << 16): pass 2 then needs the row again only where a
// second or further fragment of a thread also beats the threshold.
template <typename T>
__device__ __noinline__ Pass1 lean_pass1(uint32_t slot_a, uint32_t slot_b, const char *src0, uint32_t nfull,
                                         const uint4 *h4, uint32_t fused4, uint32_t *seen, uint32_t lo,
                                         uint32_t width, uint32_t tab) {
    constexpr uint32_t NONE = 0xFFFFFFFFu;
    const uint32_t tid = threadIdx.x;
    Pass1 out;
    out.best = neg_inf();
    out.best_r = NONE;
    out.saw_nan = 0u;
    float m2 = neg_inf(), m3 = neg_inf(), m4 = neg_inf();
    uint32_t r2 = NONE, r3 = NONE;
    Frag keep;
    keep.v[0] = make_uint4(0, 0, 0, 0);
    keep.v[1] = make_uint4(0, 0, 0, 0);
    const uint4 no_ids = make_uint4(NONE, NONE, NONE, NONE);
    uint4 hq = tid < fused4 ? __ldg(h4 + tid) : no_ids;
    const char *src = src0 + 3u * ROUND_BYTES;  // the round three ahead
    uint32_t hnext = NT + tid;
    for (uint32_t r = 0; r < nfull; r += 4u) {
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) {
            const uint32_t rr = r + j;
            if (rr < nfull) {
                if (rr + 3u < nfull) {
                    const uint32_t st = (j + 3u) & 3u;
                    lean_copy_round((st < 2u ? slot_a : slot_b) + (st & 1u) * ROUND_BYTES, src);
                }
                cp_async_commit();
                src += ROUND_BYTES;
                cp_async_wait<3>();
                Frag cur;
                lean_read_slot((j < 2u ? slot_a : slot_b) + (j & 1u) * ROUND_BYTES, cur);
                if (fused4 != 0u) {
                    const uint4 h = hq;
                    hq = hnext < fused4 ? __ldg(h4 + hnext) : no_ids;
                    hnext += NT;
                    const uint32_t ids[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t off = ids[i] - lo;
                        if (off < width) {
                            atomicOr(&seen[off >> 5], 1u << (off & 31u));
                        }
                    }
                }
                const float m = frag_max<T>(cur);
                out.saw_nan |= m != m ? 1u : 0u;
                // The three best fragments by maximum (rounds r1, r2, r3) and the
                // largest maximum among all the others (m4).
                if (out.best_r == NONE || m > out.best) {
                    m4 = fmaxf(m4, m3);
                    m3 = m2;
                    r3 = r2;
                    m2 = out.best;
                    r2 = out.best_r;
                    out.best = m;
                    out.best_r = rr;
                    keep = cur;
                } else if (r2 == NONE || m > m2) {
                    m4 = fmaxf(m4, m3);
                    m3 = m2;
                    r3 = r2;
                    m2 = m;
                    r2 = rr;
                } else if (r3 == NONE || m > m3) {
                    m4 = fmaxf(m4, m3);
                    m3 = m;
                    r3 = rr;
                } else {
                    m4 = fmaxf(m4, m);
                }
            }
        }
    }
    cp_async_wait<0>();
    lean_write_slot(slot_a + ROUND_BYTES, keep);
    // Rounds fit 16 bits (a slice has at most 2^24 / 4096 of them); 0xFFFF = none.
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(tab), "r"(__float_as_uint(m2)),
                 "r"(__float_as_uint(m3)), "r"(__float_as_uint(m4)), "r"((r2 & 0xFFFFu) | (r3 << 16))
                 : "memory");
    return out;
}

// The logits of one thread's fragment that beat the fixed threshold go to the
// candidate buffer as raw bits (ids on the bias / ban lists went in up front).
template <typename T>
__device__ __forceinline__ void lean_take(SmemFixed *sm, const Frag &cur, uint32_t base, uint32_t valid,
                                       float c_fix) {
    const RowCtx &c = sm->ctx;
    uint32_t pass = pass_mask<T>(cur, c_fix) & valid;
    while (pass != 0u) {
        const uint32_t e = (uint32_t)__ffs(pass) - 1u;
        pass &= pass - 1u;
        const uint32_t id = base + e;
        if (c.has_special && is_special(sm, c, id)) {
            continue;
        }
        push(sm, __float_as_uint(frag_pick<T>(cur, e)), id);  // a full buffer raises the overflow flag
    }
}

// Pass 2 over the full rounds of a 16-byte aligned row, from what pass 1
// left: the thread's best fragment (round r1, in its stage-1 slot) needs no
// memory at all; its second and third best (rounds r2, r3) are read again,
// both at once, only if they beat the threshold too; only if a fourth
// fragment could (m4) does the thread walk its rounds once more.
// Returns which of the steps the thread took (bit 0: second fragment read,
// bit 1: third, bit 2: the walk over all rounds), for the phase trace.
template <typename T>
__device__ __noinline__ uint32_t lean_pass2(SmemFixed *sm, const char *src0, uint32_t nfull, uint32_t base0,
                                            float c_fix, uint32_t slot_keep, uint32_t tab, float m1,
                                            uint32_t r1) {
    constexpr uint32_t NONE = 0xFFFFFFFFu;
    if (r1 == NONE) {
        return 0u;
    }
    uint32_t m2b, m3b, m4b, rr23;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(m2b), "=r"(m3b), "=r"(m4b), "=r"(rr23) : "r"(tab));
    const float m2 = __uint_as_float(m2b), m3 = __uint_as_float(m3b), m4 = __uint_as_float(m4b);
    const uint32_t r2 = (rr23 & 0xFFFFu) == 0xFFFFu ? NONE : (rr23 & 0xFFFFu);
    const uint32_t r3 = (rr23 >> 16) == 0xFFFFu ? NONE : (rr23 >> 16);
    const uint4 *src = reinterpret_cast<const uint4 *>(src0);
    constexpr uint32_t STRIDE = ROUND_BYTES / 16u;
    const bool second = r2 != NONE && !(m2 <= c_fix);
    const bool third = r3 != NONE && !(m3 <= c_fix);
    Frag f2, f3;
    if (second) {
        f2.v[0] = __ldcg(src + r2 * STRIDE);
        f2.v[1] = __ldcg(src + r2 * STRIDE + 1);
    }
    if (third) {
        f3.v[0] = __ldcg(src + r3 * STRIDE);
        f3.v[1] = __ldcg(src + r3 * STRIDE + 1);
    }
    if (!(m1 <= c_fix)) {
        Frag keep;
        lean_read_slot(slot_keep, keep);
        lean_take<T>(sm, keep, base0 + r1 * Geo<T>::ROUND, 0xFFFFFFFFu, c_fix);
    }
    if (second) {
        lean_take<T>(sm, f2, base0 + r2 * Geo<T>::ROUND, 0xFFFFFFFFu, c_fix);
    }
    if (third) {
        lean_take<T>(sm, f3, base0 + r3 * Geo<T>::ROUND, 0xFFFFFFFFu, c_fix);
    }
    if (!(m4 <= c_fix)) {
        // Very rare (a fourth fragment of this thread may matter): all rounds
        // again, four loads in flight at a time.
        for (uint32_t r0 = 0; r0 < nfull; r0 += 4u) {
            Frag f[4];
#pragma unroll
            for (uint32_t j = 0; j < 4u; ++j) {
                if (r0 + j < nfull) {
                    f[j].v[0] = __ldcg(src + (r0 + j) * STRIDE);
                    f[j].v[1] = __ldcg(src + (r0 + j) * STRIDE + 1);
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < 4u; ++j) {
                const uint32_t rr = r0 + j;
                if (rr < nfull && rr != r1 && rr != r2 && rr != r3 && !(frag_max<T>(f[j]) <= c_fix)) {
                    lean_take<T>(sm, f[j], base0 + rr * Geo<T>::ROUND, 0xFFFFFFFFu, c_fix);
                }
            }
        }
    }
    return (second ? 1u : 0u) | (third ? 2u : 0u) | (!(m4 <= c_fix) ? 4u : 0u);
}


// Phase stamps for the optional per-block timing trace.
enum { PH_START = 0, PH_BITMAPS, PH_LISTS, PH_STREAM, PH_LOCAL_SELECT, PH_MERGE, PH_SORT, PH_END,
       PH_FIRST_THRESHOLD, PH_PASS1, PH_PASS1_MET, PH_MAXIMA, PH_SEARCH, PH_THRESHOLD_SET, PH_SPARE0,
       PH_SPARE1, PH_ENTRY };


#define LILY_STAMP(phase)                                                                  \
    do {                                                                                   \
        if (a.phase_clocks != nullptr && threadIdx.x == 0) {                               \
            a.phase_clocks[((uint64_t)row * MAX_SLICES + blockIdx.x) * LILY_PHASES + (phase)] = \
                global_ns();                                                               \
        }                                                                                  \
    } while (0)

// One slice (thread block) of one row. `row` indexes every per-row array.
template <typename T, bool VEC>
__device__ __forceinline__ void sample_row(const KArgs &a, const uint32_t row, const uint32_t slice) {
    extern __shared__ uint4 smem_raw[];
    SmemFixed *sm = reinterpret_cast<SmemFixed *>(smem_raw);
    uint4 *ring = reinterpret_cast<uint4 *>(sm + 1);
    uint32_t *seen = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(ring) + RING_BYTES);

    const uint32_t tid = threadIdx.x;
    const uint32_t out_row = row;
    LILY_STAMP(PH_ENTRY);

    // What needs no input is done first: when the launch carries the
    // programmatic-serialisation attribute, the blocks of this grid start while
    // the previous kernel of the stream is still finishing, and wait below for
    // its memory before they read anything. (Without the attribute the two
    // instructions do nothing.)
    const bool whole_row_seen = a.n_slices == 1u;  // the block's slice is the whole row: the bitmap's size is known
    if (tid < BLOOM_WORDS) {
        sm->bloom[tid] = 0;
    }
    for (uint32_t b = tid; b < TH_BINS; b += NT) {
        sm->thist[b] = 0;
    }
    if (whole_row_seen) {
        const uint32_t words = (a.vocab + 31u) >> 5;
        for (uint32_t w = tid; w < words; w += NT) {
            seen[w] = 0;
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Everything the block has to know about its row is asked for first, in
    // one go: these few loads would otherwise queue behind the first rounds of
    // logits that every block of the launch asks for below.
    const uint32_t hist_len_row = (a.history_ids && a.history_len) ? __ldg(a.history_len + row) : 0u;
    const int32_t forced = a.forced_ids ? __ldg(a.forced_ids + row) : -1;
    const uint32_t bias_len_row = (a.bias_ids && a.bias_len) ? __ldg(a.bias_len + row) : 0u;
    const uint32_t ban_len_row = (a.ban_ids && a.ban_len) ? __ldg(a.ban_len + row) : 0u;
    const uint32_t slot_row = a.count_slots ? __ldg(a.count_slots + row) : 0u;
    const float u_row = a.uniforms ? __ldg(a.uniforms + row) : 0.0f;
    const uint32_t step_row = (!a.uniforms && a.steps) ? __ldg(a.steps + row) : 0u;
    lily_sampling_params_t P;
    if (a.force_greedy) {
        P.temperature = 0.0f;
        P.top_k = 1;
        P.top_p = 1.0f;
        P.min_p = 0.0f;
        P.presence_penalty = 0.0f;
        P.frequency_penalty = 0.0f;
        P.repetition_penalty = 1.0f;
        P.seed = 0;
    } else {
        // 40 bytes, 8-byte aligned: five 8-byte loads.
        const uint2 *pp = reinterpret_cast<const uint2 *>(a.params + row);
        const uint2 w0 = __ldg(pp), w1 = __ldg(pp + 1), w2 = __ldg(pp + 2), w3 = __ldg(pp + 3), w4 = __ldg(pp + 4);
        P.temperature = __uint_as_float(w0.x);
        P.top_k = w0.y;
        P.top_p = __uint_as_float(w1.x);
        P.min_p = __uint_as_float(w1.y);
        P.presence_penalty = __uint_as_float(w2.x);
        P.frequency_penalty = __uint_as_float(w2.y);
        P.repetition_penalty = __uint_as_float(w3.x);
        P.reserved = w3.y;
        P.seed = (uint64_t)w4.x | ((uint64_t)w4.y << 32);
    }
    // With one slice per row, where the logits are does not depend on the
    // row's parameters: the first three rounds are asked for before the
    // parameters have arrived (into the stages pass 1 reads them from).
    const bool early = VEC && a.n_slices == 1u && a.vocab >= 3u * Geo<T>::ROUND;
    if (early) {
        const char *src = reinterpret_cast<const char *>(reinterpret_cast<const T *>(a.logits) +
                                                         (uint64_t)row * a.logits_ld + tid * Geo<T>::GROUP);
        const uint32_t dst[3] = {(uint32_t)__cvta_generic_to_shared(ring) + tid * FRAG_BYTES,
                                 (uint32_t)__cvta_generic_to_shared(ring) + (NT + tid) * FRAG_BYTES,
                                 (uint32_t)__cvta_generic_to_shared(sm->key) + tid * FRAG_BYTES};
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            lean_copy_round(dst[j], src + (size_t)j * ROUND_BYTES);
            cp_async_commit();
        }
    }
    // ---- forced rows and parameters (uniform per block, before any barrier)
    if (forced >= 0) {
        if (slice == 0 && tid == 0) {
            a.out_ids[out_row] = (uint32_t)forced;
            if (a.out_status) {
                a.out_status[out_row] = LILY_ROW_FORCED;
            }
            if (a.kept_n) {
                a.kept_n[out_row] = 0;
            }
        }
        if (early) {
            cp_async_wait<0>();
        }
        return;
    }
    {
        // src/kernels/sample.rs:57-79, for parameters the host never saw.
        const bool fin = isfinite(P.temperature) && isfinite(P.top_p) && isfinite(P.min_p) &&
                         isfinite(P.repetition_penalty) && isfinite(P.presence_penalty) &&
                         isfinite(P.frequency_penalty);
        const bool ok = fin && P.temperature >= 0.0f && P.top_p > 0.0f && P.top_p <= 1.0f &&
                        P.min_p >= 0.0f && P.min_p <= 1.0f && P.repetition_penalty > 0.0f;
        if (!ok) {
            if (slice == 0 && tid == 0) {
                a.out_ids[out_row] = 0xFFFFFFFFu;
                if (a.out_status) {
                    a.out_status[out_row] = LILY_ROW_PARAMS;
                }
                if (a.kept_n) {
                    a.kept_n[out_row] = 0;
                }
                atomicOr(a.status_word, 1u << LILY_ROW_PARAMS);
            }
            if (early) {
                cp_async_wait<0>();
            }
            return;
        }
    }

    // A list length is a device value: one beyond what the handle was made for,
    // or beyond the row pitch, would walk into the next row or past the buffer.
    // (A pitch of 0 means one list shared by every row.)
    if (hist_len_row > a.max_history || (a.history_ld != 0u && hist_len_row > a.history_ld) ||
        bias_len_row > a.max_list || (a.bias_ld != 0u && bias_len_row > a.bias_ld) ||
        ban_len_row > a.max_list || (a.ban_ld != 0u && ban_len_row > a.ban_ld)) {
        if (slice == 0 && tid == 0) {
            a.out_ids[out_row] = 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[out_row] = LILY_ROW_LIST;
            }
            if (a.kept_n) {
                a.kept_n[out_row] = 0;
            }
            atomicOr(a.status_word, 1u << LILY_ROW_LIST);
        }
        if (early) {
            cp_async_wait<0>();
        }
        return;
    }

    RowCtx c;
    const bool greedy = P.temperature <= 0.0f || P.top_k == 1u;
    c.use_pen = P.presence_penalty != 0.0f || P.frequency_penalty != 0.0f ||
                P.repetition_penalty != 1.0f;
    c.T = greedy ? 1.0f : P.temperature;
    c.k = greedy ? 1u : (P.top_k == 0u ? KCAP : min(P.top_k, KCAP));
    if (a.cand_out && !greedy) {
        c.k = a.shard_k;  // the host made sure that top_k fits
    }
    c.rep = P.repetition_penalty;
    c.presence = P.presence_penalty;
    c.frequency = P.frequency_penalty;
    c.top_p = P.top_p;
    c.min_p = P.min_p;
    c.bias_len = bias_len_row;
    c.ban_len = ban_len_row;
    c.bias_ids = a.bias_ids ? a.bias_ids + (uint64_t)row * a.bias_ld : nullptr;
    c.bias_vals = a.bias_vals ? a.bias_vals + (uint64_t)row * a.bias_ld : nullptr;
    c.ban_ids = a.ban_ids ? a.ban_ids + (uint64_t)row * a.ban_ld : nullptr;
    c.has_special = (c.bias_len + c.ban_len) > 0u;
    c.sp_in_smem = (c.bias_len + c.ban_len) <= SP_SMEM;
    c.argmax_mode = greedy && !c.use_pen && !c.has_special;
    // Penalties that can only lower a logit let the raw threshold reject
    // seen ids without adjusting them.
    c.monotone = P.repetition_penalty >= 1.0f &&
                 !(__float_as_uint(P.presence_penalty) >> 31) &&
                 !(__float_as_uint(P.frequency_penalty) >> 31);
    c.need_counts = c.use_pen && P.frequency_penalty != 0.0f;
    // A row is cut into at most CAP / k slices so that the merge of the
    // slices' best k fits the candidate buffer; blocks past that leave.
    // (A row that keeps many candidates is not cut at all when it can take
    // the two-pass route: merging slices of a thousand candidates each costs
    // more than one block streaming the whole row.)
    const bool one_block = c.k > 128u && (!c.use_pen || c.monotone) && a.cand_out == nullptr;
    const uint32_t want = one_block ? 1u : min(a.n_slices, CAP / c.k);
    const uint32_t slice_len = (((a.vocab + want - 1u) / want) + 255u) & ~255u;
    const uint32_t n_slices = (a.vocab + slice_len - 1u) / slice_len;
    if (slice >= n_slices) {
        return;
    }
    c.lo = slice * slice_len;
    c.hi = min(a.vocab, c.lo + slice_len);
    c.seen = seen;
    const bool table_mode = a.count_slots != nullptr;
    const uint32_t slot = table_mode ? slot_row : 0u;
    uint32_t *counts_rw = nullptr;
    if (c.need_counts) {
        counts_rw = table_mode ? a.counts_table + (uint64_t)slot * a.vocab
                               : a.counts_scratch + (uint64_t)row * a.vocab;
    }
    c.counts = counts_rw;
    const uint32_t hist_len = (c.use_pen && !table_mode) ? hist_len_row : 0u;
    const uint32_t *hist = a.history_ids ? a.history_ids + (uint64_t)row * a.history_ld : nullptr;
    const uint32_t extra_len = (c.use_pen && !table_mode) ? a.extra_len : 0u;
    const T *row_ptr = reinterpret_cast<const T *>(a.logits) + (uint64_t)row * a.logits_ld;

    // The ring: STAGES rounds of this block's logits in flight, each thread
    // copying (and later reading back) its own 32 bytes.
    constexpr uint32_t GROUP = Geo<T>::GROUP;
    constexpr uint32_t ROUND = Geo<T>::ROUND;
    constexpr uint32_t RGROUP = Geo<T>::RGROUP;
    const uint32_t span = c.hi - c.lo;
    const uint32_t nrounds = (span + ROUND - 1u) / ROUND;
    const uint32_t nfull = span / ROUND;  // rounds in which every thread has all its logits
    const char *my_src = reinterpret_cast<const char *>(row_ptr + c.lo + tid * GROUP);
    auto issue = [&](uint32_t r) {
        uint4 *dst = &ring[((r % STAGES) * NT + tid) * 2u];
        if (VEC && r < nfull) {
            const char *src = my_src + (size_t)r * (ROUND * sizeof(T));
            cp_async_16(dst, src, 16u);
            cp_async_16(dst + 1, src + 16, 16u);
        } else if (VEC && r < nrounds) {
            const uint32_t base = c.lo + r * ROUND + tid * GROUP;
            const uint32_t left = base < c.hi ? (c.hi - base) * (uint32_t)sizeof(T) : 0u;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t off = 16u * i;
                const uint32_t bytes = left > off ? min(16u, left - off) : 0u;
                const char *src = bytes ? reinterpret_cast<const char *>(row_ptr + base) + off
                                        : reinterpret_cast<const char *>(row_ptr);
                cp_async_16(dst + i, src, bytes);
            }
        }
        cp_async_commit();
    };
    auto fetch = [&](uint32_t r, Frag &f) {
        if (VEC) {
            cp_async_wait<STAGES - 1>();
            const uint4 *src = &ring[((r % STAGES) * NT + tid) * 2u];
            f.v[0] = src[0];
            f.v[1] = src[1];
        } else {
            load_frag_scalar<T>(f, row_ptr, c.lo + r * ROUND + tid * GROUP, c.hi);
        }
    };
    if (!early) {
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            issue((uint32_t)st);
        }
    }
    // Small k with penalties that only lower a logit takes two passes over
    // the slice (see C0' below). Its first pass is the one that reads DRAM:
    // it runs four rounds deep, the two extra stages in the still unused
    // candidate buffer (key[] and id[] are one round each).
    // Up to k = 128 the threshold comes from one maximum per thread; beyond
    // that ("wide", up to the cap of 1024) from each thread's three best
    // fragments, which needs aligned rows and three full rounds per thread.
    const bool lean_wide = c.k > 128u;
    const bool lean_cand = (!c.use_pen || c.monotone) && nrounds > 0u &&
                           (!lean_wide || (VEC && nfull >= 3u && c.k <= 3u * NT));
    constexpr int P1_STAGES = 4;
    static_assert(STAGES == 2 && CAP * 4u == NT * FRAG_BYTES, "pass 1 stages 2 and 3 are key[] and id[]");
    const uint32_t p1_slot[P1_STAGES] = {
        (uint32_t)__cvta_generic_to_shared(ring) + tid * FRAG_BYTES,
        (uint32_t)__cvta_generic_to_shared(ring) + (NT + tid) * FRAG_BYTES,
        (uint32_t)__cvta_generic_to_shared(sm->key) + tid * FRAG_BYTES,
        (uint32_t)__cvta_generic_to_shared(sm->id) + tid * FRAG_BYTES};
    // Each thread's 16 bytes of pass 1 -> pass 2 state sit in tkey[] / tid[],
    // idle until the selection at the very end.
    static_assert(2u * KCAP * 4u >= NT * 16u, "tkey and tid hold 16 bytes per thread");
    const uint32_t lean_tab = (uint32_t)__cvta_generic_to_shared(sm->tkey) + tid * 16u;
    auto p1_issue = [&](uint32_t r) {  // full rounds only; always one commit
        if (r < nfull) {
            const char *src = my_src + (size_t)r * (ROUND * sizeof(T));
            const uint32_t dst = p1_slot[r % P1_STAGES];
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + 16u), "l"(src + 16)
                         : "memory");
        }
        cp_async_commit();
    };
    if (VEC && lean_cand && !early) {
#pragma unroll
        for (int st = STAGES - 1; st < P1_STAGES - 1; ++st) {
            p1_issue((uint32_t)st);
        }
    }
    // The slice's last, partial round (plain loads: it may end anywhere) is
    // asked for now and used at the end of pass 1 and again in pass 2: its
    // latency hides behind everything in between.
    Frag part;
    part.v[0] = make_uint4(0, 0, 0, 0);
    part.v[1] = make_uint4(0, 0, 0, 0);
    const uint32_t part_base = c.lo + nfull * ROUND + tid * GROUP;
    const uint32_t part_valid = (lean_cand && nrounds > nfull && part_base < c.hi)
                                    ? min(GROUP, c.hi - part_base)
                                    : 0u;
    if (part_valid != 0u) {
        load_frag_scalar<T>(part, row_ptr, part_base, c.hi);
    }

    // ---- A. bitmaps
    const uint32_t slice_words = (c.hi - c.lo + 31u) >> 5;
    // One unsigned compare covers both ends of the slice. Real histories
    // repeat a few ids very often: the atomic is skipped when the bit is
    // already up.
    auto mark = [&](uint32_t id) {
        const uint32_t off = id - c.lo;
        if (off < c.hi - c.lo) {
            const uint32_t bit = 1u << (off & 31u);
            uint32_t *word = &seen[off >> 5];
            if (!(*reinterpret_cast<volatile uint32_t *>(word) & bit)) {
                atomicOr(word, bit);
            }
        }
    };
    // The first part of a plain history list is marked inside pass 1, one
    // 16-byte load per thread and round, hidden behind the logits' latency.
    const bool hist_vec = (reinterpret_cast<uintptr_t>(hist) & 15u) == 0u;
    const uint32_t fused4 = (VEC && lean_cand && hist_vec && !c.need_counts && hist_len > 0u)
                                ? min(hist_len / 4u, nfull * (uint32_t)NT)
                                : 0u;
    if (tid == 0) {
        sm->ctx = c;
        sm->n = 0;
        sm->n_adj = 0;
        sm->err = 0;
        sm->tau_key = 0;
        sm->kstar = 0;
        sm->c_raw = __uint_as_float(0x7FC00000u);
        sm->th_base = 0;
        sm->th_new = 0;
        sm->overflow = 0;
        sm->ckey = sm->key;
        sm->cid = sm->id;
        sm->ccap = CAP;
        sm->u_draw = a.uniforms ? u_row : uniform_for(P.seed, step_row);
        sm->lean_abort = 0;
    }
    if (c.use_pen) {
        if (table_mode) {
            const uint32_t *src = a.seen_table + (uint64_t)slot * a.seen_words + (c.lo >> 5);
            for (uint32_t w = tid; w < slice_words; w += NT) {
                seen[w] = src[w];
            }
        } else if (!whole_row_seen) {
            for (uint32_t w = tid; w < slice_words; w += NT) {
                seen[w] = 0;
            }
        }
    }
    __syncthreads();
    LILY_STAMP(PH_START);
    if (hist_len + extra_len > 0u) {
        const uint32_t lo = c.lo;
        const uint32_t width = c.hi - c.lo;
        // With the frequency penalty the multiplicities go to the row's
        // count table as well: one global atomic per distinct id of the warp.
        auto mark_count = [&](uint32_t id) {
            const uint32_t off = id - lo;
            const bool mine = off < width;
            const unsigned live = __ballot_sync(0xFFFFFFFFu, mine);
            if (mine) {
                const uint32_t bit = 1u << (off & 31u);
                uint32_t *word = &seen[off >> 5];
                if (!(*reinterpret_cast<volatile uint32_t *>(word) & bit)) {
                    atomicOr(word, bit);
                }
                const unsigned peers = __match_any_sync(live, id);
                if ((tid & 31u) == (uint32_t)(__ffs(peers) - 1)) {
                    atomicAdd(counts_rw + id, (uint32_t)__popc(peers));
                }
            }
        };
        // The bulk of the list in 16-byte loads, four in flight per thread.
        const uint32_t n4 = hist_vec ? hist_len / 4u : 0u;
        const uint4 *h4 = reinterpret_cast<const uint4 *>(hist);
        constexpr int HB = 4;
        for (uint32_t i0 = fused4; i0 < n4; i0 += NT * HB) {
            uint4 q[HB];
#pragma unroll
            for (int j = 0; j < HB; ++j) {
                const uint32_t i = i0 + (uint32_t)j * NT + tid;
                q[j] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
                if (i < n4) {
                    q[j] = __ldg(h4 + i);
                }
            }
            if (c.need_counts) {
#pragma unroll
                for (int j = 0; j < HB; ++j) {
                    mark_count(q[j].x);
                    mark_count(q[j].y);
                    mark_count(q[j].z);
                    mark_count(q[j].w);
                }
            } else {
#pragma unroll
                for (int j = 0; j < HB; ++j) {
                    mark(q[j].x);
                    mark(q[j].y);
                    mark(q[j].z);
                    mark(q[j].w);
                }
            }
        }
        const uint32_t total = hist_len + extra_len;
        for (uint32_t i0 = n4 * 4u; i0 < total; i0 += NT) {
            const uint32_t i = i0 + tid;
            uint32_t id = 0xFFFFFFFFu;
            if (i < total) {
                id = i < hist_len ? hist[i] : a.extra_ids[i - hist_len];
            }
            if (c.need_counts) {
                mark_count(id);
            } else {
                mark(id);
            }
        }
    }
    if (c.has_special) {
        const uint32_t n_sp = c.bias_len + c.ban_len;
        for (uint32_t j = tid; j < n_sp; j += NT) {
            const uint32_t id = j < c.bias_len ? c.bias_ids[j] : c.ban_ids[j - c.bias_len];
            atomicOr(&sm->bloom[(id >> 5) & (BLOOM_WORDS - 1u)], 1u << (id & 31u));
            if (c.sp_in_smem) {
                sm->sp_ids[j] = id;
                sm->sp_vals[j] = j < c.bias_len ? c.bias_vals[j] : 0.0f;
            }
        }
        if (c.sp_in_smem && tid < 4u) {
            sm->sp_ids[n_sp + tid] = 0xFFFFFFFFu;
        }
    }
    __syncthreads();
    LILY_STAMP(PH_BITMAPS);

    // ---- C0'. small k, penalties that only lower: two passes over the slice
    // Pass 1 keeps each thread's largest logit (one packed max per round).
    // The adjusted values of those 512 logits are values of 512 different
    // ids, so their k-th largest cannot exceed the k-th largest adjusted
    // value of the slice: an exact, tight threshold before any logit is
    // looked at closely. Pass 2 (after the lists, below) streams the slice
    // again, from L2 this time, against that fixed threshold.
    bool lean = lean_cand;
    float full_best = neg_inf();           // pass 1's result over the full rounds, for pass 2
    uint32_t full_best_r = 0xFFFFFFFFu;
    if (lean) {
        constexpr uint32_t NONE = 0xFFFFFFFFu;
        float best = neg_inf();
        uint32_t best_r = NONE;
        bool saw_nan = false;
        {
            if (VEC) {
                const Pass1 p1 = lean_pass1<T>(p1_slot[0], p1_slot[2], my_src, nfull,
                                               reinterpret_cast<const uint4 *>(hist), fused4, seen, c.lo,
                                               c.hi - c.lo, lean_tab);
                best = p1.best;
                best_r = p1.best_r;
                saw_nan = p1.saw_nan != 0u;
                full_best = p1.best;
                full_best_r = p1.best_r;
            } else {
                for (uint32_t r = 0; r < nfull; ++r) {
                    Frag cur;
                    load_frag_scalar<T>(cur, row_ptr, c.lo + r * ROUND + tid * GROUP, c.hi);
                    const float m = frag_max<T>(cur);
                    saw_nan = saw_nan || m != m;
                    if (best_r == NONE || m > best) {
                        best = m;
                        best_r = r;
                    }
                }
            }
            if (part_valid != 0u) {
#pragma unroll
                for (int e = 0; e < (int)GROUP; ++e) {
                    if ((uint32_t)e < part_valid) {
                        const float l = frag_get<T>(part, e);
                        saw_nan = saw_nan || l != l;
                        if (best_r == NONE || l > best) {
                            best = l;
                            best_r = nfull;
                        }
                    }
                }
            }
            cp_async_wait<0>();
        }
        LILY_STAMP(PH_PASS1);
        // A NaN anywhere, or fewer than k threads with a logit: the general path.
        const uint32_t have = (uint32_t)__syncthreads_count(best_r != NONE) * (lean_wide ? 3u : 1u);
        lean = !__syncthreads_or(saw_nan) && have >= c.k;
        LILY_STAMP(PH_PASS1_MET);
        if (lean) {
            uint32_t key = 0u, id = NONE;
            if (best_r != NONE) {
                // Which logit of that round it was: pass 1 kept the fragment.
                Frag again;
                const uint32_t base = c.lo + best_r * ROUND + tid * GROUP;
                if (best_r == nfull) {
                    again = part;
                } else if (VEC) {
                    lean_read_slot(p1_slot[1], again);
                } else {
                    load_frag_scalar<T>(again, row_ptr, base, c.hi);
                }
                const uint32_t nvalid = min(GROUP, c.hi - base);
                uint32_t at = 0;
                float l = best;
#pragma unroll
                for (int e = (int)GROUP - 1; e >= 0; --e) {
                    const float v = frag_get<T>(again, e);
                    if ((uint32_t)e < nvalid && v == best) {
                        at = (uint32_t)e;
                        l = v;
                    }
                }
                id = base + at;
                key = adjusted_key(sm, id, l, c.has_special && is_special(sm, c, id));
            }
            // Wide: the largest logits of the thread's second and third best
            // fragments as well (other fragments, so other ids: still a lower
            // bound). Their rounds are read once more to find the ids.
            uint32_t key2 = 0u, key3 = 0u;
            if (lean_wide) {
                uint32_t m2b, m3b, m4b, rr23;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(m2b), "=r"(m3b), "=r"(m4b), "=r"(rr23)
                             : "r"(lean_tab));
                const uint32_t rr[2] = {rr23 & 0xFFFFu, rr23 >> 16};
                const float mm[2] = {__uint_as_float(m2b), __uint_as_float(m3b)};
                Frag f[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(my_src + (size_t)rr[j] * ROUND_BYTES);
                    f[j].v[0] = __ldcg(src);
                    f[j].v[1] = __ldcg(src + 1);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t at = 0;
                    float l = mm[j];
#pragma unroll
                    for (int e = (int)GROUP - 1; e >= 0; --e) {
                        const float v = frag_get<T>(f[j], e);
                        if (v == mm[j]) {
                            at = (uint32_t)e;
                            l = v;
                        }
                    }
                    const uint32_t id2 = c.lo + rr[j] * ROUND + tid * GROUP + at;
                    const uint32_t kk = adjusted_key(sm, id2, l, c.has_special && is_special(sm, c, id2));
                    if (j == 0) {
                        key2 = kk;
                    } else {
                        key3 = kk;
                    }
                }
            }
            LILY_STAMP(PH_MAXIMA);
            // The largest v (low 16 bits clear) that at least k of the keys
            // reach, bit by bit from the top: a block-wide count per bit.
            uint32_t kth = 0u;
            if (!lean_wide) {
#pragma unroll 1
                for (int bit = 31; bit >= 16; --bit) {
                    const uint32_t cand = kth | (1u << bit);
                    if ((uint32_t)__syncthreads_count(key >= cand) >= c.k) {
                        kth = cand;
                    }
                }
            } else {
                // Three keys per thread: warp sums into three rotating counters,
                // one barrier per bit.
                uint32_t *ctr = &sm->sel_digit;  // sel_digit, sel_before, sel_count
                if (tid < 3u) {
                    ctr[tid] = 0u;
                }
                __syncthreads();
#pragma unroll 1
                for (int bit = 31, it = 0; bit >= 16; --bit, ++it) {
                    const uint32_t cand = kth | (1u << bit);
                    const uint32_t mine = (key >= cand ? 1u : 0u) + (key2 >= cand ? 1u : 0u) +
                                          (key3 >= cand ? 1u : 0u);
                    const uint32_t warp_sum = __reduce_add_sync(0xFFFFFFFFu, mine);
                    if ((tid & 31u) == 0u && warp_sum != 0u) {
                        atomicAdd(&ctr[it % 3], warp_sum);
                    }
                    __syncthreads();
                    if (*reinterpret_cast<volatile uint32_t *>(&ctr[it % 3]) >= c.k) {
                        kth = cand;
                    }
                    if (tid == 0) {
                        ctr[(it + 2) % 3] = 0u;  // next used two barriers from now
                    }
                }
            }
            LILY_STAMP(PH_SEARCH);
            if (tid == 0) {
                // Ties with the k-th value must still pass: one key below it.
                set_exact_threshold(sm, kth > 0u ? kth - 1u : 0u);
            }
            __syncthreads();
            LILY_STAMP(PH_THRESHOLD_SET);
        }
        if (!lean) {
            // The general path follows: its ring starts over at round 0.
#pragma unroll
            for (int st = 0; st < STAGES - 1; ++st) {
                issue((uint32_t)st);
            }
        }
    }

    // ---- C0. (general path) the first round: a threshold from a fine histogram
    // The candidate buffer is still empty: its storage holds an 8192-bin
    // histogram of the raw keys of the round's untouched logits. The bin in
    // which the count from the top reaches k gives the first threshold.
    Frag first;
    if (!lean) {
    if (early) {
        // Round 2 was copied into key[] ahead of time: it must have landed, in
        // every thread, before the histogram takes that storage.
        cp_async_wait<0>();
        __syncthreads();
    }
    issue((uint32_t)(STAGES - 1));
    uint32_t *hist0 = sm->key;
    for (uint32_t b = tid; b < H0_BINS; b += NT) {
        hist0[b] = 0;
    }
    __syncthreads();
    fetch(0u, first);
    {
        const uint32_t base0 = c.lo + tid * GROUP;
        const uint32_t nvalid0 = base0 < c.hi ? min(GROUP, c.hi - base0) : 0u;
        // Which of the thread's logits are touched (in the history, or
        // possibly on the bias / ban list: the bloom filter, no list scan).
        uint32_t touched = 0;
        if (c.use_pen && nvalid0 > 0u) {
            const uint32_t off = base0 - c.lo;
            touched = (seen[off >> 5] >> (off & 31u)) & ((1u << GROUP) - 1u);
        }
        if (c.has_special) {
#pragma unroll
            for (int e = 0; e < (int)GROUP; ++e) {
                const uint32_t id = base0 + e;
                touched |= ((sm->bloom[(id >> 5) & (BLOOM_WORDS - 1u)] >> (id & 31u)) & 1u) << e;
            }
        }
        if (c.k <= 128u) {
            // Small k: the k-th largest of the 512 per-thread maxima (over
            // untouched logits) is nearly the k-th largest logit, and costs
            // one histogram update per thread instead of one per logit.
            float best = neg_inf();
            bool any = false;
#pragma unroll
            for (int e = 0; e < (int)GROUP; ++e) {
                if ((uint32_t)e < nvalid0 && !((touched >> e) & 1u)) {
                    // A NaN never counts: its raw key is the highest, its
                    // adjusted key is not (an error row, or never the argmax).
                    const float l = frag_get<T>(first, e);
                    if (l == l) {
                        best = any ? fmaxf(best, l) : l;
                        any = true;
                    }
                }
            }
            if (any) {
                atomicAdd(&hist0[key_of(best) >> H0_SHIFT], 1u);
            }
        } else {
#pragma unroll
            for (int e = 0; e < (int)GROUP; ++e) {
                const float l = frag_get<T>(first, e);
                if ((uint32_t)e < nvalid0 && !((touched >> e) & 1u) && l == l) {
                    atomicAdd(&hist0[key_of(l) >> H0_SHIFT], 1u);
                }
            }
        }
    }
    __syncthreads();
    find_bin<H0_BINS / NT>(sm, hist0, H0_BINS, c.k, true);  // sets sel_digit if k untouched logits exist
    uint32_t edge0 = 0;
    {
        // The total is below k when find_bin found no bin: then no threshold.
        uint32_t total = 0;
        for (uint32_t w = 0; w < NT / 32; ++w) {
            total += sm->warp_sums[w];
        }
        if (total >= c.k) {
            edge0 = sm->sel_digit << H0_SHIFT;
        }
    }
    __syncthreads();  // the histogram is read: its storage becomes the buffer again
    if (tid == 0) {
        sm->th_base = edge0 >> 16;
        set_raw_edge(sm, edge0);
    }
    }  // !lean
    LILY_STAMP(PH_FIRST_THRESHOLD);

    // ---- B. ids on the bias / ban lists, each once (adjusted right away)
    if (c.has_special) {
        const uint32_t n_sp = c.bias_len + c.ban_len;
        for (uint32_t j = tid; j < n_sp; j += NT) {
            const uint32_t id = j < c.bias_len ? c.bias_ids[j] : c.ban_ids[j - c.bias_len];
            if (id < c.lo || id >= c.hi) {
                continue;
            }
            bool first_of_id = true;
            for (uint32_t e = 0; e < j && first_of_id; ++e) {
                const uint32_t other = c.sp_in_smem
                                           ? sm->sp_ids[e]
                                           : (e < c.bias_len ? c.bias_ids[e] : c.ban_ids[e - c.bias_len]);
                first_of_id = other != id;
            }
            if (first_of_id) {
                const uint32_t key = adjusted_key(sm, id, widen(row_ptr[id]), true);
                push(sm, key, id);
            }
        }
        __syncthreads();
        if (tid == 0) {
            sm->n_adj = min(sm->n, CAP);
        }
    }
    __syncthreads();
    LILY_STAMP(PH_LISTS);

    // ---- C'. pass 2 of the two-pass route: the fixed threshold, no meetings
    if (lean) {
        const uint32_t n_lists = min(sm->n, CAP);  // what the lists pushed
        const float c_fix = sm->c_raw;
        {
            uint32_t base = c.lo + tid * GROUP;
            if (VEC) {
                (void)lean_pass2<T>(sm, my_src, nfull, base, c_fix, p1_slot[1], lean_tab, full_best, full_best_r);
                base += nfull * ROUND;
            } else {
                for (uint32_t r = 0; r < nfull; ++r) {
                    Frag cur;
                    load_frag_scalar<T>(cur, row_ptr, base, c.hi);
                    if (!(frag_max<T>(cur) <= c_fix)) {
                        lean_take<T>(sm, cur, base, 0xFFFFFFFFu, c_fix);
                    }
                    base += ROUND;
                }
            }
            if (part_valid != 0u) {
                lean_take<T>(sm, part, part_base, (1u << part_valid) - 1u, c_fix);
            }
            cp_async_wait<0>();
        }
        if (__syncthreads_or(*reinterpret_cast<volatile uint32_t *>(&sm->overflow))) {
            // More logits tie with the threshold than the buffer holds: start the
            // stream over on the general path, which makes room as it goes.
            if (tid == 0) {
                sm->n = n_lists;
                sm->n_adj = n_lists;
                sm->overflow = 0;
                sm->ckey = sm->key;
                sm->cid = sm->id;
                sm->ccap = CAP;
            }
            lean = false;
#pragma unroll
            for (int st = 0; st < STAGES - 1; ++st) {
                issue((uint32_t)st);
            }
            issue((uint32_t)(STAGES - 1));
            fetch(0u, first);
            __syncthreads();
        }
    }

    // ---- C. the stream (general path)
    if (!lean) {
    // Rounds run without block barriers. Every RGROUP rounds the block meets:
    // if a push found the buffer full, the buffer is cut back to the best k
    // and the refused elements of those rounds are offered again (re-read
    // from global memory). After those meetings, on a thinning schedule, one
    // warp (a different one each time) tightens the threshold.
    const bool always_seen = c.use_pen && !c.monotone;  // penalties may raise a seen logit
    uint32_t dropped = 0;  // GROUP refused-element bits per round of the group
    float c_raw = sm->c_raw;
    auto look = [&](const Frag &cur, uint32_t r, uint32_t base, bool full) {
        // A thread looks closer when its largest logit beats the threshold (in
        // a partial round: when it holds any logit at all).
        c_raw = *reinterpret_cast<volatile float *>(&sm->c_raw);
        bool hit = full ? !(frag_max<T>(cur) <= c_raw) : base < c.hi;
        if (always_seen && !hit && full) {
            const uint32_t off = base - c.lo;
            hit = ((seen[off >> 5] >> (off & 31u)) & ((1u << GROUP) - 1u)) != 0u;
        }
        if (hit) {
            const uint32_t nvalid = min(GROUP, c.hi - base);
            const uint32_t valid = nvalid >= 32u ? 0xFFFFFFFFu : (1u << nvalid) - 1u;
            const T *slot = VEC ? reinterpret_cast<const T *>(&ring[((r % STAGES) * NT + tid) * 2u])
                                : nullptr;
            dropped |= process_frag<T>(sm, c, cur, slot, base, valid, c_raw, always_seen)
                       << (GROUP * (r % RGROUP));
        }
    };
    auto meet = [&](uint32_t r) {
        // End of a group of rounds (r is its last round).
        const uint32_t g0 = r - (r % RGROUP);
        const uint32_t g = r / RGROUP;
        if (__syncthreads_or(*reinterpret_cast<volatile uint32_t *>(&sm->overflow))) {
            compact(sm);
            // What is left to offer fits at once when the refused elements
            // are fewer than the room the selection made; otherwise one
            // element per thread at a time, with room made in between.
            if (tid == 0) {
                sm->cnt = 0;
            }
            __syncthreads();
            atomicAdd(&sm->cnt, (uint32_t)__popc(dropped));
            __syncthreads();
            const bool at_once = sm->n + sm->cnt <= CAP;
            for (uint32_t b = 0; b < 32u; ++b) {
                const bool mine = (dropped >> b) & 1u;
                if (!at_once) {
                    if (!__syncthreads_or(mine)) {
                        continue;
                    }
                    // Nobody pushes between the two barriers: every thread
                    // reads the same count and takes the same branch.
                    if (__syncthreads_or(*reinterpret_cast<volatile uint32_t *>(&sm->n) >
                                         CAP - NT)) {
                        compact(sm);
                    }
                }
                if (mine) {
                    const uint32_t rr = g0 + b / GROUP;
                    const uint32_t id = c.lo + rr * ROUND + tid * GROUP + (b % GROUP);
                    Frag one;
                    one.v[0] = make_uint4(__float_as_uint(widen(row_ptr[id])), 0, 0, 0);
                    one.v[1] = make_uint4(0, 0, 0, 0);
                    if (sizeof(T) == 2) {
                        // frag_get reads element 0 from the low half-word.
                        one.v[0].x = (uint32_t)reinterpret_cast<const uint16_t *>(row_ptr)[id];
                    }
                    // No second test against the threshold: a refused element
                    // may tie with the k-th key and win the tie by its lower id.
                    process_frag<T>(sm, c, one, nullptr, id, 1u, __uint_as_float(0x7FC00000u),
                                    always_seen);
                }
            }
            __syncthreads();
        }
        dropped = 0;
        // Groups 0, 1, 2, 3, 4, 6, 8, 12, 16, ...: the threshold moves ever
        // more slowly as the row goes by.
        const uint32_t g3 = g / 3u;
        const bool due = g < 5u || (g & (g - 1u)) == 0u || (g3 * 3u == g && (g3 & (g3 - 1u)) == 0u);
        if (due && (tid >> 5) == (g & (NT / 32 - 1u))) {
            // The lanes may come out of the divergent pushes apart: meet
            // first, then let ONE lane's reading decide for the whole warp
            // (the flag can change between two lanes' readings).
            __syncwarp();
            uint32_t go = 0;
            if ((tid & 31u) == 0u) {
                go = *reinterpret_cast<volatile uint32_t *>(&sm->th_new);
            }
            go = __shfl_sync(0xFFFFFFFFu, go, 0);
            if (go != 0u) {
                tighten(sm);
            }
        }
    };

    // Round 0 is in `first` already.
    if (nrounds > 0u) {
        look(first, 0u, c.lo + tid * GROUP, nfull > 0u);
        if (RGROUP == 1u || nrounds == 1u) {
            meet(0u);
        }
    }
    // The full rounds: the hot loop.
    {
        const uint32_t ring_me = (uint32_t)__cvta_generic_to_shared(ring) + tid * FRAG_BYTES;
        const char *src = my_src + (size_t)STAGES * (ROUND * sizeof(T));  // round r + STAGES - 1, r = 1
        uint32_t base = c.lo + ROUND + tid * GROUP;
        for (uint32_t r = 1; r < nfull; ++r) {
            if (VEC) {
                // Prefetch round r + STAGES - 1 (STAGES == 2: the other slot).
                if (r + STAGES - 1 < nfull) {
                    const uint32_t dst = ring_me + ((r + STAGES - 1) % STAGES) * (NT * FRAG_BYTES);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src)
                                 : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + 16u),
                                 "l"(src + 16)
                                 : "memory");
                } else {
                    issue(r + STAGES - 1);  // the partial round, or nothing: commits below too
                }
                if (r + STAGES - 1 < nfull) {
                    cp_async_commit();
                }
                src += ROUND * sizeof(T);
            }
            Frag cur;
            fetch(r, cur);
            look(cur, r, base, true);
            base += ROUND;
            if ((r % RGROUP) == RGROUP - 1u || r == nrounds - 1u) {
                meet(r);
            }
        }
    }
    // The last, partial round (if any).
    if (nrounds > nfull && nfull > 0u) {
        const uint32_t r = nfull;
        issue(r + STAGES - 1);
        Frag cur;
        fetch(r, cur);
        look(cur, r, c.lo + r * ROUND + tid * GROUP, false);
        meet(r);
    }
    cp_async_wait<0>();
    }  // !lean
    __syncthreads();

    LILY_STAMP(PH_STREAM);
    if (tid < 32u && sm->th_new != 0u) {
        tighten(sm);
    }
    __syncthreads();
    filter_adjust(sm);  // reads the count table: before it is cleared
    // The count table goes back to all zero (history-list mode only).
    if (c.need_counts && !table_mode) {
        const uint32_t total = hist_len + extra_len;
        for (uint32_t i0 = 0; i0 < total; i0 += NT) {
            const uint32_t i = i0 + tid;
            uint32_t id = 0xFFFFFFFFu;
            if (i < total) {
                id = i < hist_len ? hist[i] : a.extra_ids[i - hist_len];
            }
            // The row's table is this row's alone, and a slice owns its range of
            // ids: plain stores (a frequent id is simply zeroed many times).
            if (id >= c.lo && id < c.hi) {
                counts_rw[id] = 0u;
            }
        }
    }

    uint32_t n = min(sm->n, CAP);
    __syncthreads();
    bool sorted = false;
    if (n <= RANKSORT_MAX) {
        rank_sort(sm, n, c.k);
        n = min(n, c.k);
        sorted = true;
    } else if (n_slices == 1u && n <= SORT2K) {
        // A row in one block with many candidates: sorting them all costs less
        // than selecting the best k and sorting those.
        sort_block_2k(sm, n);
        n = min(n, c.k);
        sorted = true;
        if (tid == 0) {
            sm->n = n;
            sm->n_adj = n;
            sm->tau_key = sm->key[n - 1u];
        }
        __syncthreads();
    } else if (n > c.k) {
        select_topk(sm, n, c.k);
        n = c.k;
    }
    LILY_STAMP(PH_LOCAL_SELECT);

    // ---- D. merge the slices
    if (n_slices > 1u) {
        uint2 *mine = a.part + (uint64_t)row * CAP + slice * c.k;
        for (uint32_t i = tid; i < n; i += NT) {
            mine[i] = make_uint2(sm->key[i], sm->id[i]);
        }
        if (tid == 0) {
            a.part_n[row * MAX_SLICES + slice] = n | (sm->err << 24);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const uint32_t ticket = atomicAdd(a.tickets + row, 1u);
            sm->is_last = ticket == n_slices - 1u;
        }
        __syncthreads();
        if (!sm->is_last) {
            return;
        }
        __threadfence();
        // Every slice's count at once, a prefix over them, then one parallel
        // gather of all entries.
        uint32_t *offs = sm->tkey;  // n_slices + 1 offsets
        if (tid < n_slices) {
            const uint32_t word = __ldcg(a.part_n + row * MAX_SLICES + tid);
            offs[tid + 1u] = word & 0xFFFFFFu;
            if (word >> 24) {
                sm->err = word >> 24;
            }
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t run = 0;
            offs[0] = 0;
            for (uint32_t s = 0; s < n_slices; ++s) {
                run += offs[s + 1u];
                offs[s + 1u] = run;
            }
            a.tickets[row] = 0;
            sm->n = min(run, CAP);
            sm->n_adj = min(run, CAP);
            if (run > CAP) {
                sm->err = ROW_INTERNAL;
            }
        }
        __syncthreads();
        const uint32_t total = sm->n;
        for (uint32_t i = tid; i < total; i += NT) {
            // The slice of entry i: the last offset not above i.
            uint32_t lo_s = 0, hi_s = n_slices;
            while (hi_s - lo_s > 1u) {
                const uint32_t mid = (lo_s + hi_s) >> 1;
                if (offs[mid] <= i) {
                    lo_s = mid;
                } else {
                    hi_s = mid;
                }
            }
            const uint2 e = __ldcg(a.part + (uint64_t)row * CAP + lo_s * c.k + (i - offs[lo_s]));
            sm->key[i] = e.x;
            sm->id[i] = e.y;
        }
        __syncthreads();
        n = sm->n;
        sorted = false;
        if (n <= RANKSORT_MAX) {
            rank_sort(sm, n, c.k);
            n = min(n, c.k);
            sorted = true;
        } else if (n > c.k) {
            select_topk(sm, n, c.k);
            n = c.k;
        }
    }
    if (n == 0u && a.cand_out) {
        // An empty record; the status word carries the reason.
        ShardRecord *rec = a.cand_out + row;
        for (uint32_t i = tid; i < LILY_SHARD_CANDIDATES; i += NT) {
            rec->cand[i] = make_uint2(0u, 0xFFFFFFFFu);
        }
        if (tid == 0) {
            rec->max_adj = neg_inf();
            rec->sum_exp = 0.0f;
            atomicOr(a.status_word, 1u << ((sm->err ? sm->err : ROW_INTERNAL) & 31u));
        }
        return;
    }
    if (n == 0u) {
        // Nothing but NaNs reached the buffer (or a bug): an error row.
        if (tid == 0) {
            const uint32_t err = sm->err ? sm->err : ROW_INTERNAL;
            a.out_ids[out_row] = 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[out_row] = err;
            }
            if (a.kept_n) {
                a.kept_n[out_row] = 0;
            }
            atomicOr(a.status_word, 1u << (err & 31u));
        }
        return;
    }
    LILY_STAMP(PH_MERGE);
    if (a.cand_out) {
        // A shard launch ends here: the sorted candidates are the row's record.
        if (tid < 32u) {
            if (!sorted) {
                sort_candidates<true>(sm, n);
            }
            ShardRecord *rec = a.cand_out + row;
            for (uint32_t i = tid; i < LILY_SHARD_CANDIDATES; i += 32u) {
                rec->cand[i] = i < n ? make_uint2(sm->key[i], sm->id[i] + a.id_offset)
                                     : make_uint2(0u, 0xFFFFFFFFu);
            }
            if (tid == 0) {
                rec->max_adj = float_of_key(sm->key[0]);
                rec->sum_exp = 0.0f;
                if (sm->err) {
                    atomicOr(a.status_word, 1u << (sm->err & 31u));
                }
            }
        }
        return;
    }
    if (n <= 64u) {
        // One warp finishes the row; the others are done.
        if (tid < 32u) {
            if (!sorted) {
                sort_candidates<true>(sm, n);
            }
            LILY_STAMP(PH_SORT);
            if (row < a.spec.n_spec) {
                finalize<true>(sm, a, row, n, P.seed);
            } else {
                finalize_warp(sm, a, row, n, P.seed);
            }
            LILY_STAMP(PH_END);
        }
    } else {
        if (!sorted) {
            sort_candidates<false>(sm, n);
        }
        LILY_STAMP(PH_SORT);
        finalize<false>(sm, a, row, n, P.seed);
        LILY_STAMP(PH_END);
    }
}

// Grid (slices, rows): block (x, y) takes slice x of row row0 + y.
template <typename T, bool VEC>
__global__ void __launch_bounds__(NT, 2) sample_rows_kernel(const __grid_constant__ KArgs a) {
    sample_row<T, VEC>(a, a.row0 + blockIdx.y, blockIdx.x);
}

// The whole row in one block, out of line: what stream_rows_kernel calls for a
// row it does not take itself.
template <typename T>
__device__ __noinline__ void sample_whole_row(const KArgs &a, uint32_t row) {
    sample_row<T, true>(a, row, 0u);
}

// The draw of a vocabulary-sharded row: the shards' records hold every
// candidate the row's top-k can contain (each shard kept its own best
// shard_k >= k), so selecting, cutting and drawing over their union gives
// what one pass over the whole vocabulary gives. One block per row.
__device__ __forceinline__ void peer_exchange_row(const KArgs &a, uint32_t row);

__global__ void __launch_bounds__(NT, 2) merge_rows_kernel(const __grid_constant__ KArgs a) {
    extern __shared__ uint4 smem_raw[];
    SmemFixed *sm = reinterpret_cast<SmemFixed *>(smem_raw);
    const uint32_t tid = threadIdx.x;
    const uint32_t row = a.row0 + blockIdx.x;
    if (a.peer.n != 0u) {
        peer_exchange_row(a, row);  // the row's records of all ranks are in the own buffer after this
    }
    const lily_sampling_params_t P = a.params[row];
    const bool greedy = P.temperature <= 0.0f || P.top_k == 1u;
    if (tid == 0) {
        RowCtx c;
        c.T = greedy ? 1.0f : P.temperature;
        c.k = greedy ? 1u : (P.top_k == 0u ? KCAP : min(P.top_k, KCAP));
        c.rep = 1.0f;
        c.presence = c.frequency = 0.0f;
        c.top_p = P.top_p;
        c.min_p = P.min_p;
        c.use_pen = c.need_counts = c.has_special = false;
        c.monotone = true;
        c.argmax_mode = greedy;
        c.lo = 0;
        c.hi = a.vocab;
        c.seen = nullptr;
        c.counts = nullptr;
        c.bias_ids = c.ban_ids = nullptr;
        c.bias_vals = nullptr;
        c.bias_len = c.ban_len = 0;
        c.sp_in_smem = true;
        sm->ctx = c;
        sm->n = 0;
        sm->err = 0;
        sm->u_draw = a.uniforms ? a.uniforms[row] : uniform_for(P.seed, a.steps ? a.steps[row] : 0u);
        sm->ckey = sm->key;
        sm->cid = sm->id;
        sm->ccap = CAP;
    }
    __syncthreads();
    const uint32_t slots = a.merge_shards * LILY_SHARD_CANDIDATES;
    for (uint32_t i = tid; i < slots; i += NT) {
        const ShardRecord *rec = a.merge_in + (uint64_t)(i / LILY_SHARD_CANDIDATES) * a.merge_stride + row;
        const uint2 e = rec->cand[i % LILY_SHARD_CANDIDATES];
        if (e.y != 0xFFFFFFFFu) {
            const uint32_t at = atomicAdd(&sm->n, 1u);
            sm->key[at] = e.x;
            sm->id[at] = e.y;
        }
    }
    if (a.out_lse && tid == 0) {
        // Shards in order: the largest maximum, then the sums rescaled to it.
        float top = neg_inf();
        for (uint32_t s = 0; s < a.merge_shards; ++s) {
            top = fmaxf(top, a.merge_in[(uint64_t)s * a.merge_stride + row].max_adj);
        }
        float sum = 0.0f;
        for (uint32_t s = 0; s < a.merge_shards; ++s) {
            const ShardRecord *rec = a.merge_in + (uint64_t)s * a.merge_stride + row;
            sum += rec->sum_exp * expf(rec->max_adj - top);
        }
        a.out_lse[row] = top + logf(sum);
    }
    __syncthreads();
    uint32_t n = sm->n;
    const uint32_t k = sm->ctx.k;
    if (n == 0u) {
        if (tid == 0) {
            a.out_ids[row] = 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[row] = ROW_INTERNAL;
            }
            if (a.kept_n) {
                a.kept_n[row] = 0;
            }
            atomicOr(a.status_word, 1u << ROW_INTERNAL);
        }
        return;
    }
    if (tid == 0) {
        sm->n_adj = n;
    }
    __syncthreads();
    bool sorted = false;
    if (n <= RANKSORT_MAX) {
        rank_sort(sm, n, k);
        n = min(n, k);
        sorted = true;
    } else if (n > k) {
        select_topk(sm, n, k);
        n = k;
    }
    if (n <= 64u) {
        if (tid < 32u) {
            if (!sorted) {
                sort_candidates<true>(sm, n);
            }
            finalize_warp(sm, a, row, n, P.seed);
        }
    } else {
        if (!sorted) {
            sort_candidates<false>(sm, n);
        }
        finalize<false>(sm, a, row, n, P.seed);
    }
}

// Sum over a shard row of exp(adjusted - the shard's maximum), for records
// made without penalties or lists: adjusted = l / T (l for a greedy row). A
// row is cut into gridDim.x pieces; every add happens in a fixed order (a
// thread's strided elements, the shuffle tree, the warps, the pieces), so the
// sum is reproducible. The last block of a row to finish adds the pieces up.
template <typename T>
__global__ void __launch_bounds__(1024) shard_sums_kernel(const T *logits, uint64_t ld, uint32_t vocab,
                                                           const lily_sampling_params_t *params,
                                                           ShardRecord *records, float *pieces,
                                                           uint32_t *tickets) {
    __shared__ float warp_part[32];
    __shared__ uint32_t is_last;
    const uint32_t row = blockIdx.y, piece = blockIdx.x, tid = threadIdx.x;
    const lily_sampling_params_t P = params[row];
    const bool greedy = P.temperature <= 0.0f || P.top_k == 1u;
    const float temp = greedy ? 1.0f : P.temperature;
    const float top = records[row].max_adj;
    const T *src = logits + (uint64_t)row * ld;
    const uint32_t len = (vocab + gridDim.x - 1u) / gridDim.x;
    const uint32_t lo = piece * len, hi = min(vocab, lo + len);
    // exp(l / T - top) as exp2((l - top * T) * log2(e) / T): a reported
    // statistic, not part of the draw, so the fast exponential will do.
    const float scale = 1.4426950408889634f / temp;
    const float shift = top * temp;
    float s = 0.0f;
    const bool vec = sizeof(T) == 4 && ((reinterpret_cast<uintptr_t>(src) | (lo * sizeof(T))) & 15u) == 0u;
    uint32_t i = lo + tid;
    if (vec) {
        const float4 *src4 = reinterpret_cast<const float4 *>(src + lo);
        const uint32_t n4 = (hi - lo) / 4u;
        for (uint32_t q = tid; q < n4; q += 1024u) {
            const float4 v = __ldcg(src4 + q);
            const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float t = exp2f((x[e] - shift) * scale);
                s += t == t ? t : 0.0f;
            }
        }
        i = lo + n4 * 4u + tid;
    }
    for (; i < hi; i += 1024u) {
        const float t = exp2f((widen(src[i]) - shift) * scale);
        s += t == t ? t : 0.0f;
    }
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    }
    if ((tid & 31u) == 0u) {
        warp_part[tid >> 5] = s;
    }
    __syncthreads();
    if (tid < 32u) {
        s = warp_part[tid];
        for (int o = 16; o > 0; o >>= 1) {
            s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        }
        if (tid == 0) {
            pieces[row * MAX_SLICES + piece] = s;
            __threadfence();
            is_last = atomicAdd(tickets + row, 1u) == gridDim.x - 1u;
        }
    }
    __syncthreads();
    if (is_last && tid == 0) {
        __threadfence();
        float total = 0.0f;
        for (uint32_t p = 0; p < gridDim.x; ++p) {
            total += __ldcg(pieces + row * MAX_SLICES + p);
        }
        records[row].sum_exp = total;
        tickets[row] = 0;
    }
}

// ---- records over peer memory ------------------------------------------------
//
// A rank's exchange buffer: a flag word per (rank, row), then two slots of
// n_shards x max_rows records (see lily_sampler.h). `buffers` are the ranks'
// buffers as this process sees them: the own one in this GPU's memory, the
// others across NVLink. Only plain loads and stores go there.
constexpr uint32_t PEER_MAX = 16;

__host__ __device__ inline uint32_t peer_flag_bytes(uint32_t n_shards, uint32_t max_rows) {
    return (n_shards * max_rows * 4u + 255u) & ~255u;
}

struct PeerArgs {
    void *buffers[PEER_MAX];
    const ShardRecord *records;  // this rank's records of the step
    uint32_t n_shards, rank, max_rows, rows, step;
};

__device__ __forceinline__ ShardRecord *peer_slot(void *buffer, uint32_t n_shards, uint32_t max_rows,
                                                  uint32_t step, uint32_t shard) {
    return reinterpret_cast<ShardRecord *>(static_cast<char *>(buffer) + peer_flag_bytes(n_shards, max_rows)) +
           ((size_t)(step & 1u) * n_shards + shard) * max_rows;
}

__device__ __forceinline__ void peer_raise(void *buffer, uint32_t max_rows, uint32_t rank, uint32_t row,
                                           uint32_t step) {
    uint32_t *flag = static_cast<uint32_t *>(buffer) + (size_t)rank * max_rows + row;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step) : "memory");
}

// Grid (n_shards): block b writes this rank's records into rank b's buffer with
// plain stores, fences them system-wide and then raises this rank's flag of
// every row there. (The merge kernel does the same for its own row when it is
// given the records; this kernel serves a rank that publishes apart from its
// merge, and one GPU that plays several ranks in a test.)
__global__ void __launch_bounds__(256) shard_publish_kernel(const __grid_constant__ PeerArgs p) {
    void *buffer = p.buffers[blockIdx.x];
    const uint2 *src = reinterpret_cast<const uint2 *>(p.records);
    uint2 *dst = reinterpret_cast<uint2 *>(peer_slot(buffer, p.n_shards, p.max_rows, p.step, p.rank));
    const uint32_t n8 = p.rows * (uint32_t)(sizeof(ShardRecord) / 8u);
    for (uint32_t i = threadIdx.x; i < n8; i += 256u) {
        dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    for (uint32_t r = threadIdx.x; r < p.rows; r += 256u) {
        peer_raise(buffer, p.max_rows, p.rank, r, p.step);
    }
}

// A row's block of the merge kernel, before it merges: publishes this rank's
// record of the row (if given), then waits, for at most wait_ns, until every
// rank's flag of the row in the own buffer has reached the step. A wait that
// runs out sets bit 30 of the status word; the merge then reads what is there.
__device__ __forceinline__ void peer_exchange_row(const KArgs &a, uint32_t row) {
    const KArgs::PeerLink &p = a.peer;
    const uint32_t tid = threadIdx.x;
    constexpr uint32_t W = (uint32_t)(sizeof(ShardRecord) / 8u);  // 8-byte words of a record
    if (p.own != nullptr) {
        const uint2 *src = reinterpret_cast<const uint2 *>(static_cast<const ShardRecord *>(p.own) + row);
        for (uint32_t i = tid; i < p.n * W; i += NT) {
            const uint32_t to = i / W, w = i % W;
            reinterpret_cast<uint2 *>(peer_slot(p.buffers[to], p.n, p.max_rows, p.step, p.rank) + row)[w] = src[w];
        }
        __threadfence_system();
        __syncthreads();
        if (tid < p.n) {
            peer_raise(p.buffers[tid], p.max_rows, p.rank, row, p.step);
        }
    }
    if (tid < 32u) {
        bool late = false;
        if (tid < p.n) {
            const uint32_t *flag = static_cast<const uint32_t *>(p.buffers[p.rank]) + (size_t)tid * p.max_rows + row;
            const unsigned long long t0 = (unsigned long long)global_ns();
            for (uint32_t spin = 0;; ++spin) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if ((int32_t)(v - p.step) >= 0) {
                    break;
                }
                if ((spin & 63u) == 63u && (unsigned long long)global_ns() - t0 > p.wait_ns) {
                    late = true;
                    break;
                }
            }
        }
        if (__any_sync(0xFFFFFFFFu, late) && tid == 0) {
            atomicOr(a.status_word, 1u << 30);
        }
    }
    __syncthreads();
}

// src/kernels/metal/spec.metal:14-38, one thread.
__global__ void spec_accept_kernel(const uint32_t *draws, const uint32_t *ids, uint32_t id_offset,
                                   uint32_t m, uint32_t *ctrl, uint32_t pos0, uint32_t ratio,
                                   uint32_t chain, uint32_t stride) {
    if (blockIdx.x != 0 || threadIdx.x != 0) {
        return;
    }
    // ids[j + id_offset] is the token row j's draw must equal: the verified
    // tokens start with the pending token (offset 1), a bare proposal list
    // does not (offset 0).
    uint32_t acc = 0;
    while (acc + 1u < m && draws[acc] == ids[acc + id_offset]) {
        ++acc;
    }
    ctrl[0] = acc;
    if (stride == 0u) {
        return;
    }
    ctrl[stride] = acc + 1u;
    for (uint32_t i = 0; i < chain; ++i) {
        const uint32_t p = pos0 + acc + 1u + i;
        ctrl[(2u + 3u * i) * stride] = p;
        ctrl[(3u + 3u * i) * stride] = p / ratio;
        ctrl[(4u + 3u * i) * stride] = ((p + 1u) % ratio == 0u) ? 1u : 0u;
    }
}

// Histogram-slot maintenance (src/kernels/sample.rs:145-174).
__global__ void uncount_kernel(uint32_t *counts, uint32_t *seen, uint32_t vocab, uint32_t token) {
    if (blockIdx.x != 0 || threadIdx.x != 0 || token >= vocab) {
        return;
    }
    const uint32_t cur = counts[token];
    if (cur > 0u) {
        counts[token] = cur - 1u;
        if (cur == 1u) {
            seen[token >> 5] &= ~(1u << (token & 31u));
        }
    }
}

__global__ void rebuild_seen_kernel(const uint32_t *counts, uint32_t *seen, uint32_t vocab) {
    const uint32_t w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w * 32u >= vocab) {
        return;
    }
    uint32_t bits = 0;
    for (uint32_t b = 0; b < 32u; ++b) {
        const uint32_t id = w * 32u + b;
        if (id < vocab && counts[id] > 0u) {
            bits |= 1u << b;
        }
    }
    seen[w] = bits;
}

__global__ void exp_kernel(const float *in, float *out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x) {
        out[i] = exp_f32(in[i]);
    }
}

}  // namespace lily
