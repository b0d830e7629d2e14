// The large-batch kernel: one thread block per row, the row read exactly once.
//
// When a launch has at least as many rows as the GPU has block slots, nothing
// is gained by cutting rows into slices, and what limits the step is how long a
// block does anything else than wait for DRAM. This kernel is the compact path
// for the rows such launches are made of: 16-byte aligned logits, a row of at
// least eight rounds, at most 64 candidates kept (top_k 1..64, or greedy), no
// bias / ban list, penalties that can only lower a logit (or none), no
// frequency penalty over a history list. For every other row (and for a row
// that turns out to hold a NaN, or more ties around its threshold than the
// small candidate buffer takes) the block calls the general code of
// sample_rows_kernel on the whole row instead; results do not depend on which
// of the two drew a row.
//
// The row streams through a four-stage cp.async ring. Up to round r_check a
// thread only tracks the maxima of its fragments (its best fragment stays in
// registers). At r_check every thread adjusts its largest logit so far; each
// warp sorts its 32 keys and leaves the best eight in a pool of 128 keys of
// 128 different ids, whose k-th largest is a lower bound of the row's k-th
// largest adjusted value. As soon as a warp sees the pool complete (an
// mbarrier it polls once per round: nobody waits) it takes the bound from the
// pool, collects what its rounds so far hold above it and from then on tests
// every new fragment against the bound directly. History ids are marked in
// the seen bitmap inside the first rounds (two 16-byte loads of ids per thread
// and round); a second mbarrier tells the threads that adjust a logit that
// every mark is in place. When the last round has landed the candidates are in
// the buffer: one candidate per thread is adjusted and ranked by counting, and
// one warp runs the softmax prefix, the cut and the draw in registers.
#pragma once

#include "sample_kernel.cuh"

namespace lily {

constexpr uint32_t STREAM_MIN_ROUNDS = 8;  // launches with shorter rows use sample_rows_kernel
constexpr uint32_t STREAM_K_MAX = 64;      // finalize_warp holds two candidates per lane
// AHEAD (template argument of the kernel): rounds of the ring in flight beyond the
// one being read. With a block slot's worth of rows two measured faster than
// three (33.4 against 34.0 us per 256-row launch; asking L2 for further rounds
// ahead of the ring was slower still: the stream is not short of requests). With
// fewer rows than SMs a block streams alone against the latency of its own
// requests: it has the SM's shared memory to itself, and takes a ring of eight
// stages with seven rounds in flight (112 KB per block) and four 16-byte loads of
// history ids per thread and round instead of two.
template <uint32_t AHEAD>
struct StreamDepth {
    static_assert(AHEAD == 2u || AHEAD == 3u || AHEAD == 7u, "a ring of four stages, or of eight");
    static constexpr uint32_t STAGES = AHEAD <= 3u ? 4u : 8u;     // of the ring
    static constexpr uint32_t HQ = AHEAD <= 3u ? 2u : 4u;         // 16-byte history loads per thread and round
    static constexpr uint32_t BLOCKS = AHEAD <= 3u ? 2u : 1u;     // per SM
    static constexpr uint32_t EXTRA_BYTES = (STAGES - 4u) * NT * FRAG_BYTES;  // stages beyond the four shared ones
};

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count) {
    const uint32_t at = (uint32_t)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    const uint32_t at = (uint32_t)__cvta_generic_to_shared(bar);
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(at) : "memory");
}

// Waits for the barrier's first phase, at most about a millisecond; false if
// it gave up (a bug elsewhere: the row is left to the general code).
__device__ __forceinline__ bool mbar_wait_first(unsigned long long *bar) {
    const uint32_t at = (uint32_t)__cvta_generic_to_shared(bar);
    for (uint32_t i = 0; i < (1u << 16); ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(at)
            : "memory");
        if (done) {
            return true;
        }
    }
    return false;
}

// Whether the barrier's first phase is over (does not wait).
__device__ __forceinline__ bool mbar_test_first(unsigned long long *bar) {
    const uint32_t at = (uint32_t)__cvta_generic_to_shared(bar);
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done)
                 : "r"(at)
                 : "memory");
    return done != 0u;
}

constexpr uint32_t POOL_PER_WARP = 8;
constexpr uint32_t POOL = POOL_PER_WARP * (NT / 32);
static_assert(POOL == 128, "four pool keys per lane");

__device__ __forceinline__ uint32_t warp_sort_desc(uint32_t v) {
    const uint32_t lane = threadIdx.x & 31u;
#pragma unroll
    for (uint32_t size = 2u; size <= 32u; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0u; stride >>= 1) {
            const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, v, stride);
            const bool first = ((lane & size) == 0u) == ((lane & stride) == 0u);
            v = first ? max(v, other) : min(v, other);
        }
    }
    return v;  // lane 0 holds the largest
}

// Any full warp: the largest v with its low 16 bits clear that at least k of
// the pool's keys reach, bit by bit from the top.
__device__ __forceinline__ uint32_t pool_kth(const uint32_t *pool, uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t v0 = pool[lane], v1 = pool[lane + 32u], v2 = pool[lane + 64u], v3 = pool[lane + 96u];
    uint32_t kth = 0u;
#pragma unroll 1
    for (int bit = 31; bit >= 16; --bit) {
        const uint32_t cand = kth | (1u << bit);
        const uint32_t cnt = (v0 >= cand ? 1u : 0u) + (v1 >= cand ? 1u : 0u) + (v2 >= cand ? 1u : 0u) +
                             (v3 >= cand ? 1u : 0u);
        if (__reduce_add_sync(0xFFFFFFFFu, cnt) >= k) {
            kth = cand;
        }
    }
    return kth;
}

// Elements of a fragment from `nvalid` on become -inf (the row's last,
// partial round: cp.async filled them with zeros).
template <typename T>
__device__ __forceinline__ void frag_mask_tail(Frag &f, uint32_t nvalid) {
    uint32_t *w = reinterpret_cast<uint32_t *>(&f);
    if (sizeof(T) == 4) {
#pragma unroll
        for (uint32_t e = 0; e < 8u; ++e) {
            if (e >= nvalid) {
                w[e] = 0xFF800000u;
            }
        }
    } else {
#pragma unroll
        for (uint32_t e = 0; e < 8u; ++e) {
            const uint32_t lo = 2u * e < nvalid ? (w[e] & 0xFFFFu) : 0xFF80u;
            const uint32_t hi = 2u * e + 1u < nvalid ? (w[e] & 0xFFFF0000u) : 0xFF800000u;
            w[e] = lo | hi;
        }
    }
}

// A shard's record also carries sum exp(adjusted - largest adjusted) over the
// shard (a reported statistic: the log-sum-exp of the whole vocabulary). In the
// kernel of one block per row a thread keeps it for its own logits as it reads
// them, in the base-2 domain and relative to its own running maximum:
// sum_t = sum exp2(x * scale - ref_t). A fragment whose maximum beats the
// reference rescales the sum first.
struct RunningSum {
    float ref, sum;
};

template <typename T>
__device__ __forceinline__ void running_sum_add(RunningSum &rs, const Frag &cur, float m, float scale) {
    const float y = m * scale;
    if (y > rs.ref) {
        rs.sum *= exp2f(rs.ref - y);
        rs.ref = y;
    }
#pragma unroll
    for (int e = 0; e < (int)Geo<T>::GROUP; ++e) {
        rs.sum += exp2f(fmaf(frag_get<T>(cur, e), scale, -rs.ref));  // (a masked -inf adds 0)
    }
}

// The block's total relative to `top2` (the record's largest adjusted logit, base
// 2), in a fixed order: the lanes' tree, then the warps one after the other.
__device__ __forceinline__ float running_sum_total(SmemFixed *sm, const RunningSum &rs, float top2) {
    float v = rs.sum * exp2f(rs.ref - top2);
    v = v == v ? v : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
    float *part = reinterpret_cast<float *>(sm->thist);  // (the pool is no longer needed)
    __syncthreads();
    if ((threadIdx.x & 31u) == 0u) {
        part[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < NT / 32u; ++w) {
        total += part[w];
    }
    return total;
}

// The same sum by a second look at the row, for a row that went to the general
// code (which leaves sum_exp at 0): every thread its strided share.
template <typename T>
__device__ __noinline__ float reread_sum(SmemFixed *sm, const T *row_ptr, uint32_t vocab, float scale, float top2) {
    RunningSum rs{top2, 0.0f};
    for (uint32_t i = threadIdx.x; i < vocab; i += NT) {
        const float t = exp2f(fmaf(widen(row_ptr[i]), scale, -top2));
        rs.sum += t == t ? t : 0.0f;
    }
    return running_sum_total(sm, rs, top2);
}

// End of the stream with at most one buffered candidate per thread (all raw):
// adjusts them, drops what lies below the threshold key and leaves the best k
// sorted by (key descending, id ascending) in key / id [0, result): every live
// candidate counts how many come before it (four threads share the count of a
// candidate while there are at most 128). Two block barriers.
__device__ __forceinline__ uint32_t small_select(SmemFixed *sm, uint32_t n, uint32_t k) {
    const uint32_t tid = threadIdx.x;
    unsigned long long *packed = reinterpret_cast<unsigned long long *>(sm->tkey);  // (key, ~id), 0 = dropped
    static_assert(2u * KCAP * 4u >= NT * 8u, "tkey and tid hold one packed candidate per thread");
    unsigned long long mine = 0ull;
    bool alive = false;
    if (tid < n) {
        const uint32_t id = sm->lid[tid];
        const uint32_t key = adjusted_key(sm, id, __uint_as_float(sm->lkey[tid]), false);
        alive = key >= sm->kstar;
        mine = alive ? ((unsigned long long)key << 32) | (uint32_t)~id : 0ull;
        packed[tid] = mine;
    }
    const uint32_t live = (uint32_t)__syncthreads_count(alive);
    if (n <= NT / 4u) {
        // Up to 128 candidates: four threads share a candidate's count.
        const uint32_t c = tid >> 2, part = tid & 3u;
        const unsigned long long cand = c < n ? packed[c] : 0ull;
        uint32_t rank = 0;
        if (cand != 0ull) {
#pragma unroll 4
            for (uint32_t j = part; j < n; j += 4u) {
                rank += packed[j] > cand ? 1u : 0u;
            }
        }
        rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 1);
        rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 2);
        if (cand != 0ull && part == 0u && rank < k) {
            sm->key[rank] = (uint32_t)(cand >> 32);
            sm->id[rank] = ~(uint32_t)cand;
        }
    } else if (alive) {
        uint32_t rank = 0;
#pragma unroll 4
        for (uint32_t j = 0; j < n; ++j) {
            rank += packed[j] > mine ? 1u : 0u;
        }
        if (rank < k) {
            sm->key[rank] = (uint32_t)(mine >> 32);
            sm->id[rank] = ~(uint32_t)mine;
        }
    }
    __syncthreads();
    return min(live, k);
}

template <typename T, uint32_t AHEAD>
__global__ void __launch_bounds__(NT, StreamDepth<AHEAD>::BLOCKS) stream_rows_kernel(const __grid_constant__ KArgs a) {
    constexpr uint32_t NS = StreamDepth<AHEAD>::STAGES, HQ = StreamDepth<AHEAD>::HQ;
    extern __shared__ uint4 smem_raw[];
    SmemFixed *sm = reinterpret_cast<SmemFixed *>(smem_raw);
    uint4 *ring = reinterpret_cast<uint4 *>(sm + 1);
    uint32_t *seen = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(ring) + RING_BYTES);
    constexpr uint32_t NONE = 0xFFFFFFFFu;
    constexpr uint32_t GROUP = Geo<T>::GROUP, ROUND = Geo<T>::ROUND;

    const uint32_t tid = threadIdx.x;
    const uint32_t row = a.row0 + blockIdx.x;
    long long *stamps = a.phase_clocks ? a.phase_clocks + (uint64_t)row * MAX_SLICES * LILY_PHASES : nullptr;
    if (stamps && tid == 0) {
        stamps[PH_ENTRY] = global_ns();
    }

    // What needs no input comes first: with the programmatic-serialisation
    // attribute the blocks start while the stream's previous kernel drains, and
    // wait below for its memory before they touch any.
    const uint32_t seen_words = (a.vocab + 31u) >> 5;
    for (uint32_t w = tid; w < seen_words; w += NT) {
        seen[w] = 0;
    }
    if (tid == 0) {
        mbar_init(&sm->mbar[0], NT);
        mbar_init(&sm->mbar[1], NT / 32);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // The few words the block has to know about its row, before the first
    // rounds of logits that every block asks for next.
    const uint32_t hist_len_row = (a.history_ids && a.history_len) ? __ldg(a.history_len + row) : 0u;
    const int32_t forced = a.forced_ids ? __ldg(a.forced_ids + row) : -1;
    const uint32_t bias_len_row = (a.bias_ids && a.bias_len) ? __ldg(a.bias_len + row) : 0u;
    const uint32_t ban_len_row = (a.ban_ids && a.ban_len) ? __ldg(a.ban_len + row) : 0u;
    const uint32_t slot = a.count_slots ? __ldg(a.count_slots + row) : 0u;
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
    const T *row_ptr = reinterpret_cast<const T *>(a.logits) + (uint64_t)row * a.logits_ld;
    const char *src0 = reinterpret_cast<const char *>(row_ptr + tid * GROUP);  // the thread's 32 bytes of round 0
    // The ring: stages 0 and 1 behind the fixed block, stages 2 and 3 in the
    // (here unused) candidate arrays key and id, one round each.
    static_assert(CAP * 4u == NT * FRAG_BYTES && STAGES == 2, "key[] and id[] are one round each");
    // (Stages 4 to 7 of the deep ring lie behind the seen bits, where the general
    // row code, should the row go to it, has nothing.)
    const uint32_t slot_a = (uint32_t)__cvta_generic_to_shared(ring) + tid * FRAG_BYTES;
    const uint32_t slot_b = (uint32_t)__cvta_generic_to_shared(sm->key) + tid * FRAG_BYTES;
    const uint32_t slot_c = (uint32_t)__cvta_generic_to_shared(seen) +
                            ((((a.vocab + 255u) & ~255u) + 31u) / 32u + 8u) * 4u + tid * FRAG_BYTES;
    auto stage_at = [&](uint32_t st) -> uint32_t {
        if (NS == 4u) {
            return ((st & 2u) ? slot_b : slot_a) + (st & 1u) * ROUND_BYTES;
        }
        return (st < 2u ? slot_a : st < 4u ? slot_b - 2u * ROUND_BYTES : slot_c - 4u * ROUND_BYTES) + st * ROUND_BYTES;
    };
#pragma unroll
    for (uint32_t j = 0; j < AHEAD; ++j) {
        lean_copy_round(stage_at(j), src0 + j * ROUND_BYTES);
        cp_async_commit();
    }

    // A vocabulary shard's launch ends in a record per row, not in a draw.
    auto empty_record = [&](uint32_t status) {
        ShardRecord *rec = a.cand_out + row;
        for (uint32_t i = tid; i < LILY_SHARD_CANDIDATES; i += NT) {
            rec->cand[i] = make_uint2(0u, 0xFFFFFFFFu);
        }
        if (tid == 0) {
            rec->max_adj = neg_inf();
            rec->sum_exp = 0.0f;
            atomicOr(a.status_word, 1u << (status & 31u));
        }
    };
    auto refuse = [&](uint32_t status) {
        if (a.cand_out) {
            empty_record(status);
        } else if (tid == 0) {
            a.out_ids[row] = status == LILY_ROW_FORCED ? (uint32_t)forced : 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[row] = status;
            }
            if (a.kept_n) {
                a.kept_n[row] = 0;
            }
            if (status != LILY_ROW_FORCED) {
                atomicOr(a.status_word, 1u << status);
            }
        }
        cp_async_wait<0>();
    };
    if (forced >= 0) {
        refuse(LILY_ROW_FORCED);
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
            refuse(LILY_ROW_PARAMS);
            return;
        }
    }
    // (A pitch of 0 means one list shared by every row.)
    if (hist_len_row > a.max_history || (a.history_ld != 0u && hist_len_row > a.history_ld) ||
        bias_len_row > a.max_list || (a.bias_ld != 0u && bias_len_row > a.bias_ld) ||
        ban_len_row > a.max_list || (a.ban_ld != 0u && ban_len_row > a.ban_ld)) {
        refuse(LILY_ROW_LIST);
        return;
    }

    const bool greedy = P.temperature <= 0.0f || P.top_k == 1u;
    const bool use_pen = P.presence_penalty != 0.0f || P.frequency_penalty != 0.0f ||
                         P.repetition_penalty != 1.0f;
    // (A shard keeps shard_k candidates of a sampled row, whatever its top_k: the
    // host made sure that top_k fits.)
    const uint32_t k = greedy ? 1u : a.cand_out ? a.shard_k : (P.top_k == 0u ? KCAP : min(P.top_k, KCAP));
    // (A shard's record: the sum of exponentials in the same pass, if asked for.)
    const bool sums = a.cand_out != nullptr && a.shard_sums != 0u;
    const float sum_scale = 1.4426950408889634f / (greedy ? 1.0f : P.temperature);
    const bool monotone = P.repetition_penalty >= 1.0f && !(__float_as_uint(P.presence_penalty) >> 31) &&
                          !(__float_as_uint(P.frequency_penalty) >> 31);
    const bool need_counts = use_pen && P.frequency_penalty != 0.0f;
    const bool table_mode = a.count_slots != nullptr;
    // A row this path does not take, or cannot finish (below), gets the general
    // code on the whole row, from the start.
    bool mine = !(k > STREAM_K_MAX || bias_len_row + ban_len_row != 0u || (use_pen && !monotone) ||
                  (need_counts && !table_mode) || a.extra_len != 0u);
    uint32_t n_raw = 0;
    // (-3e38, not -inf: a first fragment of nothing but -inf must not give inf - inf)
    RunningSum rs{-3.0e38f, 0.0f};
    if (mine) {
    const uint32_t vocab = a.vocab;
    const uint32_t nfull = vocab / ROUND;  // >= STREAM_MIN_ROUNDS: the host launches this kernel only then
    const uint32_t has_part = vocab % ROUND != 0u ? 1u : 0u;
    const uint32_t nproc = nfull + has_part;
    const uint32_t part_at = nfull * ROUND + tid * GROUP;
    const uint32_t part_valid = (has_part && part_at < vocab) ? min(GROUP, vocab - part_at) : 0u;
    const uint32_t hist_len = (use_pen && !table_mode) ? hist_len_row : 0u;
    const uint32_t *hist = a.history_ids ? a.history_ids + (uint64_t)row * a.history_ld : nullptr;
    const uint4 *h4 = reinterpret_cast<const uint4 *>(hist);
    const bool hist_vec = (reinterpret_cast<uintptr_t>(hist) & 15u) == 0u;
    // 16-byte words of the history marked inside the stream, at most half of the
    // rounds' worth; the rest is marked before the stream starts.
    const uint32_t n4 = hist_vec ? min(hist_len / 4u, (nfull / 2u) * HQ * (uint32_t)NT) : 0u;
    const uint32_t mark_rounds = (n4 + HQ * NT - 1u) / (HQ * NT);
    const uint32_t r_check = max(mark_rounds, nfull / 2u);  // < nfull

    if (tid == 0) {
        RowCtx c;
        c.T = greedy ? 1.0f : P.temperature;
        c.k = k;
        c.rep = P.repetition_penalty;
        c.presence = P.presence_penalty;
        c.frequency = P.frequency_penalty;
        c.top_p = P.top_p;
        c.min_p = P.min_p;
        c.use_pen = use_pen;
        c.need_counts = need_counts;
        c.argmax_mode = greedy && !use_pen;
        c.monotone = monotone;
        c.has_special = false;
        c.lo = 0;
        c.hi = vocab;
        c.seen = seen;
        c.counts = need_counts ? a.counts_table + (uint64_t)slot * vocab : nullptr;
        c.bias_ids = nullptr;
        c.bias_vals = nullptr;
        c.bias_len = 0;
        c.ban_ids = nullptr;
        c.ban_len = 0;
        c.sp_in_smem = true;
        sm->ctx = c;
        sm->n = 0;
        sm->n_adj = 0;
        sm->err = 0;
        sm->kstar = 0;
        sm->c_raw = __uint_as_float(0x7FC00000u);
        sm->overflow = 0;
        sm->ckey = sm->lkey;
        sm->cid = sm->lid;
        sm->ccap = LCAP;
        sm->u_draw = a.uniforms ? u_row : uniform_for(P.seed, step_row);
        sm->lean_abort = 0;
    }
    if (use_pen && table_mode) {
        const uint32_t *src = a.seen_table + (uint64_t)slot * a.seen_words;
        for (uint32_t w = tid; w < seen_words; w += NT) {
            seen[w] = src[w];
        }
    }
    __syncthreads();
    if (stamps && tid == 0) {
        stamps[PH_START] = global_ns();
    }
    // History ids that are not marked on the way (a list that is not 16-byte
    // aligned, or longer than half the rounds can take).
    for (uint32_t i = n4 * 4u + tid; i < hist_len; i += NT) {
        const uint32_t id = hist[i];
        if (id < vocab) {
            atomicOr(&seen[id >> 5], 1u << (id & 31u));
        }
    }

    // ---- the stream
    const uint32_t seen_at = (uint32_t)__cvta_generic_to_shared(seen);
    float best = neg_inf(), m2 = neg_inf(), m3 = neg_inf(), m4 = neg_inf();
    uint32_t best_r = NONE, r2 = NONE, r3 = NONE;
    Frag keep;
    keep.v[0] = make_uint4(0, 0, 0, 0);
    keep.v[1] = make_uint4(0, 0, 0, 0);
    uint32_t saw_nan = 0u;
    const char *src = src0 + AHEAD * ROUND_BYTES;  // the round AHEAD ahead of the one being read
    // Starts the copy of round rr + AHEAD (into a stage whose round has been read)
    // and waits for round rr.
    auto advance = [&](uint32_t rr) {
        if (rr + AHEAD < nproc) {
            const uint32_t dst = stage_at((rr + AHEAD) & (NS - 1u));
            if (rr + AHEAD < nfull) {
                lean_copy_round(dst, src);
            } else {
                const uint32_t bytes = part_valid * (uint32_t)sizeof(T);
                const uint32_t b0 = min(bytes, 16u), b1 = bytes > 16u ? bytes - 16u : 0u;
                // (A source of zero bytes is never read; it still has to be an address.)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst),
                             "l"(b0 ? src : src0), "r"(b0)
                             : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst + 16u),
                             "l"(b1 ? src + 16 : src0), "r"(b1)
                             : "memory");
            }
        }
        cp_async_commit();
        src += ROUND_BYTES;
        cp_async_wait<AHEAD>();
    };
    auto read_round = [&](uint32_t rr, Frag &cur) -> bool {
        lean_read_slot(stage_at(rr & (NS - 1u)), cur);
        if (rr == nfull) {
            frag_mask_tail<T>(cur, part_valid);
            return part_valid != 0u;
        }
        return true;
    };
    auto track = [&](const Frag &cur, uint32_t rr) {
        const float m = frag_max<T>(cur);
        saw_nan |= m != m ? 1u : 0u;
        if (sums) {
            running_sum_add<T>(rs, cur, m, sum_scale);
        }
        // The three best fragments by maximum (rounds best_r, r2, r3) and the
        // largest maximum among all the others (m4).
        if (best_r == NONE || m > best) {
            m4 = fmaxf(m4, m3);
            m3 = m2;
            r3 = r2;
            m2 = best;
            r2 = best_r;
            best = m;
            best_r = rr;
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
    };

    uint32_t rr = 0;
    // Rounds that also mark history ids (HQ 16-byte loads per thread, one round ahead).
    if (mark_rounds != 0u) {
        const uint4 no_ids = make_uint4(NONE, NONE, NONE, NONE);
        uint32_t hnext = tid;
        uint4 hq[HQ];
#pragma unroll
        for (uint32_t j = 0; j < HQ; ++j) {
            hq[j] = hnext + j * NT < n4 ? __ldg(h4 + hnext + j * NT) : no_ids;
        }
        hnext += HQ * NT;
        for (; rr < mark_rounds; ++rr) {
            advance(rr);
            {
                uint32_t ids[4u * HQ];
#pragma unroll
                for (uint32_t j = 0; j < HQ; ++j) {
                    ids[4u * j] = hq[j].x;
                    ids[4u * j + 1u] = hq[j].y;
                    ids[4u * j + 2u] = hq[j].z;
                    ids[4u * j + 3u] = hq[j].w;
                    hq[j] = hnext + j * NT < n4 ? __ldg(h4 + hnext + j * NT) : no_ids;
                }
                hnext += HQ * NT;
#pragma unroll
                for (uint32_t i = 0; i < 4u * HQ; ++i) {
                    if (ids[i] < vocab) {
                        asm volatile("red.shared.or.b32 [%0], %1;" ::"r"(seen_at + (ids[i] >> 5) * 4u),
                                     "r"(1u << (ids[i] & 31u))
                                     : "memory");
                    }
                }
            }
            Frag cur;
            read_round(rr, cur);  // (a full round: mark_rounds < nfull)
            track(cur, rr);
        }
    }
    mbar_arrive(&sm->mbar[0]);  // this thread's history marks are in place
    // Rounds up to the one after which the threshold is taken.
    for (; rr <= r_check; ++rr) {
        advance(rr);
        Frag cur;
        read_round(rr, cur);
        track(cur, rr);
    }
    {
        // The threshold, this warp's share: every thread adjusts its largest logit
        // so far; the warp's best eight keys go to the pool.
        const bool ok = mbar_wait_first(&sm->mbar[0]);
        uint32_t key = 0u;
        if (!ok || saw_nan != 0u || best_r == NONE) {
            sm->lean_abort = 1u;
        } else {
            uint32_t at = 0;
#pragma unroll
            for (int e = (int)GROUP - 1; e >= 0; --e) {
                if (frag_get<T>(keep, e) == best) {
                    at = (uint32_t)e;
                }
            }
            key = adjusted_key(sm, best_r * ROUND + tid * GROUP + at, best, false);
        }
        __syncwarp();
        key = warp_sort_desc(key);
        uint32_t *pool = sm->thist;  // POOL words
        if ((tid & 31u) < POOL_PER_WARP) {
            pool[(tid >> 5) * POOL_PER_WARP + (tid & 31u)] = key;
        }
        __syncwarp();
        if ((tid & 31u) == 0u) {
            mbar_arrive(&sm->mbar[1]);
        }
    }
    // Rounds until every warp's keys are in the pool.
    bool pooled = __all_sync(0xFFFFFFFFu, mbar_test_first(&sm->mbar[1]));
    for (; rr < nproc && !pooled; ++rr) {
        advance(rr);
        Frag cur;
        if (read_round(rr, cur)) {
            track(cur, rr);
        }
        pooled = __all_sync(0xFFFFFFFFu, mbar_test_first(&sm->mbar[1]));
    }
    if (!pooled) {
        // The stream ended first (every warp passes the round above on its own).
        cp_async_wait<0>();
        pooled = __all_sync(0xFFFFFFFFu, mbar_wait_first(&sm->mbar[1]));
    }
    bool gave_up = !pooled || *reinterpret_cast<volatile uint32_t *>(&sm->lean_abort) != 0u;
    float c_fix = 0.0f;
    if (!gave_up) {
        // Every warp takes the bound for itself (the same pool, the same result).
        const uint32_t kth = pool_kth(sm->thist, k);
        const uint32_t kstar = kth > 0u ? kth - 1u : 0u;  // ties with the k-th value must still pass
        c_fix = raw_threshold(kstar, sm->ctx.T, sm->ctx.argmax_mode);
        if (tid == 0) {
            raise_threshold(sm, c_fix, kstar);  // kstar: for the selection after the stream
            if (stamps) {
                stamps[PH_SPARE0] = global_ns();
            }
        }
        // What the rounds [0, rr) of this thread hold above the bound: its best
        // fragment is still in registers; a second or third is read again (L2 by
        // now; the partial round ends anywhere, so it comes element by element).
        const uint32_t base0 = tid * GROUP;
        auto valid_of = [&](uint32_t r) -> uint32_t { return r < nfull ? 0xFFFFFFFFu : (1u << part_valid) - 1u; };
        auto reread = [&](uint32_t r, Frag &f) {
            if (r < nfull) {
                const uint4 *p = reinterpret_cast<const uint4 *>(src0 + (size_t)r * ROUND_BYTES);
                f.v[0] = __ldcg(p);
                f.v[1] = __ldcg(p + 1);
            } else {
                f.v[0] = make_uint4(0, 0, 0, 0);
                f.v[1] = make_uint4(0, 0, 0, 0);
                const T *p = reinterpret_cast<const T *>(src0 + (size_t)r * ROUND_BYTES);
                uint32_t *w = reinterpret_cast<uint32_t *>(&f);
                for (uint32_t e = 0; e < part_valid; ++e) {
                    if (sizeof(T) == 4) {
                        w[e] = __float_as_uint(widen(p[e]));
                    } else {
                        const uint32_t b = reinterpret_cast<const uint16_t *>(p)[e];
                        w[e >> 1] |= (e & 1u) ? (b << 16) : b;
                    }
                }
                frag_mask_tail<T>(f, part_valid);
            }
        };
        if (best_r != NONE && !(best <= c_fix)) {
            lean_take<T>(sm, keep, base0 + best_r * ROUND, valid_of(best_r), c_fix);
        }
        const bool second = r2 != NONE && !(m2 <= c_fix);
        const bool third = r3 != NONE && !(m3 <= c_fix);
        Frag f2, f3;
        if (second) {
            reread(r2, f2);
        }
        if (third) {
            reread(r3, f3);
        }
        if (second) {
            lean_take<T>(sm, f2, base0 + r2 * ROUND, valid_of(r2), c_fix);
        }
        if (third) {
            lean_take<T>(sm, f3, base0 + r3 * ROUND, valid_of(r3), c_fix);
        }
        if (!(m4 <= c_fix)) {
            // Very rare: a fourth fragment of this thread may matter.
            for (uint32_t r = 0; r < rr; ++r) {
                if (r == best_r || r == r2 || r == r3) {
                    continue;
                }
                Frag f;
                reread(r, f);
                if (!(frag_max<T>(f) <= c_fix)) {
                    lean_take<T>(sm, f, base0 + r * ROUND, valid_of(r), c_fix);
                }
            }
        }
        if (stamps && tid == 0) {
            stamps[PH_SPARE1] = global_ns();
        }
        // The remaining rounds: every fragment straight against the bound.
        for (; rr < nproc; ++rr) {
            advance(rr);
            Frag cur;
            if (read_round(rr, cur)) {
                const float m = frag_max<T>(cur);
                saw_nan |= m != m ? 1u : 0u;
                if (sums) {
                    running_sum_add<T>(rs, cur, m, sum_scale);
                }
                if (!(m <= c_fix)) {
                    lean_take<T>(sm, cur, rr * ROUND + tid * GROUP, valid_of(rr), c_fix);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (stamps && tid == 0) {
        stamps[PH_PASS1] = global_ns();
    }
    // A NaN anywhere, a wait that gave up, more ties around the bound than the
    // small buffer takes: the row goes to the general code as it came.
    const bool redo = __syncthreads_or(gave_up || saw_nan != 0u) ||
                      *reinterpret_cast<volatile uint32_t *>(&sm->overflow) != 0u;
    n_raw = min(*reinterpret_cast<volatile uint32_t *>(&sm->n), LCAP);
    if (stamps && tid == 0) {
        stamps[PH_PASS1_MET] = global_ns();
    }
    mine = !redo && n_raw <= (uint32_t)NT;
    }
    if (!mine) {
        cp_async_wait<0>();
        __syncthreads();
        sample_whole_row<T>(a, row);
        if (sums) {
            __syncthreads();
            const float top = a.cand_out[row].max_adj;  // (written by this block, by thread 0 among others)
            const float total = reread_sum<T>(sm, row_ptr, a.vocab, sum_scale, top * 1.4426950408889634f);
            if (tid == 0) {
                a.cand_out[row].sum_exp = total;
            }
        }
        return;
    }

    // ---- selection and draw
    const uint32_t n = small_select(sm, n_raw, k);
    if (stamps && tid == 0) {
        stamps[PH_LOCAL_SELECT] = global_ns();
    }
    if (a.cand_out) {
        float total = 0.0f;
        if (sums && n != 0u) {
            total = running_sum_total(sm, rs, float_of_key(sm->key[0]) * 1.4426950408889634f);
        }
        if (n == 0u) {
            empty_record(sm->err ? sm->err : ROW_INTERNAL);
        } else if (tid < 32u) {
            // The sorted candidates are the row's record (ids in the whole vocabulary's numbering).
            ShardRecord *rec = a.cand_out + row;
            for (uint32_t i = tid; i < LILY_SHARD_CANDIDATES; i += 32u) {
                rec->cand[i] = i < n ? make_uint2(sm->key[i], sm->id[i] + a.id_offset) : make_uint2(0u, 0xFFFFFFFFu);
            }
            if (tid == 0) {
                rec->max_adj = float_of_key(sm->key[0]);
                rec->sum_exp = total;
                if (sm->err) {
                    atomicOr(a.status_word, 1u << (sm->err & 31u));
                }
                if (stamps) {
                    stamps[PH_END] = global_ns();
                }
            }
        }
        return;
    }
    if (n == 0u) {
        // Nothing reached the buffer (a bug, never expected): an error row.
        if (tid == 0) {
            const uint32_t err = sm->err ? sm->err : ROW_INTERNAL;
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
    if (tid < 32u) {
        finalize_warp(sm, a, row, n, P.seed);
        if (stamps && tid == 0) {
            stamps[PH_END] = global_ns();
        }
    }
}

}  // namespace lily
