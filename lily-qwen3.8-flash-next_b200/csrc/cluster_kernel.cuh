// The small-batch kernel: a thread-block cluster of eight per row.
//
// A decode step of a few rows is all latency: the whole batch is a megabyte,
// 0.2 us of HBM time. What counts is how many dependent steps lie between the
// launch and the token, and how many SMs share a row's work. Here a row is
// spread over a cluster of eight blocks that talk through distributed shared
// memory: no global scratch, no ticket, nothing is read twice.
//
//   1. each block loads its eighth of the row into shared memory as f32, and
//      counts the history ids that fall into its range into a count table in
//      shared memory (one shared-memory atomic per distinct id of a
//      warp's 32 ids: real histories repeat a few ids very often);
//   2. bias entries are added in place in list order, banned ids become -inf in
//      place, then the penalties are applied to EVERY logit of the slice: no
//      thresholds, no second pass. The division by the temperature keeps the
//      order, so the selection works on the values before it and only the
//      candidates are divided;
//   3. the cluster agrees on the row's largest such value (one exchange); every
//      block bins its values by their distance from it (32 bins per unit, 1024
//      bins) into a shared-memory histogram;
//   4. every block adds the eight histograms up for itself (distributed shared
//      memory reads) and finds the bin in which the count from the top reaches
//      k. The candidates are the values down to one bin past it (the margin
//      catches a value that rounds to the same quotient as the k-th): k plus a
//      handful. The summed histogram also says where each bin's candidates go
//      in the order of the bins, and the other blocks' histograms where this
//      block's share of a bin starts;
//   5. every block writes its candidates (divided, as key << 32 | ~id) to those
//      places in all eight blocks, ranks each of its own against the few others
//      of the same bin ((key descending, id ascending), as the reference's CPU
//      sampler orders them) and stores those of rank below k at their rank in
//      the leader's shared memory;
//   6. the leader runs the softmax weights, the sequential prefix sums in rank
//      order, the top-p / min-p cut and the draw (tests/unit/kernels/
//      sample.rs:8-54 of the reference), and writes the outputs.
//
// Every block of a cluster passes the same cluster barriers the same number of
// times: all decisions between the first and the last barrier are taken from
// data every block of the cluster has. A row this kernel does not take (a
// vocabulary, history or list beyond its shared memory, a value range that
// leaves more candidates than its buffers hold) is drawn by the leader alone
// with the general row code of sample_rows_kernel.
#pragma once

#include <cooperative_groups.h>

#include "sample_kernel.cuh"

namespace lily {

namespace cgx = cooperative_groups;

constexpr uint32_t CL = 8;                   // blocks per row (the portable cluster size)
constexpr uint32_t CL_SLICE_MAX = 20480;     // logits per block: 80 KB as f32 and as much for their counts
constexpr uint32_t CL_BINS = 1024;
constexpr float CL_BINS_PER_UNIT = 32.0f;    // of logit: the histogram spans 32 units below the top
constexpr float CL_TOP_MAX = 65536.0f;       // beyond it a bin is no wider than a rounding step: the general code
constexpr uint32_t CL_CAND = 1536;           // candidates of a row, k = 1024 plus what shares the last bin
constexpr uint32_t CL_LIST = SP_SMEM;        // bias + ban entries staged in shared memory
constexpr uint32_t CL_MAX_ROWS = 8;          // rows whose parameters travel in the kernel's arguments

struct alignas(16) ClusterSmem {
    uint32_t hist[CL_BINS];            // this block's histogram, read by the whole cluster; then fill[]: this
                                       //   block's candidates placed so far, per bin
    uint32_t ghist[CL_BINS];           // the cluster's sum
    uint32_t pre[CL_BINS];             // candidates in the bins before a bin; later the leader's weights p
    uint32_t boff[CL_BINS];            // of a bin, what the blocks of lower rank hold; later the prefix sums
    unsigned long long cand[CL_CAND];  // every candidate of the row in bin order: key << 32 | ~id
    uint32_t myslot[CL_CAND];          // this block's candidates: place in cand[] | bin << 16
    unsigned long long sorted[KCAP];   // leader: the best k in rank order
    float cmax[CL];                    // each block's largest value
    uint32_t cerr[CL];                 // each block's error word
    uint32_t warp_sums[NT / 32];
    float warp_max[NT / 32];
    alignas(16) uint32_t sp_ids[CL_LIST + 4];
    float sp_vals[CL_LIST];
    uint32_t n_mine;
    uint32_t bstar;
    uint32_t err;
    uint32_t n_keep;
    uint32_t chosen;
};
static_assert(CL_CAND <= 65536u && CL_BINS <= 65536u, "place and bin share a word");
static_assert(CL_BINS >= KCAP, "p and the prefix sums fit pre[] and boff[]");

// The two arrays behind the fixed part: the slice as f32 (later its adjusted
// values) and its counts.
__host__ __device__ inline uint32_t cluster_slice_len(uint32_t vocab) {
    const uint32_t per = (vocab + CL - 1u) / CL;
    return (per + 15u) & ~15u;
}

__host__ __device__ inline size_t cluster_smem_bytes(uint32_t vocab) {
    const size_t sl = cluster_slice_len(vocab);
    return sizeof(ClusterSmem) + sl * 4u + sl * 4u + 16u;
}

// The bin of value q under the row's largest one: 0 holds the top.
__device__ __forceinline__ uint32_t cluster_bin(float q, float top) {
    if (q == top) {
        return 0u;
    }
    const float d = __fmul_rn(__fsub_rn(top, q), CL_BINS_PER_UNIT);
    return d < (float)(CL_BINS - 1u) ? (uint32_t)d : CL_BINS - 1u;  // (a NaN lands in the last bin)
}

struct ClusterArgs {
    KArgs a;
    // Host parameters of up to CL_MAX_ROWS rows travel here, in the kernel's
    // arguments: no staging copy in front of the launch, no DRAM round trip in it.
    lily_sampling_params_t params[CL_MAX_ROWS];
    uint32_t steps[CL_MAX_ROWS];
    uint32_t slots[CL_MAX_ROWS];
    uint32_t inline_params;  // params / steps above are valid (else a.params / a.steps on the device)
    uint32_t inline_slots;   // slots above are the rows' histogram slots (else a.count_slots, or none)
    // Device words of the handle, CL_MAX_ROWS each: where the leader puts a row's
    // parameters when it hands the row to the general code, which reads them
    // from device memory.
    lily_sampling_params_t *spill_params;
    uint32_t *spill_steps;
    uint32_t *spill_slots;
};

// The leader's last step on the best n candidates in rank order (sorted[]): the
// softmax weights, the prefix sums in rank order, one rounding per add
// (tests/unit/kernels/sample.rs:37-46), the cut, the draw, the outputs.
__device__ __forceinline__ void cluster_finalize(ClusterSmem *sm, const KArgs &a, uint32_t row, uint32_t n,
                                                 float top_p, float min_p, bool argmax_mode, bool count_draw,
                                                 uint32_t slot, float u) {
    const uint32_t tid = threadIdx.x;
    float *p = reinterpret_cast<float *>(sm->pre);
    float *cum = reinterpret_cast<float *>(sm->boff);
    const uint32_t top_key = (uint32_t)(sm->sorted[0] >> 32);
    const float top = float_of_key(top_key);
    if (argmax_mode) {
        if (tid == 0) {
            const uint32_t id = ~(uint32_t)sm->sorted[0];
            a.out_ids[row] = id;
            if (a.out_status) {
                a.out_status[row] = LILY_ROW_OK;
            }
            if (a.kept_n) {
                a.kept_n[row] = 1;
                a.kept_ids[(uint64_t)row * a.kept_ld] = id;
                a.kept_probs[(uint64_t)row * a.kept_ld] = 1.0f;
            }
        }
        return;
    }
    for (uint32_t i = tid; i < n; i += NT) {
        p[i] = exp_f32(__fsub_rn(float_of_key((uint32_t)(sm->sorted[i] >> 32)), top));
    }
    __syncthreads();
    if (tid == 0) {
        // One thread, rank order. The loads run ahead of the chain of adds.
        float s = 0.0f;
        uint32_t i = 0;
        for (; i + 8u <= n; i += 8u) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = p[i + j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s = __fadd_rn(s, v[j]);
                cum[i + j] = s;
            }
        }
        for (; i < n; ++i) {
            s = __fadd_rn(s, p[i]);
            cum[i] = s;
        }
        sm->n_keep = n;
    }
    __syncthreads();
    const float limit = __fmul_rn(top_p, cum[n - 1u]);
    for (uint32_t i = tid + 1u; i < n; i += NT) {
        if (!(cum[i - 1u] < limit && p[i] >= min_p)) {
            atomicMin(&sm->n_keep, i);
        }
    }
    __syncthreads();
    const uint32_t n_keep = sm->n_keep;
    const float mass = cum[n_keep - 1u];
    if (a.kept_n) {
        for (uint32_t i = tid; i < n_keep; i += NT) {
            a.kept_ids[(uint64_t)row * a.kept_ld + i] = ~(uint32_t)sm->sorted[i];
            a.kept_probs[(uint64_t)row * a.kept_ld + i] = __fdiv_rn(p[i], mass);
        }
        if (tid == 0) {
            a.kept_n[row] = n_keep;
        }
    }
    // First kept rank whose prefix sum exceeds the target, else the last one.
    const float target = __fmul_rn(u, mass);
    if (tid == 0) {
        sm->chosen = n_keep - 1u;
    }
    __syncthreads();
    for (uint32_t i = tid; i < n_keep; i += NT) {
        if (target < cum[i]) {
            atomicMin(&sm->chosen, i);
        }
    }
    __syncthreads();
    if (tid == 0) {
        const uint32_t id = ~(uint32_t)sm->sorted[sm->chosen];
        a.out_ids[row] = id;
        if (a.out_status) {
            a.out_status[row] = LILY_ROW_OK;
        }
        if (count_draw && id < a.vocab) {
            // src/kernels/metal/sample.metal:509-511: the draw is counted.
            atomicAdd(a.counts_table + (uint64_t)slot * a.vocab + id, 1u);
            atomicOr(a.seen_table + (uint64_t)slot * a.seen_words + (id >> 5), 1u << (id & 31u));
        }
    }
}

// Grid (CL, rows), cluster (CL, 1, 1), NT threads, dynamic shared memory
// max(cluster_smem_bytes, what the general row code needs).
template <typename T>
__global__ void __launch_bounds__(NT, 1) cluster_rows_kernel(const __grid_constant__ ClusterArgs ca) {
    const KArgs &a = ca.a;
    extern __shared__ uint4 smem_raw[];
    ClusterSmem *sm = reinterpret_cast<ClusterSmem *>(smem_raw);
    cgx::cluster_group cluster = cgx::this_cluster();
    constexpr uint32_t NONE = 0xFFFFFFFFu;
    constexpr unsigned FULL = 0xFFFFFFFFu;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rank = cluster.block_rank();
    const uint32_t row = a.row0 + blockIdx.y;
    const uint32_t vocab = a.vocab;
    const uint32_t sl = cluster_slice_len(vocab);
    float *vals = reinterpret_cast<float *>(sm + 1);
    uint32_t *cnt = reinterpret_cast<uint32_t *>(vals + sl);
    const uint32_t lo = min(vocab, rank * sl), hi = min(vocab, lo + sl), len = hi - lo;
    long long *stamps =
        a.phase_clocks ? a.phase_clocks + ((uint64_t)row * MAX_SLICES + rank) * LILY_PHASES : nullptr;
    if (stamps && tid == 0) {
        stamps[PH_ENTRY] = global_ns();
    }
#define CL_STAMP(i)                      \
    do {                                 \
        if (stamps && tid == 0) {        \
            stamps[(i)] = global_ns();   \
        }                                \
    } while (0)

    // What needs no input comes first (see sample_row on the launch attribute).
    for (uint32_t b = tid; b < CL_BINS; b += NT) {
        sm->hist[b] = 0;
    }
    for (uint32_t i = tid; i < sl; i += NT) {
        cnt[i] = 0;
    }
    if (tid == 0) {
        sm->n_mine = 0;
        sm->err = 0;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- the row's parameters; rows that end here (every block of the cluster alike)
    const uint32_t hist_len_row = (a.history_ids && a.history_len) ? __ldg(a.history_len + row) : 0u;
    const int32_t forced = a.forced_ids ? __ldg(a.forced_ids + row) : -1;
    const uint32_t n_bias = (a.bias_ids && a.bias_len) ? __ldg(a.bias_len + row) : 0u;
    const uint32_t n_ban = (a.ban_ids && a.ban_len) ? __ldg(a.ban_len + row) : 0u;
    const bool table_mode = ca.inline_slots != 0u || a.count_slots != nullptr;
    const uint32_t slot = ca.inline_slots ? ca.slots[blockIdx.y] : (a.count_slots ? __ldg(a.count_slots + row) : 0u);
    lily_sampling_params_t P;
    uint32_t step = 0;
    if (a.force_greedy) {
        P.temperature = 0.0f;
        P.top_k = 1;
        P.top_p = 1.0f;
        P.min_p = 0.0f;
        P.presence_penalty = 0.0f;
        P.frequency_penalty = 0.0f;
        P.repetition_penalty = 1.0f;
        P.seed = 0;
    } else if (ca.inline_params) {
        P = ca.params[blockIdx.y];
        step = ca.steps[blockIdx.y];
    } else {
        P = a.params[row];
        step = a.steps ? a.steps[row] : 0u;
    }
    const float u = a.uniforms ? __ldg(a.uniforms + row) : uniform_for(P.seed, step);
    const T *row_ptr = reinterpret_cast<const T *>(a.logits) + (uint64_t)row * a.logits_ld;
    // ---- 1. the slice into shared memory as f32. It does not depend on the row's
    // parameters, whose loads (above) are still on their way.
    {
        constexpr uint32_t PER = 16u / (uint32_t)sizeof(T);
        const T *src = row_ptr + lo;
        const uint32_t nvec = len / PER;
        for (uint32_t v = tid; v < nvec; v += NT) {
            const uint4 q = __ldg(reinterpret_cast<const uint4 *>(src) + v);
            float4 *dst = reinterpret_cast<float4 *>(vals + (size_t)v * PER);
            if (sizeof(T) == 4) {
                dst[0] = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z),
                                     __uint_as_float(q.w));
            } else {
                dst[0] = make_float4(bf16_lo(q.x), bf16_hi(q.x), bf16_lo(q.y), bf16_hi(q.y));
                dst[1] = make_float4(bf16_lo(q.z), bf16_hi(q.z), bf16_lo(q.w), bf16_hi(q.w));
            }
        }
        for (uint32_t i = nvec * PER + tid; i < len; i += NT) {
            vals[i] = widen(src[i]);
        }
    }

    auto refuse = [&](uint32_t status) {
        if (rank == 0 && tid == 0) {
            a.out_ids[row] = status == LILY_ROW_FORCED ? (uint32_t)forced : 0xFFFFFFFFu;
            if (a.out_status) {
                a.out_status[row] = status;
            }
            if (a.kept_n) {
                a.kept_n[row] = 0;
            }
            if (status != LILY_ROW_FORCED) {
                atomicOr(a.status_word, 1u << (status & 31u));
            }
        }
    };
    // The leader alone, with the general row code on the whole row.
    auto leader_draws_alone = [&]() {
        if (rank == 0) {
            KArgs whole = a;
            whole.n_slices = 1;
            if (ca.inline_params) {
                if (tid == 0) {
                    ca.spill_params[blockIdx.y] = P;
                    ca.spill_steps[blockIdx.y] = step;
                }
                whole.params = ca.spill_params - a.row0;
                whole.steps = ca.spill_steps - a.row0;
            }
            if (ca.inline_slots) {
                if (tid == 0) {
                    ca.spill_slots[blockIdx.y] = slot;
                }
                whole.count_slots = ca.spill_slots - a.row0;
            }
            __threadfence();
            __syncthreads();
            sample_whole_row<T>(whole, row);
        }
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
        n_bias > a.max_list || (a.bias_ld != 0u && n_bias > a.bias_ld) || n_ban > a.max_list ||
        (a.ban_ld != 0u && n_ban > a.ban_ld)) {
        refuse(LILY_ROW_LIST);
        return;
    }
    const bool greedy = P.temperature <= 0.0f || P.top_k == 1u;
    const bool use_pen = P.presence_penalty != 0.0f || P.frequency_penalty != 0.0f ||
                         P.repetition_penalty != 1.0f;
    const float temp = greedy ? 1.0f : P.temperature;
    const uint32_t k = greedy ? 1u : (P.top_k == 0u ? KCAP : min(P.top_k, KCAP));
    const uint32_t n_sp = n_bias + n_ban;
    const bool argmax_mode = greedy && !use_pen && n_sp == 0u;
    if (n_sp > CL_LIST || sl > CL_SLICE_MAX || row < a.spec.n_spec || a.extra_len != 0u) {
        leader_draws_alone();
        return;
    }

    // ---- 1b. the history into the count table
    cluster.sync();  // 0: every block of the cluster is running, its count table zeroed
    CL_STAMP(0);
    const bool scattered = use_pen && !table_mode && hist_len_row != 0u;
    // (The lists first: their loads are on their way while the history is counted.)
    if (n_sp != 0u) {
        for (uint32_t j = tid; j < n_sp; j += NT) {
            sm->sp_ids[j] = j < n_bias ? a.bias_ids[(uint64_t)row * a.bias_ld + j]
                                       : a.ban_ids[(uint64_t)row * a.ban_ld + (j - n_bias)];
            sm->sp_vals[j] = j < n_bias ? a.bias_vals[(uint64_t)row * a.bias_ld + j] : 0.0f;
        }
    }
    if (use_pen) {
        if (table_mode) {
            const uint32_t *src = a.counts_table + (uint64_t)slot * vocab + lo;
            for (uint32_t i = tid; i < len; i += NT) {
                cnt[i] = src[i];
            }
        } else if (hist_len_row != 0u) {
            // Each block takes an eighth of the LIST, whatever ids it holds, and adds
            // into the count table of the block that owns an id (a real history
            // repeats a few ids very often, and they all live in one block's range:
            // this spreads the work of counting them). One atomic per distinct id of
            // a warp's 32.
            const uint32_t *hist = a.history_ids + (uint64_t)row * a.history_ld;
            const uint32_t share = (hist_len_row + CL - 1u) / CL;
            const uint32_t h_lo = min(hist_len_row, rank * share), h_hi = min(hist_len_row, h_lo + share);
            constexpr uint32_t HB = 4;  // loads in flight per thread
            for (uint32_t i0 = h_lo; i0 < h_hi; i0 += NT * HB) {
                uint32_t ids[HB];
#pragma unroll
                for (uint32_t j = 0; j < HB; ++j) {
                    const uint32_t i = i0 + j * NT + tid;
                    ids[j] = i < h_hi ? __ldg(hist + i) : NONE;
                }
#pragma unroll
                for (uint32_t j = 0; j < HB; ++j) {
                    const bool in = ids[j] < vocab;
                    const unsigned live = __ballot_sync(FULL, in);
                    if (in) {
                        const unsigned peers = __match_any_sync(live, ids[j]);
                        if (lane == (uint32_t)(__ffs(peers) - 1)) {
                            const uint32_t owner = ids[j] / sl;
                            atomicAdd(cluster.map_shared_rank(cnt, owner) + (ids[j] - owner * sl),
                                      (uint32_t)__popc(peers));
                        }
                    }
                }
            }
        }
    }
    if (scattered) {
        cluster.sync();  // every block's counts have arrived
    } else {
        __syncthreads();
    }
    CL_STAMP(1);

    // ---- 2. bias in list order (duplicates add), then bans, in place
    if (n_sp != 0u) {
        for (uint32_t j = tid; j < n_bias; j += NT) {
            const uint32_t id = sm->sp_ids[j];
            const uint32_t off = id - lo;
            if (off < len) {
                // The first entry of an id adds every entry of that id, in list order.
                uint32_t earlier = 0;
#pragma unroll 8
                for (uint32_t e = 0; e < j; ++e) {
                    earlier += sm->sp_ids[e] == id ? 1u : 0u;
                }
                if (earlier == 0u) {
                    float x = __fadd_rn(vals[off], sm->sp_vals[j]);
                    uint32_t later = 0;
#pragma unroll 8
                    for (uint32_t e = j + 1u; e < n_bias; ++e) {
                        later += sm->sp_ids[e] == id ? 1u : 0u;
                    }
                    if (later != 0u) {
                        for (uint32_t e = j + 1u; e < n_bias; ++e) {
                            if (sm->sp_ids[e] == id) {
                                x = __fadd_rn(x, sm->sp_vals[e]);
                            }
                        }
                    }
                    vals[off] = x;
                }
            }
        }
        __syncthreads();
        // (A banned id ends at -inf whatever the penalties make of it: -inf stays -inf
        // under a positive repetition factor and a finite subtraction.)
        for (uint32_t j = n_bias + tid; j < n_sp; j += NT) {
            const uint32_t off = sm->sp_ids[j] - lo;
            if (off < len) {
                vals[off] = neg_inf();
            }
        }
        __syncthreads();
    }

    CL_STAMP(2);
    // ---- 3. the penalties on every logit; the block's largest value
    float tmax = neg_inf();
#pragma unroll 4
    for (uint32_t i = tid; i < len; i += NT) {
        float x = vals[i];
        if (use_pen) {
            const uint32_t c = cnt[i];
            if (c != 0u) {
                if (P.repetition_penalty != 1.0f) {  // (x / 1 and x * 1 are x)
                    x = x > 0.0f ? __fdiv_rn(x, P.repetition_penalty) : __fmul_rn(x, P.repetition_penalty);
                }
                x = __fsub_rn(x, __fadd_rn(P.presence_penalty, __fmul_rn(P.frequency_penalty, (float)c)));
                vals[i] = x;
            }
        }
        if (x != x) {
            if (argmax_mode) {
                // NaN never wins (src/kernels/metal/elementwise.metal:145-150).
                x = neg_inf();
                vals[i] = x;
            } else {
                sm->err = LILY_ROW_NAN;
            }
        }
        tmax = fmaxf(tmax, x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        tmax = fmaxf(tmax, __shfl_xor_sync(FULL, tmax, o));
    }
    if (lane == 0) {
        sm->warp_max[warp] = tmax;
    }
    __syncthreads();
    if (tid < CL) {
        float bm = neg_inf();
        for (uint32_t w = 0; w < NT / 32; ++w) {
            bm = fmaxf(bm, sm->warp_max[w]);
        }
        cluster.map_shared_rank(sm->cmax, tid)[rank] = bm;
        cluster.map_shared_rank(sm->cerr, tid)[rank] = sm->err;
    }
    CL_STAMP(2);
    cluster.sync();  // 1: every block has every block's maximum and error word
    CL_STAMP(3);
    float top = neg_inf();
    uint32_t err = 0;
    for (uint32_t r = 0; r < CL; ++r) {
        top = fmaxf(top, sm->cmax[r]);
        err |= sm->cerr[r];
    }
    if (err != 0u) {
        refuse(LILY_ROW_NAN);
        return;
    }
    if (top == neg_inf() || top == -neg_inf()) {
        if (argmax_mode) {
            leader_draws_alone();  // (every logit -inf or NaN, or a +inf: the general code's rules)
        } else {
            refuse(LILY_ROW_NONFINITE);
        }
        return;
    }
    if (!(fabsf(top) < CL_TOP_MAX)) {
        leader_draws_alone();
        return;
    }

    // ---- 4. histogram of the distances from the top; the bin where the count reaches k
#pragma unroll 4
    for (uint32_t i = tid; i < len; i += NT) {
        const uint32_t bin = cluster_bin(vals[i], top);
        if (bin != CL_BINS - 1u) {  // (what lies 32 units below the top is never a candidate)
            atomicAdd(&sm->hist[bin], 1u);
        }
    }
    CL_STAMP(9);
    cluster.sync();  // 2: every block's histogram is complete
    CL_STAMP(4);
    {
        constexpr uint32_t BPT = CL_BINS / NT;
        uint32_t v[BPT][CL];
#pragma unroll
        for (uint32_t j = 0; j < BPT; ++j) {
#pragma unroll
            for (uint32_t r = 0; r < CL; ++r) {
                v[j][r] = cluster.map_shared_rank(sm->hist, r)[tid + j * NT];
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < BPT; ++j) {
            uint32_t s = 0, lower = 0;
#pragma unroll
            for (uint32_t r = 0; r < CL; ++r) {
                s += v[j][r];
                lower += r < rank ? v[j][r] : 0u;
            }
            sm->ghist[tid + j * NT] = s;
            sm->boff[tid + j * NT] = lower;
        }
    }
    __syncthreads();
    {
        // Thread t owns BPT neighbouring bins: how many candidates lie in the bins
        // before each, and the bin in which that count, from bin 0 up, reaches k.
        constexpr uint32_t BPT = CL_BINS / NT;
        uint32_t c[BPT], sum = 0;
#pragma unroll
        for (uint32_t j = 0; j < BPT; ++j) {
            c[j] = sm->ghist[tid * BPT + j];
            sum += c[j];
        }
        uint32_t incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(FULL, incl, o);
            if (lane >= (uint32_t)o) {
                incl += t;
            }
        }
        if (lane == 31u) {
            sm->warp_sums[warp] = incl;
        }
        if (tid == 0) {
            sm->bstar = NONE;
        }
        __syncthreads();
        uint32_t cum = incl - sum;
        for (uint32_t w = 0; w < warp; ++w) {
            cum += sm->warp_sums[w];
        }
#pragma unroll
        for (uint32_t j = 0; j < BPT; ++j) {
            sm->pre[tid * BPT + j] = cum;
            if (cum < k && k <= cum + c[j]) {
                sm->bstar = tid * BPT + j;
            }
            cum += c[j];
        }
        __syncthreads();
    }
    const uint32_t bstar = sm->bstar;
    // One bin of margin: a value there may round to the quotient of the k-th.
    const uint32_t blast = bstar == NONE ? NONE : min(bstar + 1u, CL_BINS - 2u);
    const uint32_t n = bstar == NONE ? 0u : sm->pre[blast] + sm->ghist[blast];
    cluster.sync();  // 3: nobody reads another block's histogram any more
    CL_STAMP(5);
    if (bstar == NONE || bstar + 1u > CL_BINS - 2u || n > CL_CAND) {
        // Fewer than k values within 32 units of the top, or too many around the
        // k-th (a flat row, heavy ties): the general code selects without binning.
        leader_draws_alone();
        return;
    }

    // ---- 5. candidates to their places in every block; ranks within the bins
    uint32_t *fill = sm->hist;
    for (uint32_t b = tid; b <= blast; b += NT) {
        fill[b] = 0;
    }
    __syncthreads();
#pragma unroll 4
    for (uint32_t i = tid; i < len; i += NT) {
        const float x = vals[i];
        const uint32_t bin = cluster_bin(x, top);
        if (bin <= blast) {
            float q = __fdiv_rn(x, temp);
            if (argmax_mode) {
                q = __fadd_rn(q, 0.0f);  // the two zeros tie (src/kernels/metal/elementwise.metal:145-150)
            }
            const unsigned long long v = ((unsigned long long)key_of(q) << 32) | (uint32_t)~(lo + i);
            const uint32_t at = sm->pre[bin] + sm->boff[bin] + atomicAdd(&fill[bin], 1u);
            sm->myslot[atomicAdd(&sm->n_mine, 1u)] = at | (bin << 16);
#pragma unroll
            for (uint32_t r = 0; r < CL; ++r) {
                cluster.map_shared_rank(sm->cand, r)[at] = v;
            }
        }
    }
    CL_STAMP(10);
    cluster.sync();  // 4: every block holds all n candidates, grouped by bin
    CL_STAMP(6);
    {
        unsigned long long *leader_sorted = cluster.map_shared_rank(sm->sorted, 0);
        const uint32_t mine_n = sm->n_mine;
        for (uint32_t i = tid; i < mine_n; i += NT) {
            const uint32_t at = sm->myslot[i] & 0xFFFFu, bin = sm->myslot[i] >> 16;
            const unsigned long long me = sm->cand[at];
            const uint32_t first = sm->pre[bin], last = first + sm->ghist[bin];
            uint32_t place = first;
            for (uint32_t j = first; j < last; ++j) {
                place += sm->cand[j] > me ? 1u : 0u;
            }
            // Two values one rounding step apart can sit on the two sides of a bin
            // edge and still divide to the same quotient: then the id decides
            // across the edge as well. (Keys never rise from a bin to the next.)
            if (bin < blast) {
                for (uint32_t j = last; j < last + sm->ghist[bin + 1u]; ++j) {
                    place += sm->cand[j] > me ? 1u : 0u;
                }
            }
            if (bin > 0u) {
                for (uint32_t j = sm->pre[bin - 1u]; j < first; ++j) {
                    place -= sm->cand[j] < me ? 1u : 0u;
                }
            }
            if (place < k) {
                leader_sorted[place] = me;
            }
        }
    }
    CL_STAMP(11);
    cluster.sync();  // 5: the leader holds the best min(n, k) in rank order
    CL_STAMP(8);
    if (rank != 0u) {
        return;
    }

    // ---- 6. the draw
    cluster_finalize(sm, a, row, min(n, k), P.top_p, P.min_p, argmax_mode, use_pen && table_mode, slot, u);
    if (stamps && tid == 0) {
        stamps[PH_END] = global_ns();
    }
}

}  // namespace lily
