// Host side of the C ABI declared in include/lily_sampler.h: argument
// checks, parameter staging, launch geometry. All device work is enqueued on
// the caller's stream; nothing here falls back to the CPU.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/lily_batch.h"
#include "../../include/lily_sampler.h"
#include "sample_kernel.cuh"
#include "stream_kernel.cuh"
#include "cluster_kernel.cuh"
#include "lmhead_kernel.cuh"

namespace {

constexpr int RING = 8;

struct StageLayout {
    size_t params, steps, slots, hist_len, total;
};

StageLayout stage_layout(uint32_t max_rows) {
    StageLayout l;
    size_t off = 0;
    l.params = off;
    off += sizeof(lily_sampling_params_t) * max_rows;
    l.steps = off;
    off += sizeof(uint32_t) * max_rows;
    l.slots = off;
    off += sizeof(uint32_t) * max_rows;
    l.hist_len = off;
    off += sizeof(uint32_t) * max_rows;
    l.total = (off + 255) & ~size_t(255);
    return l;
}

}  // namespace

struct lily_sampler {
    int device = 0;
    uint32_t vocab = 0, max_rows = 0, max_history = 0, max_list = 0, flags = 0;
    std::string last_error;
    int32_t fault = 0;
    uint64_t wait_ns = 1000000000ull;     // bound of the waits inside the LM-head kernel
    uint32_t lost_stage = 0xFFFFFFFFu;    // test hook: a weight copy the next head launch leaves out
    int sm_count = 0;
    int max_smem = 0;
    uint2 *part = nullptr;
    uint32_t *part_n = nullptr;
    uint32_t *tickets = nullptr;
    uint32_t *status_word = nullptr;
    char *spill = nullptr;  // parameters of rows the small-batch kernel hands to the general code
    int max_clusters = -1;  // clusters of the small-batch kernel the GPU runs at once (-1: not asked yet)
    uint32_t *counts_scratch = nullptr;
    uint32_t *counts_table = nullptr;
    uint32_t *seen_table = nullptr;
    uint32_t seen_words = 0;
    StageLayout layout{};
    char *h_stage[RING] = {};
    char *d_stage[RING] = {};
    cudaEvent_t ev[RING] = {};
    int ring_pos = 0;
    uint32_t *h_status = nullptr;
    uint32_t attr_mask = 0;  // kernel variants whose shared-memory limit is raised
    long long *phase_clocks = nullptr;
    // The parameters a sharded call staged last: a decode step stages the same
    // rows for its candidate call and its merge call, and usually again next step.
    uint64_t slot_serial[RING] = {};
    int shard_slot = -1;
    uint64_t shard_serial = 0;
    std::vector<char> shard_bytes;
    float *lm_logits = nullptr;  // LILY_FLAG_LMHEAD: F32 [64, lm_ld]
    uint64_t lm_ld = 0;
    float *lm_hsum = nullptr;    // affine heads: sums of hidden values, F32 [BIAS_MAX_GROUPS, 64]
    bool lm_attr = false, lm_attr_affine = false, lm_attr_q4 = false, lm_attr_bias = false, merge_attr = false;
};

namespace {

int32_t fail(lily_sampler *h, int32_t code, const char *msg) {
    if (h) {
        h->last_error = msg;
    }
    return code;
}

int32_t cuda_fail(lily_sampler *h, cudaError_t e, const char *what) {
    if (h) {
        h->last_error = std::string(what) + ": " + cudaGetErrorString(e);
    }
    return LILY_ERR_CUDA;
}

#define CU(h, call)                              \
    do {                                         \
        cudaError_t e_ = (call);                 \
        if (e_ != cudaSuccess) {                 \
            return cuda_fail((h), e_, #call);    \
        }                                        \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) {
            prev = -1;
        }
        if (prev != dev) {
            ok = cudaSetDevice(dev) == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (prev >= 0) {
            cudaSetDevice(prev);
        }
    }
};

bool params_ok(const lily_sampling_params_t &p) {
    return std::isfinite(p.temperature) && p.temperature >= 0.0f && std::isfinite(p.top_p) &&
           p.top_p > 0.0f && p.top_p <= 1.0f && std::isfinite(p.min_p) && p.min_p >= 0.0f &&
           p.min_p <= 1.0f && std::isfinite(p.repetition_penalty) &&
           p.repetition_penalty > 0.0f && std::isfinite(p.presence_penalty) &&
           std::isfinite(p.frequency_penalty);
}

bool is_greedy(const lily_sampling_params_t &p) {
    return p.temperature <= 0.0f || p.top_k == 1u;
}

bool uses_penalties(const lily_sampling_params_t &p) {
    return p.presence_penalty != 0.0f || p.frequency_penalty != 0.0f ||
           p.repetition_penalty != 1.0f;
}

uint32_t effective_k(const lily_sampling_params_t &p) {
    if (is_greedy(p)) {
        return 1u;
    }
    return p.top_k == 0u ? LILY_K_CAP : (p.top_k < LILY_K_CAP ? p.top_k : LILY_K_CAP);
}

// A staging slot whose previous use has left the stream.
int32_t next_stage(lily_sampler *h, int *slot) {
    const int s = h->ring_pos;
    h->ring_pos = (h->ring_pos + 1) % RING;
    CU(h, cudaEventSynchronize(h->ev[s]));
    ++h->slot_serial[s];
    *slot = s;
    return LILY_OK;
}

size_t smem_bytes(uint32_t vocab, uint32_t n_slices) {
    // The largest slice a row can get is the whole row: a row that keeps many
    // candidates and takes the two-pass route is not cut, whatever n_slices is
    // (the kernel decides per row; the seen bitmap must fit either way).
    (void)n_slices;
    const uint32_t slice_len = (vocab + 255u) & ~255u;
    const size_t words = (slice_len + 31u) / 32u + 8u;
    return sizeof(lily::SmemFixed) + lily::RING_BYTES + words * sizeof(uint32_t);
}

// Programmatic stream serialisation: the grid may be set up and its blocks may
// start while the stream's previous kernel drains; the kernels wait
// (griddepcontrol.wait) before they read or write any global memory.
template <typename Kernel>
int32_t launch_serialised(lily_sampler *h, cudaStream_t stream, Kernel kernel, dim3 grid, size_t smem,
                          const lily::KArgs &a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lily::NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU(h, cudaLaunchKernelEx(&cfg, kernel, a));
    return LILY_OK;
}

template <typename Kernel>
int32_t raise_smem_limit(lily_sampler *h, Kernel kernel, uint32_t bit) {
    if (!(h->attr_mask & bit)) {
        CU(h, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h->max_smem));
        h->attr_mask |= bit;
    }
    return LILY_OK;
}

// Whether a call goes to the kernel of one block per row (see launch_one).
bool stream_route(const lily::KArgs &a, uint32_t rows, uint32_t dtype) {
    const size_t esize = dtype == LILY_F32 ? 4 : 2;
    const bool vec = (reinterpret_cast<uintptr_t>(a.logits) % 16u == 0u) && ((a.logits_ld * esize) % 16u == 0u);
    const uint32_t round = dtype == LILY_F32 ? lily::Geo<float>::ROUND : lily::Geo<__nv_bfloat16>::ROUND;
    return vec && a.vocab / round >= lily::STREAM_MIN_ROUNDS && a.merge_in == nullptr && a.spec.n_spec == 0u &&
           a.extra_len == 0u && rows >= 16u && (a.cand_out == nullptr || a.shard_k <= lily::STREAM_K_MAX);
}

template <typename T, bool VEC>
int32_t launch_one(lily_sampler *h, cudaStream_t stream_, const lily::KArgs &a, uint32_t rows,
                   size_t smem) {
    // More rows than the small-batch kernel takes (and at least 16: fewer rows with
    // lists or wide cuts are better off cut into slices), aligned logits, long rows
    // and nothing special about the call: the kernel of one block per row (which runs
    // the general code itself, on the whole row, for the rows it does not take).
    // Below a block slot's worth of rows a block streams alone, and gets a deeper
    // ring. A vocabulary shard's candidate launch goes the same way and ends in the
    // rows' records. (Short rows, unaligned logits, speculative calls and the merge
    // of shards: the general kernel, rows cut into slices.)
    const bool stream = VEC && stream_route(a, rows, sizeof(T) == 4 ? LILY_F32 : LILY_BF16);
    if (stream) {
        lily::KArgs whole = a;
        whole.n_slices = 1;
        const size_t smem1 = smem_bytes(a.vocab, 1);
        if (rows > (uint32_t)h->sm_count) {
            auto kernel = lily::stream_rows_kernel<T, 2>;
            const int32_t st = raise_smem_limit(h, kernel, 1u << (sizeof(T) == 4 ? 4 : 5));
            if (st != LILY_OK) {
                return st;
            }
            return launch_serialised(h, stream_, kernel, dim3(rows, 1, 1), smem1, whole);
        }
        // A block per SM at most: the deep ring, if the SM's shared memory holds it.
        const size_t deep = ((smem1 + 15u) & ~size_t(15)) + lily::StreamDepth<7>::EXTRA_BYTES;
        if (deep <= (size_t)h->max_smem) {
            auto kernel = lily::stream_rows_kernel<T, 7>;
            const int32_t st = raise_smem_limit(h, kernel, 1u << (sizeof(T) == 4 ? 10 : 11));
            if (st != LILY_OK) {
                return st;
            }
            return launch_serialised(h, stream_, kernel, dim3(rows, 1, 1), deep, whole);
        }
        auto kernel = lily::stream_rows_kernel<T, 3>;
        const int32_t st = raise_smem_limit(h, kernel, 1u << (sizeof(T) == 4 ? 6 : 7));
        if (st != LILY_OK) {
            return st;
        }
        return launch_serialised(h, stream_, kernel, dim3(rows, 1, 1), smem1, whole);
    }
    auto kernel = lily::sample_rows_kernel<T, VEC>;
    const int32_t st = raise_smem_limit(h, kernel, 1u << ((sizeof(T) == 4 ? 0 : 2) + (VEC ? 1 : 0)));
    if (st != LILY_OK) {
        return st;
    }
    return launch_serialised(h, stream_, kernel, dim3(a.n_slices, rows, 1), smem, a);
}

// Whether a call goes to the small-batch kernel (a cluster of eight blocks per
// row): few enough rows for every cluster to have SMs of its own, aligned logits,
// a vocabulary whose eighth fits a block's shared memory, a plain draw.
size_t cluster_launch_smem(uint32_t vocab) {
    const size_t own = lily::cluster_smem_bytes(vocab);
    const size_t general = smem_bytes(vocab, 1);  // the leader may run the general row code
    return own > general ? own : general;
}

// How many clusters of the small-batch kernel run at once: a launch of more
// rows than that would take its rows in turns, which the kernel of one block per
// row does not. (A cluster needs eight free SMs of one GPC.)
int max_active_clusters(lily_sampler *h) {
    if (h->max_clusters < 0) {
        h->max_clusters = 0;
        auto kernel = lily::cluster_rows_kernel<__nv_bfloat16>;
        const size_t smem = cluster_launch_smem(h->vocab);
        if (smem <= (size_t)h->max_smem &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h->max_smem) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(lily::CL, 64, 1);
            cfg.blockDim = dim3(lily::NT, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = lily::CL;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess) {
                h->max_clusters = n;
            }
        }
        (void)cudaGetLastError();
    }
    return h->max_clusters;
}

bool cluster_call(lily_sampler *h, const void *logits, uint64_t logits_ld, uint32_t dtype,
                  uint32_t rows, bool plain) {
    const size_t esize = dtype == LILY_F32 ? 4 : 2;
    const bool vec = (reinterpret_cast<uintptr_t>(logits) % 16u == 0u) && ((logits_ld * esize) % 16u == 0u);
    return plain && vec && lily::cluster_slice_len(h->vocab) <= lily::CL_SLICE_MAX && h->vocab >= 4096u &&
           (int)rows <= max_active_clusters(h);
}

int32_t launch_cluster(lily_sampler *h, cudaStream_t stream, const lily::ClusterArgs &ca_, uint32_t rows,
                       uint32_t dtype) {
    const size_t smem = cluster_launch_smem(ca_.a.vocab);
    if (smem > (size_t)h->max_smem) {
        return fail(h, LILY_ERR_CAPACITY, "vocabulary too large for the small-batch kernel");
    }
    lily::ClusterArgs ca = ca_;
    ca.spill_params = reinterpret_cast<lily_sampling_params_t *>(h->spill);
    ca.spill_steps = reinterpret_cast<uint32_t *>(h->spill + lily::CL_MAX_ROWS * sizeof(lily_sampling_params_t));
    ca.spill_slots = ca.spill_steps + lily::CL_MAX_ROWS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(lily::CL, rows, 1);
    cfg.blockDim = dim3(lily::NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = lily::CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (dtype == LILY_F32) {
        auto kernel = lily::cluster_rows_kernel<float>;
        const int32_t st = raise_smem_limit(h, kernel, 1u << 8);
        if (st != LILY_OK) {
            return st;
        }
        CU(h, cudaLaunchKernelEx(&cfg, kernel, ca));
    } else {
        auto kernel = lily::cluster_rows_kernel<__nv_bfloat16>;
        const int32_t st = raise_smem_limit(h, kernel, 1u << 9);
        if (st != LILY_OK) {
            return st;
        }
        CU(h, cudaLaunchKernelEx(&cfg, kernel, ca));
    }
    return LILY_OK;
}

int32_t launch(lily_sampler *h, cudaStream_t stream, const lily::KArgs &a, uint32_t rows,
               uint32_t dtype) {
    const size_t smem = smem_bytes(a.vocab, a.n_slices);
    if (smem > (size_t)h->max_smem) {
        return fail(h, LILY_ERR_CAPACITY, "vocabulary too large for the shared-memory bitmap");
    }
    const bool plain = a.cand_out == nullptr && a.merge_in == nullptr && a.spec.n_spec == 0u &&
                       a.extra_len == 0u;
    if (cluster_call(h, a.logits, a.logits_ld, dtype, rows, plain)) {
        lily::ClusterArgs ca;
        std::memset(&ca, 0, sizeof(ca));
        ca.a = a;
        return launch_cluster(h, stream, ca, rows, dtype);
    }
    const size_t esize = dtype == LILY_F32 ? 4 : 2;
    const bool vec = (reinterpret_cast<uintptr_t>(a.logits) % 16u == 0u) &&
                     ((a.logits_ld * esize) % 16u == 0u);
    if (dtype == LILY_F32) {
        return vec ? launch_one<float, true>(h, stream, a, rows, smem)
                   : launch_one<float, false>(h, stream, a, rows, smem);
    }
    return vec ? launch_one<__nv_bfloat16, true>(h, stream, a, rows, smem)
               : launch_one<__nv_bfloat16, false>(h, stream, a, rows, smem);
}

uint32_t choose_slices(const lily_sampler *h, uint32_t rows) {
    const uint32_t target = 2u * (uint32_t)h->sm_count;
    uint32_t s = target / rows;
    if (s < 1u) {
        s = 1u;
    }
    if (s > lily::MAX_SLICES) {
        s = lily::MAX_SLICES;
    }
    // Short slices cost more in merging than they save.
    const uint32_t by_len = (h->vocab + lily::MIN_SLICE - 1u) / lily::MIN_SLICE;
    if (s > by_len) {
        s = by_len;
    }
    return s < 1u ? 1u : s;
}

void base_args(const lily_sampler *h, lily::KArgs *a) {
    std::memset(a, 0, sizeof(*a));
    a->vocab = h->vocab;
    a->counts_table = h->counts_table;
    a->seen_table = h->seen_table;
    a->seen_words = h->seen_words;
    a->counts_scratch = h->counts_scratch;
    a->max_history = h->max_history;
    a->max_list = h->max_list;
    a->part = h->part;
    a->part_n = h->part_n;
    a->tickets = h->tickets;
    a->status_word = h->status_word;
    a->phase_clocks = h->phase_clocks;
}

int32_t check_handle(lily_sampler *h) {
    if (h == nullptr) {
        return LILY_ERR_ARG;
    }
    if (h->fault != 0) {
        return fail(h, LILY_ERR_FAULT, "a fault is latched on this sampler");
    }
    return LILY_OK;
}

}  // namespace

extern "C" {

uint32_t lily_abi_version(void) { return LILY_ABI_VERSION; }

int32_t lily_params_validate(const lily_sampling_params_t *p) {
    if (p == nullptr) {
        return LILY_ERR_ARG;
    }
    return params_ok(*p) ? LILY_OK : LILY_ERR_PARAMS;
}

int32_t lily_params_is_greedy(const lily_sampling_params_t *p) { return p && is_greedy(*p); }

int32_t lily_params_uses_penalties(const lily_sampling_params_t *p) {
    return p && uses_penalties(*p);
}

void lily_params_effective(const lily_sampling_params_t *p, float *temperature, uint32_t *top_k) {
    if (p == nullptr) {
        return;
    }
    if (temperature) {
        *temperature = is_greedy(*p) ? 1.0f : p->temperature;
    }
    if (top_k) {
        *top_k = effective_k(*p);
    }
}

void lily_draft_params(const lily_sampling_params_t *p, lily_sampling_params_t *out) {
    if (p == nullptr || out == nullptr) {
        return;
    }
    *out = *p;
    out->presence_penalty = 0.0f;
    out->frequency_penalty = 0.0f;
    out->repetition_penalty = 1.0f;
}

float lily_uniform_for(uint64_t seed, uint32_t step) { return lily::uniform_for(seed, step); }

uint32_t lily_draft_step(uint32_t step) { return step | 0x40000000u; }

uint32_t lily_residual_step(uint32_t step) { return step | 0x80000000u; }

int32_t lily_sampler_create(int32_t device, uint32_t vocab, uint32_t max_rows,
                            uint32_t max_history, uint32_t max_list, uint32_t flags,
                            lily_sampler_t **out) {
    if (out == nullptr || vocab == 0u || max_rows == 0u || max_list > 512u ||
        vocab > (1u << 24)) {
        return LILY_ERR_ARG;
    }
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        return LILY_ERR_CUDA;
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return LILY_ERR_CUDA;
    }
    lily_sampler *h = new (std::nothrow) lily_sampler();
    if (h == nullptr) {
        return LILY_ERR_ARG;
    }
    h->device = device;
    h->vocab = vocab;
    h->max_rows = max_rows;
    h->max_history = max_history;
    h->max_list = max_list;
    h->flags = flags;
    h->seen_words = (vocab + 31u) / 32u;
    h->layout = stage_layout(max_rows);
    auto bail = [&](cudaError_t e, const char *what) {
        std::fprintf(stderr, "lily_sampler_create: %s: %s\n", what, cudaGetErrorString(e));
        lily_sampler_destroy(h);
        return (int32_t)LILY_ERR_CUDA;
    };
    cudaError_t e;
    if ((e = cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device)) !=
        cudaSuccess) {
        return bail(e, "sm count");
    }
    if ((e = cudaDeviceGetAttribute(&h->max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                    device)) != cudaSuccess) {
        return bail(e, "shared memory limit");
    }
    if ((e = cudaMalloc(&h->part, (size_t)max_rows * lily::CAP * sizeof(uint2))) != cudaSuccess) {
        return bail(e, "candidate scratch");
    }
    if ((e = cudaMalloc(&h->part_n, (size_t)max_rows * lily::MAX_SLICES * 4)) != cudaSuccess) {
        return bail(e, "slice counters");
    }
    if ((e = cudaMalloc(&h->tickets, (size_t)max_rows * 4)) != cudaSuccess) {
        return bail(e, "tickets");
    }
    if ((e = cudaMemset(h->tickets, 0, (size_t)max_rows * 4)) != cudaSuccess) {
        return bail(e, "tickets");
    }
    if ((e = cudaMalloc(&h->spill, lily::CL_MAX_ROWS * (sizeof(lily_sampling_params_t) + 8))) != cudaSuccess) {
        return bail(e, "parameter words of the small-batch kernel");
    }
    if ((e = cudaMalloc(&h->status_word, 4)) != cudaSuccess ||
        (e = cudaMemset(h->status_word, 0, 4)) != cudaSuccess) {
        return bail(e, "status word");
    }
    if ((e = cudaMallocHost(&h->h_status, 4)) != cudaSuccess) {
        return bail(e, "status word (host)");
    }
    if ((e = cudaMalloc(&h->lm_hsum, (size_t)lily_head::BIAS_MAX_GROUPS * lily_head::TOK * sizeof(float))) !=
        cudaSuccess) {
        return bail(e, "LM head group sums");
    }
    if (max_history > 0u) {
        // A row with a frequency penalty over a history LIST counts the list's ids
        // into this table and clears it again before the launch ends: all zero
        // between launches. Made here, never inside a draw.
        const size_t bytes = (size_t)max_rows * vocab * sizeof(uint32_t);
        if ((e = cudaMalloc(&h->counts_scratch, bytes)) != cudaSuccess ||
            (e = cudaMemset(h->counts_scratch, 0, bytes)) != cudaSuccess) {
            return bail(e, "count table of the history lists");
        }
    }
    if (flags & LILY_FLAG_COUNTS_TABLE) {
        const size_t cb = (size_t)max_rows * vocab * 4, sb = (size_t)max_rows * h->seen_words * 4;
        if ((e = cudaMalloc(&h->counts_table, cb)) != cudaSuccess ||
            (e = cudaMemset(h->counts_table, 0, cb)) != cudaSuccess ||
            (e = cudaMalloc(&h->seen_table, sb)) != cudaSuccess ||
            (e = cudaMemset(h->seen_table, 0, sb)) != cudaSuccess) {
            return bail(e, "histogram slots");
        }
    }
    if (flags & LILY_FLAG_LMHEAD) {
        h->lm_ld = ((uint64_t)vocab + 3u) & ~uint64_t(3);
        if ((e = cudaMalloc(&h->lm_logits, (size_t)lily_head::TOK * h->lm_ld * sizeof(float))) !=
            cudaSuccess) {
            return bail(e, "LM head logits");
        }
    }
    if (flags & LILY_FLAG_PHASE_CLOCKS) {
        const size_t pb = (size_t)max_rows * LILY_MAX_SLICES * LILY_PHASES * sizeof(long long);
        if ((e = cudaMalloc(&h->phase_clocks, pb)) != cudaSuccess ||
            (e = cudaMemset(h->phase_clocks, 0, pb)) != cudaSuccess) {
            return bail(e, "phase clocks");
        }
    }
    for (int i = 0; i < RING; ++i) {
        if ((e = cudaMallocHost(&h->h_stage[i], h->layout.total)) != cudaSuccess ||
            (e = cudaMalloc(&h->d_stage[i], h->layout.total)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h->ev[i], cudaEventDisableTiming)) != cudaSuccess) {
            return bail(e, "staging ring");
        }
    }
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) {
        return bail(e, "create");
    }
    *out = h;
    return LILY_OK;
}

void lily_sampler_destroy(lily_sampler_t *h) {
    if (h == nullptr) {
        return;
    }
    DeviceGuard guard(h->device);
    cudaDeviceSynchronize();
    cudaFree(h->part);
    cudaFree(h->part_n);
    cudaFree(h->tickets);
    cudaFree(h->status_word);
    cudaFree(h->spill);
    cudaFree(h->counts_scratch);
    cudaFree(h->counts_table);
    cudaFree(h->seen_table);
    cudaFree(h->phase_clocks);
    cudaFree(h->lm_logits);
    cudaFree(h->lm_hsum);
    if (h->h_status) {
        cudaFreeHost(h->h_status);
    }
    for (int i = 0; i < RING; ++i) {
        if (h->h_stage[i]) {
            cudaFreeHost(h->h_stage[i]);
        }
        cudaFree(h->d_stage[i]);
        if (h->ev[i]) {
            cudaEventDestroy(h->ev[i]);
        }
    }
    delete h;
}

uint32_t lily_sampler_vocab(const lily_sampler_t *h) { return h ? h->vocab : 0u; }

const char *lily_sampler_last_error(const lily_sampler_t *h) {
    return h ? h->last_error.c_str() : "null sampler";
}

void lily_sampler_inject_fault(lily_sampler_t *h, int32_t code) {
    if (h) {
        h->fault = code;
    }
}

void lily_sampler_clear_fault(lily_sampler_t *h) {
    if (h) {
        h->fault = 0;
    }
}

int32_t lily_sampler_set_wait_limit(lily_sampler_t *h, uint64_t nanoseconds) {
    if (h == nullptr) {
        return LILY_ERR_ARG;
    }
    h->wait_ns = nanoseconds == 0 ? 1000000000ull : nanoseconds;
    return LILY_OK;
}

void lily_sampler_inject_lost_copy(lily_sampler_t *h, uint32_t stage) {
    if (h) {
        h->lost_stage = stage;
    }
}

int32_t lily_sampler_status(lily_sampler_t *h, void *stream_) {
    if (h == nullptr) {
        return LILY_ERR_ARG;
    }
    if (h->fault != 0) {
        return fail(h, LILY_ERR_FAULT, "a fault is latched on this sampler");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    CU(h, cudaMemcpyAsync(h->h_status, h->status_word, 4, cudaMemcpyDeviceToHost, stream));
    CU(h, cudaMemsetAsync(h->status_word, 0, 4, stream));
    CU(h, cudaStreamSynchronize(stream));
    if (*h->h_status & (1u << lily_head::STATUS_TIMEOUT_BIT)) {
        return fail(h, LILY_ERR_TIMEOUT,
                    "a bounded wait ran out (inside the LM-head kernel, or for a peer's records): the results are not valid");
    }
    if (*h->h_status != 0u) {
        char buf[96];
        std::snprintf(buf, sizeof buf, "rows reported error bits 0x%x", *h->h_status);
        return fail(h, LILY_ERR_DEVICE_ROW, buf);
    }
    return LILY_OK;
}

// ------------------------------------------------------------- histogram --

int32_t lily_sampler_reset_counts(lily_sampler_t *h, void *stream_, uint32_t slot) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (h->counts_table == nullptr || slot >= h->max_rows) {
        return fail(h, LILY_ERR_ARG, "no such histogram slot");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    CU(h, cudaMemsetAsync(h->counts_table + (size_t)slot * h->vocab, 0, (size_t)h->vocab * 4,
                          stream));
    CU(h, cudaMemsetAsync(h->seen_table + (size_t)slot * h->seen_words, 0,
                          (size_t)h->seen_words * 4, stream));
    return LILY_OK;
}

int32_t lily_sampler_uncount(lily_sampler_t *h, void *stream_, uint32_t slot, uint32_t token) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (h->counts_table == nullptr || slot >= h->max_rows) {
        return fail(h, LILY_ERR_ARG, "no such histogram slot");
    }
    if (token >= h->vocab) {
        return LILY_OK;  // src/kernels/sample.rs:148-151: out of range is ignored
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    lily::uncount_kernel<<<1, 1, 0, stream>>>(h->counts_table + (size_t)slot * h->vocab,
                                              h->seen_table + (size_t)slot * h->seen_words,
                                              h->vocab, token);
    CU(h, cudaGetLastError());
    return LILY_OK;
}

int32_t lily_sampler_copy_counts(lily_sampler_t *dst, uint32_t dst_slot, const lily_sampler_t *src,
                                 uint32_t src_slot, void *stream_) {
    int32_t st = check_handle(dst);
    if (st != LILY_OK) {
        return st;
    }
    if (src == nullptr || dst->counts_table == nullptr || src->counts_table == nullptr ||
        dst_slot >= dst->max_rows || src_slot >= src->max_rows) {
        return fail(dst, LILY_ERR_ARG, "no such histogram slot");
    }
    if (src->vocab != dst->vocab) {
        return fail(dst, LILY_ERR_VOCAB, "sampler scratches for different vocabularies");
    }
    DeviceGuard guard(dst->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    CU(dst, cudaMemcpyAsync(dst->counts_table + (size_t)dst_slot * dst->vocab,
                            src->counts_table + (size_t)src_slot * src->vocab,
                            (size_t)dst->vocab * 4, cudaMemcpyDefault, stream));
    CU(dst, cudaMemcpyAsync(dst->seen_table + (size_t)dst_slot * dst->seen_words,
                            src->seen_table + (size_t)src_slot * src->seen_words,
                            (size_t)dst->seen_words * 4, cudaMemcpyDefault, stream));
    return LILY_OK;
}

// include/lily_batch.h: CountsSlot::Engine is the engine handle's slot 0,
// CountsSlot::Batch(i) slot i of the batch handle.
int32_t lily_move_counts(lily_sampler_t *engine, lily_sampler_t *batch, void *stream_,
                         uint32_t from, uint32_t to) {
    if (from == to) {
        return LILY_OK;
    }
    int32_t st = check_handle(engine);
    if (st != LILY_OK) {
        return st;
    }
    st = check_handle(batch);
    if (st != LILY_OK) {
        return st;
    }
    for (uint32_t slot : {from, to}) {
        if (slot != LILY_COUNTS_ENGINE && slot >= batch->max_rows) {
            std::string msg = "batch slot " + std::to_string(slot) + " of " +
                              std::to_string(batch->max_rows);
            fail(engine, LILY_ERR_ARG, msg.c_str());
            return fail(batch, LILY_ERR_ARG, msg.c_str());
        }
    }
    lily_sampler_t *src = from == LILY_COUNTS_ENGINE ? engine : batch;
    lily_sampler_t *dst = to == LILY_COUNTS_ENGINE ? engine : batch;
    return lily_sampler_copy_counts(dst, to == LILY_COUNTS_ENGINE ? 0u : to, src,
                                    from == LILY_COUNTS_ENGINE ? 0u : from, stream_);
}

int32_t lily_sampler_read_counts(lily_sampler_t *h, void *stream_, uint32_t slot,
                                 uint32_t *host_out) {
    if (h == nullptr || host_out == nullptr || h->counts_table == nullptr ||
        slot >= h->max_rows) {
        return fail(h, LILY_ERR_ARG, "no such histogram slot");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    CU(h, cudaMemcpyAsync(host_out, h->counts_table + (size_t)slot * h->vocab,
                          (size_t)h->vocab * 4, cudaMemcpyDeviceToHost, stream));
    CU(h, cudaStreamSynchronize(stream));
    return LILY_OK;
}

int32_t lily_sampler_write_counts(lily_sampler_t *h, void *stream_, uint32_t slot,
                                  const uint32_t *host_in) {
    if (h == nullptr || host_in == nullptr || h->counts_table == nullptr ||
        slot >= h->max_rows) {
        return fail(h, LILY_ERR_ARG, "no such histogram slot");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    uint32_t *counts = h->counts_table + (size_t)slot * h->vocab;
    CU(h, cudaMemcpyAsync(counts, host_in, (size_t)h->vocab * 4, cudaMemcpyHostToDevice, stream));
    const uint32_t threads = 256, blocks = (h->seen_words + threads - 1u) / threads;
    lily::rebuild_seen_kernel<<<blocks, threads, 0, stream>>>(
        counts, h->seen_table + (size_t)slot * h->seen_words, h->vocab);
    CU(h, cudaGetLastError());
    CU(h, cudaStreamSynchronize(stream));
    return LILY_OK;
}

int32_t lily_sampler_read_phase_clocks(lily_sampler_t *h, void *stream_, int64_t *host_out) {
    if (h == nullptr || host_out == nullptr || h->phase_clocks == nullptr) {
        return fail(h, LILY_ERR_ARG, "the sampler was not created with LILY_FLAG_PHASE_CLOCKS");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t pb = (size_t)h->max_rows * LILY_MAX_SLICES * LILY_PHASES * sizeof(long long);
    CU(h, cudaMemcpyAsync(host_out, h->phase_clocks, pb, cudaMemcpyDeviceToHost, stream));
    CU(h, cudaMemsetAsync(h->phase_clocks, 0, pb, stream));
    CU(h, cudaStreamSynchronize(stream));
    return LILY_OK;
}

// ------------------------------------------------------------------ draw --

int32_t lily_sample_batch(lily_sampler_t *h, void *stream_, const lily_sample_args_t *args) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t)) {
        return fail(h, LILY_ERR_ARG, "args is null or of another ABI version");
    }
    const lily_sample_args_t &g = *args;
    if (g.rows == 0u || g.rows > h->max_rows) {
        return fail(h, LILY_ERR_CAPACITY, "rows outside 1..max_rows");
    }
    if (g.logits == nullptr || g.out_ids == nullptr || g.params == nullptr ||
        g.logits_ld < h->vocab || g.logits_dtype > LILY_BF16) {
        return fail(h, LILY_ERR_ARG, "logits must be F32 or BF16 [rows, ld >= vocab]; out and params set");
    }
    if (g.uniforms == nullptr && g.steps == nullptr) {
        return fail(h, LILY_ERR_ARG, "either uniforms or steps must be given");
    }
    if ((g.history_ids != nullptr) != (g.history_len != nullptr) ||
        (g.bias_ids != nullptr) != (g.bias_len != nullptr) ||
        (g.bias_ids != nullptr) != (g.bias_vals != nullptr) ||
        (g.ban_ids != nullptr) != (g.ban_len != nullptr)) {
        return fail(h, LILY_ERR_ARG, "a list needs both its ids and its lengths");
    }
    if (g.kept_n != nullptr &&
        (g.kept_ids == nullptr || g.kept_probs == nullptr || g.kept_ld < LILY_K_CAP)) {
        return fail(h, LILY_ERR_ARG, "kept_n needs kept_ids, kept_probs and kept_ld >= 1024");
    }
    if (g.count_slots != nullptr && h->counts_table == nullptr) {
        return fail(h, LILY_ERR_ARG, "count_slots needs LILY_FLAG_COUNTS_TABLE");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    lily::KArgs a;
    base_args(h, &a);
    const lily_sampling_params_t *d_params = g.params;
    const uint32_t *d_steps = g.steps;
    const uint32_t *d_slots = nullptr;
    int slot = -1;
    // A small batch's host parameters (and slots) travel in the kernel's own
    // arguments: nothing is staged, no copy sits in front of the launch.
    const bool in_args = !g.params_on_device && g.rows <= lily::CL_MAX_ROWS &&
                         cluster_call(h, g.logits, g.logits_ld, g.logits_dtype, g.rows, true);
    if (!in_args && (!g.params_on_device || g.count_slots != nullptr)) {
        st = next_stage(h, &slot);
        if (st != LILY_OK) {
            return st;
        }
    }
    if (!g.params_on_device) {
        for (uint32_t r = 0; r < g.rows; ++r) {
            if (!params_ok(g.params[r])) {
                char buf[64];
                std::snprintf(buf, sizeof buf, "row %u: invalid sampling parameters", r);
                return fail(h, LILY_ERR_PARAMS, buf);
            }
        }
    }
    if (g.count_slots != nullptr) {
        for (uint32_t r = 0; r < g.rows; ++r) {
            if (g.count_slots[r] >= h->max_rows) {
                return fail(h, LILY_ERR_ARG, "no such histogram slot");
            }
        }
    }
    if (!g.params_on_device && !in_args) {
        char *hs = h->h_stage[slot];
        std::memcpy(hs + h->layout.params, g.params, sizeof(lily_sampling_params_t) * g.rows);
        d_params = reinterpret_cast<const lily_sampling_params_t *>(h->d_stage[slot] +
                                                                    h->layout.params);
        if (g.steps != nullptr) {
            std::memcpy(hs + h->layout.steps, g.steps, sizeof(uint32_t) * g.rows);
            d_steps = reinterpret_cast<const uint32_t *>(h->d_stage[slot] + h->layout.steps);
        }
    }
    if (g.count_slots != nullptr && !in_args) {
        std::memcpy(h->h_stage[slot] + h->layout.slots, g.count_slots, sizeof(uint32_t) * g.rows);
        d_slots = reinterpret_cast<const uint32_t *>(h->d_stage[slot] + h->layout.slots);
    }
    if (slot >= 0) {
        CU(h, cudaMemcpyAsync(h->d_stage[slot], h->h_stage[slot], h->layout.total,
                              cudaMemcpyHostToDevice, stream));
    }
    a.logits = g.logits;
    a.logits_ld = g.logits_ld;
    a.rows = g.rows;
    a.params = d_params;
    a.uniforms = g.uniforms;
    a.steps = d_steps;
    a.history_ids = g.history_ids;
    a.history_len = g.history_len;
    a.history_ld = g.history_ld;
    a.bias_ids = g.bias_ids;
    a.bias_vals = g.bias_vals;
    a.bias_len = g.bias_len;
    a.bias_ld = g.bias_ld;
    a.ban_ids = g.ban_ids;
    a.ban_len = g.ban_len;
    a.ban_ld = g.ban_ld;
    a.forced_ids = g.forced_ids;
    a.count_slots = d_slots;
    a.out_ids = g.out_ids;
    a.out_status = g.out_status;
    a.kept_n = g.kept_n;
    a.kept_ids = g.kept_ids;
    a.kept_probs = g.kept_probs;
    a.kept_ld = g.kept_ld;
    a.n_slices = choose_slices(h, g.rows);
    if (in_args) {
        lily::ClusterArgs ca;
        std::memset(&ca, 0, sizeof(ca));
        ca.a = a;
        ca.a.params = nullptr;
        ca.a.steps = nullptr;
        ca.inline_params = 1;
        std::memcpy(ca.params, g.params, sizeof(lily_sampling_params_t) * g.rows);
        if (g.steps != nullptr) {
            std::memcpy(ca.steps, g.steps, sizeof(uint32_t) * g.rows);
        }
        if (g.count_slots != nullptr) {
            ca.inline_slots = 1;
            std::memcpy(ca.slots, g.count_slots, sizeof(uint32_t) * g.rows);
        }
        return launch_cluster(h, stream, ca, g.rows, g.logits_dtype);
    }
    st = launch(h, stream, a, g.rows, g.logits_dtype);
    if (slot >= 0) {
        CU(h, cudaEventRecord(h->ev[slot], stream));
    }
    return st;
}

int32_t lily_argmax_batch(lily_sampler_t *h, void *stream_, const void *logits,
                          uint32_t logits_dtype, uint64_t logits_ld, uint32_t rows,
                          uint32_t *out_ids) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (rows == 0u || rows > h->max_rows) {
        return fail(h, LILY_ERR_CAPACITY, "rows outside 1..max_rows");
    }
    if (logits == nullptr || out_ids == nullptr || logits_ld < h->vocab ||
        logits_dtype > LILY_BF16) {
        return fail(h, LILY_ERR_ARG, "logits must be F32 or BF16 [rows, ld >= vocab]");
    }
    DeviceGuard guard(h->device);
    lily::KArgs a;
    base_args(h, &a);
    a.logits = logits;
    a.logits_ld = logits_ld;
    a.rows = rows;
    a.force_greedy = 1;
    a.out_ids = out_ids;
    a.n_slices = choose_slices(h, rows);
    return launch(h, static_cast<cudaStream_t>(stream_), a, rows, logits_dtype);
}

// ------------------------------------------------ LM head, vocab shards --

namespace {

// cuTensorMapEncodeTiled through the runtime's entry-point query: the library
// does not link against the driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

int32_t lmhead_launch(lily_sampler *h, cudaStream_t stream, const lily_lmhead_t *head,
                      const void *hidden, uint64_t hidden_ld, uint32_t tokens, float *out,
                      uint64_t out_ld) {
    if (head == nullptr || head->struct_size != sizeof(lily_lmhead_t)) {
        return fail(h, LILY_ERR_ARG, "head is null or of another ABI version");
    }
    if (head->weights == nullptr || head->scales_bf16 == nullptr || hidden == nullptr || out == nullptr) {
        return fail(h, LILY_ERR_ARG, "weights, scales, hidden and out must be set");
    }
    if (head->group != (uint32_t)lily_head::GROUP_K || head->hidden == 0u || head->hidden % 512u != 0u) {
        return fail(h, LILY_ERR_ARG, "group must be 64 and hidden a multiple of 512");
    }
    if (tokens == 0u || tokens > (uint32_t)lily_head::TOK) {
        return fail(h, LILY_ERR_CAPACITY, "tokens outside 1..64");
    }
    if (head->rows == 0u || out_ld < head->rows || hidden_ld < head->hidden) {
        return fail(h, LILY_ERR_ARG, "out_ld < rows or hidden_ld < hidden");
    }
    if (reinterpret_cast<uintptr_t>(head->weights) % 16u || reinterpret_cast<uintptr_t>(head->scales_bf16) % 16u ||
        reinterpret_cast<uintptr_t>(head->biases_bf16) % 16u || reinterpret_cast<uintptr_t>(hidden) % 16u ||
        (hidden_ld * 2u) % 16u) {
        return fail(h, LILY_ERR_ARG, "weights, scales, biases and hidden rows must be 16-byte aligned");
    }
    const bool affine = head->biases_bf16 != nullptr;
    if (affine && head->hidden / lily_head::GROUP_K > lily_head::BIAS_MAX_GROUPS) {
        return fail(h, LILY_ERR_CAPACITY, "an affine head takes a hidden size of at most 8192");
    }
    if (head->code_bits != 0u && head->code_bits != 8u && head->code_bits != 4u) {
        return fail(h, LILY_ERR_ARG, "code_bits must be 0, 8 or 4");
    }
    const bool q4 = head->code_bits == 4u;
    if (q4 && !affine) {
        return fail(h, LILY_ERR_ARG, "4-bit codes are the affine storage: biases must be set");
    }
    auto kernel = q4 ? lily_head::lmhead_int8_kernel<lily_head::VARIANT_AFFINE | lily_head::VARIANT_Q4>
                     : affine ? lily_head::lmhead_int8_kernel<lily_head::VARIANT_AFFINE>
                              : lily_head::lmhead_int8_kernel<0>;
    bool &attr_set = q4 ? h->lm_attr_q4 : affine ? h->lm_attr_affine : h->lm_attr;
    if (!attr_set) {
        CU(h, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)lily_head::Smem::BYTES));
        attr_set = true;
    }
    EncodeTiledFn encode = tensor_map_encoder();
    if (encode == nullptr) {
        return fail(h, LILY_ERR_CUDA, "the driver does not offer cuTensorMapEncodeTiled");
    }
    lily_head::Args a;
    {
        // Weights: uint8 [rows, hidden] (4-bit codes: [rows, hidden / 2]), boxes of 256 rows x 128 bytes.
        const cuuint64_t row_bytes = q4 ? head->hidden / 2u : head->hidden;
        const cuuint64_t dims[2] = {row_bytes, head->rows};
        const cuuint64_t strides[1] = {row_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)(lily_head::GROUP_K * lily_head::RAW_GROUPS),
                                   (cuuint32_t)lily_head::TILE_ROWS};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&a.w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(head->weights), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return fail(h, LILY_ERR_CUDA, "cuTensorMapEncodeTiled refused the weights");
        }
    }
    {
        // Hidden states: bf16 [tokens, hidden], boxes of 64 rows x 64 columns.
        const cuuint64_t dims[2] = {head->hidden, tokens};
        const cuuint64_t strides[1] = {hidden_ld * 2u};
        const cuuint32_t box[2] = {(cuuint32_t)lily_head::GROUP_K, (cuuint32_t)lily_head::TOK};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&a.h_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(hidden), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return fail(h, LILY_ERR_CUDA, "cuTensorMapEncodeTiled refused the hidden states");
        }
    }
    a.scales = static_cast<const __nv_bfloat16 *>(head->scales_bf16);
    if (affine) {
        const uint32_t head_groups = head->hidden / lily_head::GROUP_K;
        lily_head::hidden_group_sums_kernel<<<head_groups, lily_head::TOK, 0, stream>>>(
            static_cast<const __nv_bfloat16 *>(hidden), hidden_ld, tokens, h->lm_hsum);
        if (!h->lm_attr_bias) {
            CU(h, cudaFuncSetAttribute(lily_head::affine_bias_term_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)lily_head::bias_smem_bytes(lily_head::BIAS_MAX_GROUPS)));
            h->lm_attr_bias = true;
        }
        lily_head::affine_bias_term_kernel<<<(head->rows + lily_head::BIAS_ROWS - 1) / lily_head::BIAS_ROWS,
                                             lily_head::BIAS_THREADS, lily_head::bias_smem_bytes(head_groups),
                                             stream>>>(
            h->lm_hsum, tokens, static_cast<const __nv_bfloat16 *>(head->scales_bf16),
            static_cast<const __nv_bfloat16 *>(head->biases_bf16), head_groups, head->rows, out, out_ld,
            q4 ? 0.0f : 128.0f);
        CU(h, cudaGetLastError());
    }
    a.tokens = tokens;
    a.k = head->hidden;
    a.rows = head->rows;
    a.out = out;
    a.ldo = out_ld;
    a.status_word = h->status_word;
    a.wait_ns = h->wait_ns;
    a.lost_stage = h->lost_stage;
    h->lost_stage = 0xFFFFFFFFu;  // one launch only
    const uint32_t tiles = (head->rows + lily_head::TILE_ROWS - 1) / lily_head::TILE_ROWS;
    const uint32_t grid = tiles < (uint32_t)h->sm_count ? tiles : (uint32_t)h->sm_count;
    kernel<<<grid, lily_head::THREADS, lily_head::Smem::BYTES, stream>>>(a);
    CU(h, cudaGetLastError());
    return LILY_OK;
}

// Host parameters of a sharded call: checked, then staged to the device.
int32_t stage_shard_params(lily_sampler *h, cudaStream_t stream, const lily_sample_args_t &g,
                           const lily_sampling_params_t **d_params, const uint32_t **d_steps,
                           int *slot_out) {
    if (g.rows == 0u || g.rows > h->max_rows) {
        return fail(h, LILY_ERR_CAPACITY, "rows outside 1..max_rows");
    }
    if (g.params == nullptr || g.params_on_device) {
        return fail(h, LILY_ERR_ARG, "sharded calls take host params");
    }
    if (g.history_ids || g.history_len || g.bias_ids || g.bias_vals || g.bias_len || g.ban_ids ||
        g.ban_len || g.forced_ids || g.count_slots) {
        return fail(h, LILY_ERR_ARG, "no penalties state, lists or forced ids in sharded calls");
    }
    for (uint32_t r = 0; r < g.rows; ++r) {
        const lily_sampling_params_t &p = g.params[r];
        if (!params_ok(p)) {
            return fail(h, LILY_ERR_PARAMS, "invalid sampling parameters");
        }
        if (uses_penalties(p)) {
            return fail(h, LILY_ERR_ARG, "no penalties in sharded calls");
        }
        if (!is_greedy(p) && (p.top_k == 0u || p.top_k > LILY_SHARD_CANDIDATES)) {
            return fail(h, LILY_ERR_ARG, "sharded sampling needs 1 <= top_k <= 64");
        }
    }
    // What would be staged: [rows][has steps][params][steps].
    const size_t pb = sizeof(lily_sampling_params_t) * g.rows, sb = g.steps ? sizeof(uint32_t) * g.rows : 0;
    std::vector<char> want(8 + pb + sb);
    const uint32_t head[2] = {g.rows, g.steps != nullptr ? 1u : 0u};
    std::memcpy(want.data(), head, 8);
    std::memcpy(want.data() + 8, g.params, pb);
    if (sb) {
        std::memcpy(want.data() + 8 + pb, g.steps, sb);
    }
    int slot = h->shard_slot;
    const bool reuse = slot >= 0 && h->slot_serial[slot] == h->shard_serial && want == h->shard_bytes;
    if (!reuse) {
        int32_t st = next_stage(h, &slot);
        if (st != LILY_OK) {
            return st;
        }
        char *hs = h->h_stage[slot];
        std::memcpy(hs + h->layout.params, g.params, pb);
        if (sb) {
            std::memcpy(hs + h->layout.steps, g.steps, sb);
        }
        CU(h, cudaMemcpyAsync(h->d_stage[slot], h->h_stage[slot], h->layout.total, cudaMemcpyHostToDevice,
                              stream));
        h->shard_slot = slot;
        h->shard_serial = h->slot_serial[slot];
        h->shard_bytes.swap(want);
    }
    // (A reused slot is read by one more launch: the caller records the slot's
    // event after it, so the ring does not overwrite the slot under that launch.)
    *d_params = reinterpret_cast<const lily_sampling_params_t *>(h->d_stage[slot] + h->layout.params);
    *d_steps = g.steps != nullptr ? reinterpret_cast<const uint32_t *>(h->d_stage[slot] + h->layout.steps)
                                  : nullptr;
    *slot_out = slot;
    return LILY_OK;
}

int32_t shard_candidates(lily_sampler *h, cudaStream_t stream, const lily_sample_args_t &g,
                         uint32_t first_id, int32_t want_sums, void *records) {
    if (g.logits == nullptr || records == nullptr || g.logits_ld < h->vocab || g.logits_dtype > LILY_BF16) {
        return fail(h, LILY_ERR_ARG, "logits must be F32 or BF16 [rows, ld >= vocab]; records set");
    }
    if ((uint64_t)first_id + h->vocab > 0xFFFFFFFFull) {
        return fail(h, LILY_ERR_ARG, "first_id + vocab overflows an id");
    }
    const lily_sampling_params_t *d_params = nullptr;
    const uint32_t *d_steps = nullptr;
    int slot = -1;
    int32_t st = stage_shard_params(h, stream, g, &d_params, &d_steps, &slot);
    if (st != LILY_OK) {
        return st;
    }
    lily::KArgs a;
    base_args(h, &a);
    a.logits = g.logits;
    a.logits_ld = g.logits_ld;
    a.rows = g.rows;
    a.params = d_params;
    a.steps = d_steps;
    a.out_ids = nullptr;
    a.shard_k = LILY_SHARD_CANDIDATES;
    a.id_offset = first_id;
    a.cand_out = static_cast<lily::ShardRecord *>(records);
    a.n_slices = choose_slices(h, g.rows);
    // (The kernel of one block per row sums the exponentials in the same pass.)
    a.shard_sums = want_sums && stream_route(a, g.rows, g.logits_dtype) ? 1u : 0u;
    st = launch(h, stream, a, g.rows, g.logits_dtype);
    if (st == LILY_OK && want_sums && a.shard_sums == 0u) {
        // The candidate launch has left the slice counters and the tickets (all
        // zero again) free: the sums use them for their pieces.
        uint32_t pieces = (2u * (uint32_t)h->sm_count + g.rows - 1u) / g.rows;
        const uint32_t by_len = (h->vocab + 8191u) / 8192u;
        pieces = pieces > by_len ? by_len : pieces;
        pieces = pieces < 1u ? 1u : (pieces > lily::MAX_SLICES ? lily::MAX_SLICES : pieces);
        const dim3 grid(pieces, g.rows, 1);
        float *scratch = reinterpret_cast<float *>(h->part_n);
        if (g.logits_dtype == LILY_F32) {
            lily::shard_sums_kernel<float><<<grid, 1024, 0, stream>>>(
                static_cast<const float *>(g.logits), g.logits_ld, h->vocab, d_params, a.cand_out, scratch,
                h->tickets);
        } else {
            lily::shard_sums_kernel<__nv_bfloat16><<<grid, 1024, 0, stream>>>(
                static_cast<const __nv_bfloat16 *>(g.logits), g.logits_ld, h->vocab, d_params, a.cand_out,
                scratch, h->tickets);
        }
        CU(h, cudaGetLastError());
    }
    CU(h, cudaEventRecord(h->ev[slot], stream));
    return st;
}

}  // namespace

int32_t lily_lmhead_logits(lily_sampler_t *h, void *stream_, const lily_lmhead_t *head,
                           const void *hidden_bf16, uint64_t hidden_ld, uint32_t tokens,
                           float *out_logits, uint64_t out_ld) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    DeviceGuard guard(h->device);
    return lmhead_launch(h, static_cast<cudaStream_t>(stream_), head, hidden_bf16, hidden_ld, tokens,
                         out_logits, out_ld);
}

int32_t lily_shard_candidates(lily_sampler_t *h, void *stream_, const lily_sample_args_t *args,
                              uint32_t first_id, int32_t want_sums, void *records) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t)) {
        return fail(h, LILY_ERR_ARG, "args is null or of another ABI version");
    }
    DeviceGuard guard(h->device);
    return shard_candidates(h, static_cast<cudaStream_t>(stream_), *args, first_id, want_sums, records);
}

int32_t lily_lmhead_shard_candidates(lily_sampler_t *h, void *stream_, const lily_lmhead_t *head,
                                     const void *hidden_bf16, uint64_t hidden_ld,
                                     const lily_sample_args_t *args, uint32_t first_id,
                                     int32_t want_sums, void *records) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t)) {
        return fail(h, LILY_ERR_ARG, "args is null or of another ABI version");
    }
    if (h->lm_logits == nullptr) {
        return fail(h, LILY_ERR_ARG, "the sampler was not created with LILY_FLAG_LMHEAD");
    }
    if (head == nullptr || head->rows != h->vocab) {
        return fail(h, LILY_ERR_VOCAB, "the head's rows must equal the sampler's vocabulary");
    }
    if (args->logits != nullptr) {
        return fail(h, LILY_ERR_ARG, "the logits come from the head: args->logits must be NULL");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    st = lmhead_launch(h, stream, head, hidden_bf16, hidden_ld, args->rows, h->lm_logits, h->lm_ld);
    if (st != LILY_OK) {
        return st;
    }
    lily_sample_args_t g = *args;
    g.logits = h->lm_logits;
    g.logits_dtype = LILY_F32;
    g.logits_ld = h->lm_ld;
    return shard_candidates(h, stream, g, first_id, want_sums, records);
}

namespace {
int32_t merge_draw(lily_sampler_t *h, void *stream_, const void *gathered, uint32_t n_shards,
                   uint64_t shard_stride, const lily_sample_args_t *args, float *out_lse,
                   const lily::KArgs::PeerLink *peer);

}  // namespace

int32_t lily_merge_draw(lily_sampler_t *h, void *stream_, const void *gathered, uint32_t n_shards,
                        uint64_t shard_stride, const lily_sample_args_t *args, float *out_lse) {
    return merge_draw(h, stream_, gathered, n_shards, shard_stride, args, out_lse, nullptr);
}

namespace {

int32_t merge_draw(lily_sampler_t *h, void *stream_, const void *gathered, uint32_t n_shards,
                   uint64_t shard_stride, const lily_sample_args_t *args, float *out_lse,
                   const lily::KArgs::PeerLink *peer) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t)) {
        return fail(h, LILY_ERR_ARG, "args is null or of another ABI version");
    }
    const lily_sample_args_t &g = *args;
    if (gathered == nullptr || n_shards == 0u || n_shards > 64u || shard_stride < g.rows ||
        g.out_ids == nullptr || g.logits != nullptr) {
        return fail(h, LILY_ERR_ARG, "records and out_ids set, 1..64 shards, stride >= rows, no logits");
    }
    if (g.uniforms == nullptr && g.steps == nullptr) {
        return fail(h, LILY_ERR_ARG, "either uniforms or steps must be given");
    }
    if (g.kept_n != nullptr &&
        (g.kept_ids == nullptr || g.kept_probs == nullptr || g.kept_ld < LILY_SHARD_CANDIDATES)) {
        return fail(h, LILY_ERR_ARG, "kept_n needs kept_ids, kept_probs and kept_ld >= 64");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const lily_sampling_params_t *d_params = nullptr;
    const uint32_t *d_steps = nullptr;
    int slot = -1;
    st = stage_shard_params(h, stream, g, &d_params, &d_steps, &slot);
    if (st != LILY_OK) {
        return st;
    }
    if (!h->merge_attr) {
        CU(h, cudaFuncSetAttribute(lily::merge_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(lily::SmemFixed)));
        h->merge_attr = true;
    }
    lily::KArgs a;
    base_args(h, &a);
    a.vocab = 0xFFFFFFFFu;  // ids are global here
    a.rows = g.rows;
    a.params = d_params;
    a.uniforms = g.uniforms;
    a.steps = d_steps;
    a.out_ids = g.out_ids;
    a.out_status = g.out_status;
    a.kept_n = g.kept_n;
    a.kept_ids = g.kept_ids;
    a.kept_probs = g.kept_probs;
    a.kept_ld = g.kept_ld;
    a.merge_in = static_cast<const lily::ShardRecord *>(gathered);
    a.merge_shards = n_shards;
    a.merge_stride = shard_stride;
    a.out_lse = out_lse;
    if (peer != nullptr) {
        a.peer = *peer;
    }
    lily::merge_rows_kernel<<<g.rows, lily::NT, sizeof(lily::SmemFixed), stream>>>(a);
    CU(h, cudaGetLastError());
    CU(h, cudaEventRecord(h->ev[slot], stream));
    return LILY_OK;
}

}  // namespace

// ------------------------------------------------- records over peer memory --

namespace {

int32_t peer_check(lily_sampler *h, const lily_peer_exchange_t *x) {
    if (x == nullptr || x->struct_size != sizeof(lily_peer_exchange_t)) {
        return fail(h, LILY_ERR_ARG, "exchange is null or of another ABI version");
    }
    if (x->n_shards == 0u || x->n_shards > LILY_PEER_MAX || x->rank >= x->n_shards || x->max_rows == 0u) {
        return fail(h, LILY_ERR_ARG, "1..16 shards, rank below them, max_rows set");
    }
    for (uint32_t r = 0; r < x->n_shards; ++r) {
        if (x->buffers[r] == nullptr) {
            return fail(h, LILY_ERR_ARG, "every rank's buffer must be set");
        }
    }
    return LILY_OK;
}

}  // namespace

uint64_t lily_peer_buffer_bytes(uint32_t n_shards, uint32_t max_rows) {
    return (uint64_t)lily::peer_flag_bytes(n_shards, max_rows) +
           2ull * n_shards * max_rows * sizeof(lily::ShardRecord);
}

int32_t lily_peer_buffer_create(int32_t device, uint32_t n_shards, uint32_t max_rows, void **buffer,
                                void *ipc_handle) {
    if (buffer == nullptr || ipc_handle == nullptr || n_shards == 0u || n_shards > LILY_PEER_MAX ||
        max_rows == 0u) {
        return LILY_ERR_ARG;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == LILY_IPC_HANDLE_BYTES, "the handle travels as 64 bytes");
    DeviceGuard guard(device);
    const size_t bytes = lily_peer_buffer_bytes(n_shards, max_rows);
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        return LILY_ERR_CUDA;
    }
    cudaIpcMemHandle_t handle;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&handle, p) != cudaSuccess) {
        cudaFree(p);
        return LILY_ERR_CUDA;
    }
    std::memcpy(ipc_handle, &handle, sizeof handle);
    *buffer = p;
    return LILY_OK;
}

int32_t lily_peer_buffer_open(int32_t device, const void *ipc_handle, void **buffer) {
    if (buffer == nullptr || ipc_handle == nullptr) {
        return LILY_ERR_ARG;
    }
    DeviceGuard guard(device);
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, ipc_handle, sizeof handle);
    return cudaIpcOpenMemHandle(buffer, handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? LILY_OK
                                                                                                : LILY_ERR_CUDA;
}

int32_t lily_peer_buffer_close(int32_t device, void *buffer) {
    DeviceGuard guard(device);
    return buffer != nullptr && cudaIpcCloseMemHandle(buffer) == cudaSuccess ? LILY_OK : LILY_ERR_CUDA;
}

int32_t lily_peer_buffer_destroy(int32_t device, void *buffer) {
    DeviceGuard guard(device);
    return cudaFree(buffer) == cudaSuccess ? LILY_OK : LILY_ERR_CUDA;
}

int32_t lily_shard_publish(lily_sampler_t *h, void *stream_, const lily_peer_exchange_t *x,
                           const void *records, uint32_t rows, uint32_t step) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if ((st = peer_check(h, x)) != LILY_OK) {
        return st;
    }
    if (records == nullptr || rows == 0u || rows > x->max_rows || reinterpret_cast<uintptr_t>(records) % 8u) {
        return fail(h, LILY_ERR_ARG, "records set and 8-byte aligned, 1 <= rows <= max_rows");
    }
    DeviceGuard guard(h->device);
    lily::PeerArgs p;
    std::memset(&p, 0, sizeof p);
    for (uint32_t r = 0; r < x->n_shards; ++r) {
        p.buffers[r] = x->buffers[r];
    }
    p.n_shards = x->n_shards;
    p.rank = x->rank;
    p.max_rows = x->max_rows;
    p.records = static_cast<const lily::ShardRecord *>(records);
    p.rows = rows;
    p.step = step;
    lily::shard_publish_kernel<<<x->n_shards, 256, 0, static_cast<cudaStream_t>(stream_)>>>(p);
    CU(h, cudaGetLastError());
    return LILY_OK;
}

int32_t lily_merge_draw_peer(lily_sampler_t *h, void *stream_, const lily_peer_exchange_t *x,
                             const void *records, uint32_t step, const lily_sample_args_t *args,
                             float *out_lse) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if ((st = peer_check(h, x)) != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t) || args->rows > x->max_rows) {
        return fail(h, LILY_ERR_ARG, "args is null, of another ABI version, or has more rows than max_rows");
    }
    if (reinterpret_cast<uintptr_t>(records) % 8u) {
        return fail(h, LILY_ERR_ARG, "records must be 8-byte aligned");
    }
    lily::KArgs::PeerLink peer;
    std::memset(&peer, 0, sizeof peer);
    for (uint32_t r = 0; r < x->n_shards; ++r) {
        peer.buffers[r] = x->buffers[r];
    }
    peer.own = records;
    peer.wait_ns = h->wait_ns;
    peer.n = x->n_shards;
    peer.rank = x->rank;
    peer.max_rows = x->max_rows;
    peer.step = step;
    const char *slot = static_cast<const char *>(x->buffers[x->rank]) +
                       lily::peer_flag_bytes(x->n_shards, x->max_rows) +
                       (size_t)(step & 1u) * x->n_shards * x->max_rows * sizeof(lily::ShardRecord);
    return merge_draw(h, stream_, slot, x->n_shards, x->max_rows, args, out_lse, &peer);
}

// ----------------------------------------------------------- speculation --

int32_t lily_spec_verify(lily_sampler_t *h, void *stream_, const lily_spec_args_t *args) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (args == nullptr || args->struct_size != sizeof(lily_spec_args_t)) {
        return fail(h, LILY_ERR_ARG, "args is null or of another ABI version");
    }
    const lily_spec_args_t &g = *args;
    if (g.m == 0u || g.m > 8u || g.m > h->max_rows) {
        return fail(h, LILY_ERR_CAPACITY, "m outside 1..min(8, max_rows)");
    }
    if (g.target_logits == nullptr || g.params == nullptr || g.out_ids == nullptr ||
        g.out_accepted == nullptr || g.logits_ld < h->vocab || g.logits_dtype > LILY_BF16 ||
        g.mode > LILY_SPEC_GREEDY_MATCH) {
        return fail(h, LILY_ERR_ARG, "target logits, params and outputs must be set");
    }
    if (g.m > 1u && g.draft_ids == nullptr) {
        return fail(h, LILY_ERR_ARG, "draft_ids missing");
    }
    if (!params_ok(*g.params)) {
        return fail(h, LILY_ERR_PARAMS, "invalid sampling parameters");
    }
    lily_sampling_params_t p = *g.params;
    if (g.mode == LILY_SPEC_GREEDY_MATCH) {
        p.temperature = 0.0f;
    }
    const bool pen = uses_penalties(p);
    const bool argmax_rows = is_greedy(p) && !pen;
    const bool spec_rows = g.mode == LILY_SPEC_REJECTION && !argmax_rows && g.m > 1u;
    if (spec_rows) {
        const bool dense = g.q_dense != nullptr;
        const bool sparse = g.q_ids != nullptr && g.q_probs != nullptr && g.q_n != nullptr;
        if (dense == sparse) {
            return fail(h, LILY_ERR_ARG, "give the draft distribution dense or sparse, not both");
        }
        if (dense && g.q_ld < h->vocab) {
            return fail(h, LILY_ERR_ARG, "q_ld < vocab");
        }
    }
    if (g.history_len > 0u && g.history_ids == nullptr) {
        return fail(h, LILY_ERR_ARG, "history_len without history_ids");
    }
    if (g.count_slot != nullptr && (h->counts_table == nullptr || *g.count_slot >= h->max_rows)) {
        return fail(h, LILY_ERR_ARG, "no such histogram slot");
    }
    DeviceGuard guard(h->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int slot = -1;
    st = next_stage(h, &slot);
    if (st != LILY_OK) {
        return st;
    }
    char *hs = h->h_stage[slot];
    auto *sp = reinterpret_cast<lily_sampling_params_t *>(hs + h->layout.params);
    auto *ss = reinterpret_cast<uint32_t *>(hs + h->layout.steps);
    auto *sl = reinterpret_cast<uint32_t *>(hs + h->layout.slots);
    auto *sh = reinterpret_cast<uint32_t *>(hs + h->layout.hist_len);
    for (uint32_t j = 0; j < g.m; ++j) {
        sp[j] = p;
        ss[j] = g.step0 + j;
        sl[j] = g.count_slot ? *g.count_slot : 0u;
        sh[j] = g.history_len;
    }
    CU(h, cudaMemcpyAsync(h->d_stage[slot], hs, h->layout.total, cudaMemcpyHostToDevice, stream));
    char *ds = h->d_stage[slot];

    lily::KArgs a;
    base_args(h, &a);
    a.logits = g.target_logits;
    a.logits_ld = g.logits_ld;
    a.rows = g.m;
    a.params = reinterpret_cast<const lily_sampling_params_t *>(ds + h->layout.params);
    a.uniforms = g.u_accept;
    a.steps = reinterpret_cast<const uint32_t *>(ds + h->layout.steps);
    a.history_ids = g.history_ids;
    a.history_len = g.history_ids ? reinterpret_cast<const uint32_t *>(ds + h->layout.hist_len)
                                  : nullptr;
    a.history_ld = 0;  // every row of the step reads the same list
    a.count_slots = g.count_slot ? reinterpret_cast<const uint32_t *>(ds + h->layout.slots)
                                 : nullptr;
    a.out_ids = g.out_ids;
    a.out_status = g.out_status;
    if (spec_rows) {
        a.spec.draft_ids = g.draft_ids;
        a.spec.q_dense = g.q_dense;
        a.spec.q_ld = g.q_ld;
        a.spec.q_ids = g.q_ids;
        a.spec.q_probs = g.q_probs;
        a.spec.q_n = g.q_n;
        a.spec.u_resid = g.u_resid;
        a.spec.n_spec = g.m - 1u;
    }
    if (!pen) {
        // Without penalties the rows do not depend on one another.
        a.n_slices = choose_slices(h, g.m);
        st = launch(h, stream, a, g.m, g.logits_dtype);
    } else {
        // Row j's penalties see the draws of rows < j (the reference's rows
        // share one histogram, src/qwen4exp/model.rs:3008-3012): one launch
        // per row, in stream order.
        a.n_slices = choose_slices(h, 1u);
        for (uint32_t j = 0; j < g.m && st == LILY_OK; ++j) {
            a.row0 = j;
            if (g.count_slot == nullptr) {
                a.extra_ids = g.out_ids;
                a.extra_len = j;
            }
            st = launch(h, stream, a, 1u, g.logits_dtype);
        }
    }
    if (st == LILY_OK) {
        if (g.m > 1u) {
            lily::spec_accept_kernel<<<1, 1, 0, stream>>>(g.out_ids, g.draft_ids, 0u, g.m,
                                                          g.out_accepted, 0u, 1u, 0u, 0u);
        } else {
            CU(h, cudaMemsetAsync(g.out_accepted, 0, 4, stream));
        }
        CU(h, cudaGetLastError());
    }
    CU(h, cudaEventRecord(h->ev[slot], stream));
    return st;
}

int32_t lily_spec_accept(lily_sampler_t *h, void *stream_, const uint32_t *draws,
                         const uint32_t *ids, uint32_t m, uint32_t *ctrl, uint32_t pos0,
                         uint32_t ratio, uint32_t chain, uint32_t stride) {
    int32_t st = check_handle(h);
    if (st != LILY_OK) {
        return st;
    }
    if (draws == nullptr || ids == nullptr || ctrl == nullptr || m == 0u) {
        return fail(h, LILY_ERR_ARG, "draws and ids must both hold the verified rows");
    }
    if (ratio == 0u) {
        return fail(h, LILY_ERR_ARG, "indexer block ratio must be nonzero");
    }
    if (stride == 0u) {
        return fail(h, LILY_ERR_ARG, "stride must be nonzero");
    }
    DeviceGuard guard(h->device);
    lily::spec_accept_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(
        draws, ids, 1u, m, ctrl, pos0, ratio, chain, stride);
    CU(h, cudaGetLastError());
    return LILY_OK;
}

// ------------------------------------------------ allocation-free draw --

}  // extern "C"

namespace {

// Everything the kernel needs beyond its inputs and outputs, for up to
// LILY_NOALLOC_MAX_ROWS rows. The layout is what the kernel indexes:
// part[row][CAP], part_n[row][MAX_SLICES], tickets[row].
struct NoAllocScratch {
    uint2 part[LILY_NOALLOC_MAX_ROWS][lily::CAP];
    uint32_t part_n[LILY_NOALLOC_MAX_ROWS][lily::MAX_SLICES];
    uint32_t tickets[LILY_NOALLOC_MAX_ROWS];
    uint32_t status_word;
    uint32_t steps[LILY_NOALLOC_MAX_ROWS];
    lily_sampling_params_t params[LILY_NOALLOC_MAX_ROWS];
};
static_assert(sizeof(NoAllocScratch) <= LILY_NOALLOC_SCRATCH_BYTES, "stated size too small");

// Static device storage: no allocation call ever makes or frees it. In host
// code this name is only a stand-in for the array, not a device address: the
// address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[LILY_NOALLOC_SCRATCH_BYTES];

struct NoAllocDevice {
    bool ready = false;
    NoAllocScratch *scratch = nullptr;  // device address on this device
    int sm_count = 0;
    int max_smem = 0;
    uint32_t attr_mask = 0;
};
NoAllocDevice g_noalloc_devices[64];
std::mutex g_noalloc_mutex;  // guards the per-device set-up above (host threads may race to the first call)

int32_t noalloc_fail(int32_t code, const char *msg, char *err, uint32_t err_cap) {
    if (err != nullptr && err_cap > 0u) {
        std::snprintf(err, err_cap, "%s", msg);
    }
    return code;
}

template <typename T, bool VEC>
cudaError_t noalloc_launch_one(NoAllocDevice *d, cudaStream_t stream, const lily::KArgs &a,
                               uint32_t rows, size_t smem) {
    auto kernel = lily::sample_rows_kernel<T, VEC>;
    const uint32_t bit = 1u << ((sizeof(T) == 4 ? 0 : 2) + (VEC ? 1 : 0));
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!(d->attr_mask & bit)) {
            const cudaError_t e = cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, d->max_smem);
            if (e != cudaSuccess) {
                return e;
            }
            d->attr_mask |= bit;
        }
    }
    dim3 grid(a.n_slices, rows, 1);
    kernel<<<grid, lily::NT, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

extern "C" {

int32_t lily_sample_batch_noalloc(void *stream_, uint32_t vocab, const lily_sample_args_t *args,
                                  char *err, uint32_t err_cap) {
    if (args == nullptr || args->struct_size != sizeof(lily_sample_args_t)) {
        return noalloc_fail(LILY_ERR_ARG, "args is null or of another ABI version", err, err_cap);
    }
    const lily_sample_args_t &g = *args;
    if (g.rows == 0u || g.rows > LILY_NOALLOC_MAX_ROWS) {
        return noalloc_fail(LILY_ERR_CAPACITY, "rows outside 1..LILY_NOALLOC_MAX_ROWS", err, err_cap);
    }
    if (vocab == 0u || vocab > (1u << 24) || g.logits == nullptr || g.out_ids == nullptr ||
        g.params == nullptr || g.logits_ld < vocab || g.logits_dtype > LILY_BF16) {
        return noalloc_fail(LILY_ERR_ARG,
                            "logits must be F32 or BF16 [rows, ld >= vocab]; out and params set",
                            err, err_cap);
    }
    if (g.params_on_device != 0u || g.count_slots != nullptr) {
        return noalloc_fail(LILY_ERR_ARG,
                            "the allocation-free draw takes host params and no histogram slots",
                            err, err_cap);
    }
    if (g.uniforms == nullptr && g.steps == nullptr) {
        return noalloc_fail(LILY_ERR_ARG, "either uniforms or steps must be given", err, err_cap);
    }
    if ((g.history_ids != nullptr) != (g.history_len != nullptr) ||
        (g.bias_ids != nullptr) != (g.bias_len != nullptr) ||
        (g.bias_ids != nullptr) != (g.bias_vals != nullptr) ||
        (g.ban_ids != nullptr) != (g.ban_len != nullptr)) {
        return noalloc_fail(LILY_ERR_ARG, "a list needs both its ids and its lengths", err, err_cap);
    }
    if (g.kept_n != nullptr &&
        (g.kept_ids == nullptr || g.kept_probs == nullptr || g.kept_ld < LILY_K_CAP)) {
        return noalloc_fail(LILY_ERR_ARG, "kept_n needs kept_ids, kept_probs and kept_ld >= 1024",
                            err, err_cap);
    }
    for (uint32_t r = 0; r < g.rows; ++r) {
        if (!params_ok(g.params[r])) {
            return noalloc_fail(LILY_ERR_PARAMS, "invalid sampling parameters", err, err_cap);
        }
        if (g.history_ids != nullptr && uses_penalties(g.params[r]) &&
            g.params[r].frequency_penalty != 0.0f) {
            return noalloc_fail(LILY_ERR_CAPACITY,
                                "a frequency penalty over a history list needs a vocabulary-sized "
                                "count table, which the allocation-free draw does not carry",
                                err, err_cap);
        }
    }
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        return noalloc_fail(LILY_ERR_CUDA, "no current CUDA device", err, err_cap);
    }
    NoAllocDevice *d = &g_noalloc_devices[device];
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!d->ready) {
            // Set-up, once per device, with that device current: the array's
            // address ON THIS DEVICE. (Passing the host-side name to the kernel
            // instead would hand it a host address.)
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || p == nullptr) {
                return noalloc_fail(LILY_ERR_CUDA, "cudaGetSymbolAddress failed for the static scratch",
                                    err, err_cap);
            }
            if (cudaDeviceGetAttribute(&d->sm_count, cudaDevAttrMultiProcessorCount, device) !=
                    cudaSuccess ||
                cudaDeviceGetAttribute(&d->max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) !=
                    cudaSuccess) {
                return noalloc_fail(LILY_ERR_CUDA, "device attributes unavailable", err, err_cap);
            }
            d->scratch = static_cast<NoAllocScratch *>(p);
            d->ready = true;
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    NoAllocScratch *sc = d->scratch;
    // The array keeps the last call's contents: the tickets and the status
    // word must start at zero; the parameters are overwritten.
    if (cudaMemsetAsync(sc->tickets, 0, sizeof(sc->tickets) + sizeof(sc->status_word), stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(sc->params, g.params, sizeof(lily_sampling_params_t) * g.rows,
                        cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        (g.steps != nullptr &&
         cudaMemcpyAsync(sc->steps, g.steps, sizeof(uint32_t) * g.rows, cudaMemcpyHostToDevice,
                         stream) != cudaSuccess)) {
        return noalloc_fail(LILY_ERR_CUDA, "staging the parameters failed", err, err_cap);
    }
    lily::KArgs a;
    std::memset(&a, 0, sizeof(a));
    a.vocab = vocab;
    a.max_history = 1u << 16;
    a.max_list = 512u;
    a.part = &sc->part[0][0];
    a.part_n = &sc->part_n[0][0];
    a.tickets = sc->tickets;
    a.status_word = &sc->status_word;
    a.logits = g.logits;
    a.logits_ld = g.logits_ld;
    a.rows = g.rows;
    a.params = sc->params;
    a.uniforms = g.uniforms;
    a.steps = g.steps != nullptr ? sc->steps : nullptr;
    a.history_ids = g.history_ids;
    a.history_len = g.history_len;
    a.history_ld = g.history_ld;
    a.bias_ids = g.bias_ids;
    a.bias_vals = g.bias_vals;
    a.bias_len = g.bias_len;
    a.bias_ld = g.bias_ld;
    a.ban_ids = g.ban_ids;
    a.ban_len = g.ban_len;
    a.ban_ld = g.ban_ld;
    a.forced_ids = g.forced_ids;
    a.out_ids = g.out_ids;
    a.out_status = g.out_status;
    a.kept_n = g.kept_n;
    a.kept_ids = g.kept_ids;
    a.kept_probs = g.kept_probs;
    a.kept_ld = g.kept_ld;
    uint32_t slices = 2u * (uint32_t)d->sm_count / g.rows;
    const uint32_t by_len = (vocab + lily::MIN_SLICE - 1u) / lily::MIN_SLICE;
    slices = slices > lily::MAX_SLICES ? lily::MAX_SLICES : slices;
    slices = slices > by_len ? by_len : slices;
    a.n_slices = slices < 1u ? 1u : slices;
    const size_t smem = smem_bytes(vocab, a.n_slices);
    if (smem > (size_t)d->max_smem) {
        return noalloc_fail(LILY_ERR_CAPACITY, "vocabulary too large for the shared-memory bitmap",
                            err, err_cap);
    }
    const size_t esize = g.logits_dtype == LILY_F32 ? 4 : 2;
    const bool vec = (reinterpret_cast<uintptr_t>(a.logits) % 16u == 0u) &&
                     ((a.logits_ld * esize) % 16u == 0u);
    cudaError_t e;
    if (g.logits_dtype == LILY_F32) {
        e = vec ? noalloc_launch_one<float, true>(d, stream, a, g.rows, smem)
                : noalloc_launch_one<float, false>(d, stream, a, g.rows, smem);
    } else {
        e = vec ? noalloc_launch_one<__nv_bfloat16, true>(d, stream, a, g.rows, smem)
                : noalloc_launch_one<__nv_bfloat16, false>(d, stream, a, g.rows, smem);
    }
    if (e != cudaSuccess) {
        return noalloc_fail(LILY_ERR_CUDA, cudaGetErrorString(e), err, err_cap);
    }
    return LILY_OK;
}

int32_t lily_debug_exp(void *stream_, const float *in, float *out, uint64_t n) {
    if (in == nullptr || out == nullptr) {
        return LILY_ERR_ARG;
    }
    if (n == 0u) {
        return LILY_OK;
    }
    const uint32_t threads = 256;
    const uint64_t blocks = (n + threads - 1u) / threads;
    lily::exp_kernel<<<(uint32_t)(blocks > 65535u * 16u ? 65535u * 16u : blocks), threads, 0,
                       static_cast<cudaStream_t>(stream_)>>>(in, out, n);
    return cudaGetLastError() == cudaSuccess ? LILY_OK : LILY_ERR_CUDA;
}

}  // extern "C"
