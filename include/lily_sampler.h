/*
 * lily_sampler.h -- C ABI of the B200 token sampler.
 *
 * A drop-in for the sampling step of lily's decode loop: every entry point
 * below names the item of the reference project it replaces (paths relative
 * to that project). Host code in any language binds these symbols; nothing
 * in the signatures is a C++ or torch type.
 *
 * Conventions (they mirror the reference's, src/kernels/sample.rs:251-266,
 * docs/architecture.md:133-138, src/metal.rs:681-696):
 *   - Every call that takes a `stream` (a cudaStream_t, passed as void*) only
 *     ENQUEUES work on it and returns; results are valid once the stream has
 *     reached that point. Nothing synchronises unless it says so.
 *   - The caller owns every buffer it passes and keeps it alive until the
 *     stream has consumed it. The library owns what `lily_sampler_create`
 *     allocates.
 *   - Return value: 0 = LILY_OK; negative = the arguments were refused on the
 *     host before anything was enqueued; positive = CUDA / device error. The
 *     text of the last error of a handle: lily_sampler_last_error().
 *   - A handle is not thread-safe: one handle per engine thread.
 *   - Determinism: same logits, history / counts, params and uniforms give
 *     the same token, whatever the batch around the row and however the row
 *     is split over thread blocks.
 *   - There is no CPU fallback: without a CUDA device every call that needs
 *     one fails with LILY_ERR_CUDA.
 */
#ifndef LILY_SAMPLER_H
#define LILY_SAMPLER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LILY_ABI_VERSION 1u

/* src/kernels/sample.rs:17 SAMPLE_K_CAP: largest candidate set. */
#define LILY_K_CAP 1024u

enum lily_status {
    LILY_OK = 0,
    LILY_ERR_ARG = -1,        /* null / out-of-range argument */
    LILY_ERR_PARAMS = -2,     /* SamplingParams::validate refused a row */
    LILY_ERR_CAPACITY = -3,   /* rows / vocab / list length beyond the handle's */
    LILY_ERR_FAULT = -4,      /* an injected or latched fault (see inject_fault) */
    LILY_ERR_VOCAB = -5,      /* handles of different vocabularies */
    LILY_ERR_CUDA = 1,        /* a CUDA runtime call failed */
    LILY_ERR_DEVICE_ROW = 2,  /* a row reported an error word (see row status) */
    LILY_ERR_TIMEOUT = 3      /* a bounded wait inside a kernel ran out (lily_sampler_status) */
};

/* Per-row status words written to `out_status` (0 = drawn normally). */
enum lily_row_status {
    LILY_ROW_OK = 0,
    LILY_ROW_NAN = 1,        /* a NaN among the adjusted logits */
    LILY_ROW_NONFINITE = 2,  /* largest adjusted logit not finite (all banned) */
    LILY_ROW_PARAMS = 3,     /* device-resident params failed validation */
    LILY_ROW_LIST = 4,       /* history_len / bias_len / ban_len beyond max_history /
                                max_list or beyond the list's row pitch: row refused */
    LILY_ROW_FORCED = 16     /* informational: the row returned its forced id */
};

enum lily_dtype { LILY_F32 = 0, LILY_BF16 = 1 };

/*
 * src/kernels/sample.rs:19-31 SamplingParams, as a 40-byte POD (top_k as
 * u32, 0 = off; negative API values map to 0 as src/serve/api.rs:802-806).
 * `seed` is used only when a call is given draw indices instead of uniforms.
 */
typedef struct lily_sampling_params {
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
    uint32_t reserved;
    uint64_t seed;
} lily_sampling_params_t;

typedef struct lily_sampler lily_sampler_t;

/* ------------------------------------------------------------ host-only -- */

uint32_t lily_abi_version(void);

/* src/kernels/sample.rs:57-79 SamplingParams::validate. */
int32_t lily_params_validate(const lily_sampling_params_t *p);
/* src/kernels/sample.rs:47-49 is_greedy; :51-55 uses_penalties. */
int32_t lily_params_is_greedy(const lily_sampling_params_t *p);
int32_t lily_params_uses_penalties(const lily_sampling_params_t *p);
/* src/kernels/sample.rs:83-94 effective(): what the kernel consumes. */
void lily_params_effective(const lily_sampling_params_t *p, float *temperature,
                           uint32_t *top_k);
/* src/kernels/sample.rs:227-234 draft_params: the request's sampler without
 * the penalties. */
void lily_draft_params(const lily_sampling_params_t *p, lily_sampling_params_t *out);
/* src/kernels/sample.rs:435-441 uniform_for (bit-exact). */
float lily_uniform_for(uint64_t seed, uint32_t step);
/* src/kernels/sample.rs:220-222 draft_step: step | 0x4000_0000. */
uint32_t lily_draft_step(uint32_t step);
/* src/kernels/metal/sample.metal:649 residual-draw domain: step | 0x8000_0000. */
uint32_t lily_residual_step(uint32_t step);

/* ---------------------------------------------------------------- handle -- */

/* lily_sampler_create flags */
#define LILY_FLAG_COUNTS_TABLE 1u /* keep a persistent u32[max_rows, vocab]
                                     emission histogram (the reference's
                                     SamplerScratch::counts), one slot per row */

#define LILY_FLAG_PHASE_CLOCKS 2u /* record per-block phase time stamps (the
                                     counterpart of LILY_KERNEL_PROFILE,
                                     src/metal.rs:140-198); off by default */
#define LILY_MAX_SLICES 128u      /* most thread blocks a row is split over */
#define LILY_PHASES 20u           /* stamps per block, see lily_sampler_read_phase_clocks */

/*
 * src/kernels/sample.rs:130-143 SamplerScratch::new, for `max_rows` rows at
 * once. Allocates on `device`: the per-row candidate scratch, the parameter
 * staging ring, the status words and (with LILY_FLAG_COUNTS_TABLE) the
 * histogram slots. `max_history` bounds history_len; `max_list` bounds the
 * bias and ban list lengths.
 */
int32_t lily_sampler_create(int32_t device, uint32_t vocab, uint32_t max_rows,
                            uint32_t max_history, uint32_t max_list, uint32_t flags,
                            lily_sampler_t **out);
void lily_sampler_destroy(lily_sampler_t *h);
/* src/kernels/sample.rs:176-178 SamplerScratch::vocab. */
uint32_t lily_sampler_vocab(const lily_sampler_t *h);
const char *lily_sampler_last_error(const lily_sampler_t *h);

/*
 * src/metal.rs:681-696 fault latch and MetalContext::inject_fault
 * (src/main.rs:296-301 --debug-inject-metal-fault). Host-side only: after
 * inject_fault(code != 0) every enqueueing call returns LILY_ERR_FAULT until
 * clear_fault. `lily_sampler_status` synchronises `stream`, then returns the
 * latched fault, else the OR-reduced error words of the rows drawn since the
 * last call to it (LILY_ERR_DEVICE_ROW if any row failed).
 */
void lily_sampler_inject_fault(lily_sampler_t *h, int32_t code);
void lily_sampler_clear_fault(lily_sampler_t *h);
int32_t lily_sampler_status(lily_sampler_t *h, void *stream);

/*
 * src/metal.rs:856-861 wait_fence and :1276-1279 Fence::wait_until(value,
 * timeout_ms): the reference bounds its waits on the GPU on the host side. Here
 * the only waits are inside the LM-head kernel (one role of a block waiting for
 * another's copies, conversions or multiplies), and each is bounded on the
 * device: after `nanoseconds` (default and 0: one second) the block gives up,
 * lets the copies and multiplies it still has in flight land, frees its tensor
 * memory and returns. The launch completes like any other; the logits it was to
 * write are not valid, and the next lily_sampler_status returns
 * LILY_ERR_TIMEOUT (once: the status is cleared by reading it). The handle stays
 * usable. The sampler's own kernels wait on nothing another block produces.
 *
 * inject_lost_copy is the device-side sibling of inject_fault, for tests: the
 * next LM-head launch on this handle (and only that one) leaves out the copy of
 * weight stage `stage` of its first block, so that the wait of the stage's
 * consumers runs out. No reference counterpart.
 */
int32_t lily_sampler_set_wait_limit(lily_sampler_t *h, uint64_t nanoseconds);
void lily_sampler_inject_lost_copy(lily_sampler_t *h, uint32_t stage);

/*
 * src/kernels/sample.rs:145-174 reset_counts / uncount / copy_counts_from on
 * histogram slot `slot` (needs LILY_FLAG_COUNTS_TABLE). Stream-ordered.
 * copy_counts refuses handles of different vocabularies (LILY_ERR_VOCAB).
 */
int32_t lily_sampler_reset_counts(lily_sampler_t *h, void *stream, uint32_t slot);
int32_t lily_sampler_uncount(lily_sampler_t *h, void *stream, uint32_t slot, uint32_t token);
int32_t lily_sampler_copy_counts(lily_sampler_t *dst, uint32_t dst_slot,
                                 const lily_sampler_t *src, uint32_t src_slot, void *stream);
/* Test / checkpoint access to a slot's histogram (device-to-host or
 * host-to-device copy of vocab words, stream-ordered then synchronised). */
int32_t lily_sampler_read_counts(lily_sampler_t *h, void *stream, uint32_t slot, uint32_t *host_out);
int32_t lily_sampler_write_counts(lily_sampler_t *h, void *stream, uint32_t slot, const uint32_t *host_in);

/*
 * With LILY_FLAG_PHASE_CLOCKS: copies the time stamps of the last launch
 * (nanoseconds of the GPU's global timer: one time base for all blocks)
 * to host_out[max_rows][LILY_MAX_SLICES][LILY_PHASES] (int64 each, 0 where a
 * block did not pass) and clears them; synchronises `stream`. Stamps 0..7,
 * in order: start, history bitmap built, bias/ban ids done, vocabulary
 * streamed, block's best k selected, slices merged, candidates sorted, draw
 * done. Stamps 8..13 lie between "bitmap built" and "bias/ban ids done":
 * 8 first threshold known; and on the two-pass route (small k) before it
 * 9 pass 1 over the logits done (thread 0), 10 whole block done with it,
 * 11 thread maxima adjusted, 12 threshold searched, 13 threshold stored.
 * 14, 15: on the route that takes its threshold while the row streams,
 * thread 0 has the threshold / has collected what its earlier rounds hold
 * above it; 16 is the block's first instruction.
 * The small-batch kernel (a cluster of eight blocks per row, block r of the
 * cluster in place of slice r) stamps 16 entry, 0 slice loaded and cluster
 * running, 1 history counted, 2 lists / penalties / block maximum, 3 cluster
 * maximum, 9 histogram, 4 barrier, 5 histograms summed and k-th bin found,
 * 10 candidates placed, 6 barrier, 11 ranked, 8 barrier, 7 draw written.
 */
int32_t lily_sampler_read_phase_clocks(lily_sampler_t *h, void *stream, int64_t *host_out);

/* ------------------------------------------------------------------ draw -- */

/*
 * One batch of independent draws: src/kernels/sample.rs:373-387 sample_f32
 * for each row (its greedy route, the exact lowest-index argmax of
 * src/kernels/elementwise.rs:297-308, included), and with the `kept_*`
 * outputs set also :394-408 sample_draft_f32.
 *
 * Order of operations on a row's logits, all in fp32 (bf16 widens exactly):
 *   l = logit + sum of the row's bias entries for that id (list order)
 *   if penalties are on and count(id) > 0:
 *       l = l > 0 ? l / repetition : l * repetition
 *       l -= presence + frequency * count(id)
 *   banned ids: l = -inf
 *   l /= temperature                    (IEEE division)
 * then the top-k by (value descending, id ascending), p = exp(l - l_top),
 * sequential prefix sums in rank order, the top-p / min-p cut relative to
 * the top-k mass, and the inverse-CDF draw on uniform * kept mass.
 *
 * count(id) is the multiplicity of id in the row's history list, or, with
 * `count_slots`, the slot's persistent histogram (which the draw then
 * increments, src/kernels/metal/sample.metal:509-511).
 *
 * Device pointers unless marked HOST. Optional pointers may be NULL.
 */
typedef struct lily_sample_args {
    uint32_t struct_size;        /* sizeof(lily_sample_args_t) */
    uint32_t rows;               /* B, 1..max_rows */
    const void *logits;          /* [rows, logits_ld] of logits_dtype */
    uint32_t logits_dtype;       /* enum lily_dtype */
    uint32_t params_on_device;   /* 0: `params`/`steps` are HOST arrays */
    uint64_t logits_ld;          /* elements between rows (>= vocab) */
    const lily_sampling_params_t *params; /* [rows] */
    const float *uniforms;       /* [rows] in [0,1), or NULL: use steps */
    const uint32_t *steps;       /* [rows] draw indices for uniform_for(seed, step);
                                    same side as params; used when uniforms == NULL */
    const uint32_t *history_ids; /* [rows, history_ld] or NULL */
    const uint32_t *history_len; /* [rows] */
    uint64_t history_ld;
    const uint32_t *bias_ids;    /* [rows, bias_ld] or NULL */
    const float *bias_vals;      /* [rows, bias_ld] */
    const uint32_t *bias_len;    /* [rows] */
    uint64_t bias_ld;
    const uint32_t *ban_ids;     /* [rows, ban_ld] or NULL */
    const uint32_t *ban_len;     /* [rows] */
    uint64_t ban_ld;
    const int32_t *forced_ids;   /* [rows], < 0 = none: the row returns this id
                                    without drawing (thinking-budget forcing) */
    const uint32_t *count_slots; /* HOST [rows] histogram slots, or NULL */
    uint32_t *out_ids;           /* [rows] */
    uint32_t *out_status;        /* [rows] enum lily_row_status, or NULL */
    uint32_t *kept_n;            /* [rows] size of the kept set, or NULL */
    uint32_t *kept_ids;          /* [rows, kept_ld] kept ids in rank order */
    float *kept_probs;           /* [rows, kept_ld] probabilities over the kept mass */
    uint64_t kept_ld;            /* >= LILY_K_CAP when kept_* are set */
} lily_sample_args_t;

int32_t lily_sample_batch(lily_sampler_t *h, void *stream, const lily_sample_args_t *args);

/*
 * The same draw for callers that cannot allocate device memory. (No
 * counterpart in the reference.)
 *
 * Some host programs run with allocation closed: an engine whose memory plan
 * was fixed at start-up and hands every byte of the device to its own pool, a
 * plugin loaded into a process that forbids cudaMalloc after initialisation,
 * or code that must not disturb a stream capture in progress elsewhere with
 * an allocation. lily_sampler_create (which allocates the scratch a handle
 * owns) is of no use to them. This entry point takes no handle and calls no
 * cudaMalloc / cudaFree or any other allocating routine: the scratch the
 * kernel needs (the slices' candidate lists, their counters and tickets, the
 * staged parameters) lives in one array of static device storage inside the
 * library, LILY_NOALLOC_SCRATCH_BYTES large, which every GPU that loads the
 * library holds until the process exits.
 *
 * Limits: rows <= LILY_NOALLOC_MAX_ROWS; `params` (and `steps`) HOST arrays;
 * no histogram slots (`count_slots` must be NULL); a history-list row may not
 * use a frequency penalty (that needs a vocabulary-sized count table): such
 * calls are refused with LILY_ERR_CAPACITY. Results are the same as
 * lily_sample_batch's.
 *
 * The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; make it
 * before any stream capture. All calls share the one array: it keeps the last
 * call's contents (the entry point clears the words that must start at zero),
 * and two calls that overlap on the GPU, on any streams, race on it. On the
 * host the entry point may be called from several threads (the one-time
 * set-up is behind a mutex); keeping their launches from overlapping on the
 * GPU stays the caller's job. A row that fails on the device (a NaN, no
 * finite logit, an over-long list) is reported through `out_status` only:
 * there is no handle whose status word could be read back, so pass
 * `out_status` when such rows are possible.
 * `vocab` is the row length; errors are written to err[0..err_cap).
 */
#define LILY_NOALLOC_MAX_ROWS 8u
#define LILY_NOALLOC_SCRATCH_BYTES (LILY_NOALLOC_MAX_ROWS * (4096u * 8u + 128u * 4u + 64u) + 256u)
int32_t lily_sample_batch_noalloc(void *stream, uint32_t vocab, const lily_sample_args_t *args,
                                  char *err, uint32_t err_cap);

/*
 * src/kernels/elementwise.rs:297-308 argmax_f32 for each row: first maximum,
 * lowest index on ties, NaN never wins.
 */
int32_t lily_argmax_batch(lily_sampler_t *h, void *stream, const void *logits,
                          uint32_t logits_dtype, uint64_t logits_ld, uint32_t rows,
                          uint32_t *out_ids);

/* ------------------------------------------------------------ speculation -- */

enum lily_spec_mode {
    LILY_SPEC_REJECTION = 0,   /* speculative sampling with the residual draw */
    LILY_SPEC_GREEDY_MATCH = 1 /* every row is the argmax; equality accepts */
};

/*
 * One verify step of a speculative decode: src/qwen4exp/model.rs:3013-3040
 * (rows j < m-1: src/kernels/sample.rs:417-432 sample_spec_f32 against
 * proposal j; last row: sample_f32), followed by the accepted count of
 * src/kernels/metal/spec.metal:26-29. Rows share the request's penalty
 * state: with penalties on, row j sees the draws of rows < j of this step.
 *
 * The draft distribution of proposal j is either dense, q_dense[j, id], or
 * the reference's sparse export (src/kernels/sample.rs:186-215 DraftDists):
 * q_ids / q_probs [m-1, LILY_K_CAP] with q_n[j] entries.
 */
typedef struct lily_spec_args {
    uint32_t struct_size;
    uint32_t m;                  /* verified rows: drafts + 1 (<= 8) */
    const void *target_logits;   /* [m, logits_ld] */
    uint32_t logits_dtype;
    uint32_t mode;               /* enum lily_spec_mode */
    uint64_t logits_ld;
    const lily_sampling_params_t *params; /* HOST, one request */
    const uint32_t *draft_ids;   /* [m-1] proposals */
    const float *q_dense;        /* [m-1, q_ld] or NULL */
    uint64_t q_ld;
    const uint32_t *q_ids;       /* [m-1, LILY_K_CAP] or NULL */
    const float *q_probs;        /* [m-1, LILY_K_CAP] */
    const uint32_t *q_n;         /* [m-1] */
    const float *u_accept;       /* [m] accept test / plain draw uniforms, or NULL */
    const float *u_resid;        /* [m-1] residual draw uniforms, or NULL */
    uint32_t step0;              /* with NULL uniforms: row j draws uniform_for(seed, step0+j)
                                    and its residual on step | 0x8000_0000 */
    uint32_t history_len;        /* HOST value */
    const uint32_t *history_ids; /* [history_len] or NULL */
    const uint32_t *count_slot;  /* HOST pointer to one slot index, or NULL */
    uint32_t *out_ids;           /* [m] */
    uint32_t *out_accepted;      /* [1] */
    uint32_t *out_status;        /* [m] or NULL */
} lily_spec_args_t;

int32_t lily_spec_verify(lily_sampler_t *h, void *stream, const lily_spec_args_t *args);

/*
 * src/kernels/spec.rs:52-91 spec_accept with its control block
 * (src/kernels/metal/spec.metal:8-38): ctrl[0] = a, ctrl[stride] = a + 1,
 * then per chain row i the position pos0 + a + 1 + i, its block
 * (position / ratio) and whether it completes one. `stride` words between
 * slots (the reference uses 4). ctrl holds (2 + 3*chain) * stride words.
 */
int32_t lily_spec_accept(lily_sampler_t *h, void *stream, const uint32_t *draws,
                         const uint32_t *ids, uint32_t m, uint32_t *ctrl, uint32_t pos0,
                         uint32_t ratio, uint32_t chain, uint32_t stride);

/* ------------------------------------------- 8-bit LM head, vocab shards -- */

/*
 * The projection that produces the logits the sampler reads, for a head
 * stored in 8 bits. In the reference this is gemv_quant
 * (src/kernels/quant.rs:141-175) called per row from
 * src/qwen4exp/model.rs:2999-3006 on MLX affine 4/8-bit weights; the format
 * here is the symmetric one of the vocab-sharded configuration:
 *
 *   logits[t, n] = sum_g scale[n, g] * sum_{c in group g} w[n, c] * hidden[t, c]
 *
 * w int8 [rows, hidden], scale bf16 [rows, hidden / 64] (one per 64 columns),
 * hidden bf16 [tokens, hidden_ld], all sums in binary32 (group sums on the
 * tensor cores, exact products, then scaled and added in group order).
 * tokens <= 64, hidden a multiple of 512, every pointer 16-byte aligned.
 *
 * With `biases_bf16` set the head is in MLX affine 8-bit storage and
 *
 *   logits[t, n] = sum_g ( scale[n, g] * sum_c (q[n, c] - 128) * hidden[t, c]
 *                          + (128 * scale[n, g] + bias[n, g]) * sum_c hidden[t, c] )
 *
 * which is sum_c (scale * q + bias) * hidden up to binary32 rounding (the
 * reference's own test allows 2e-2 + 2e-2 |x| against a dequantise-then-
 * multiply sum, tests/unit/kernels/quant.rs:418-434). With `code_bits` = 4 the
 * codes are 4 bits wide (q in 0..15, widened as they are) and
 *
 *   logits[t, n] = sum_g ( scale[n, g] * sum_c q[n, c] * hidden[t, c]
 *                          + bias[n, g] * sum_c hidden[t, c] ).
 */
typedef struct lily_lmhead {
    uint32_t struct_size;        /* sizeof(lily_lmhead_t) */
    uint32_t rows;               /* vocabulary rows held here (a shard, or all) */
    uint32_t hidden;             /* columns */
    uint32_t group;              /* columns per scale: 64 */
    const int8_t *weights;       /* device [rows, hidden] */
    const void *scales_bf16;     /* device [rows, hidden / group] */
    const void *biases_bf16;     /* NULL: the symmetric format above. Else the
                                    reference's own 8-bit storage, MLX affine
                                    (src/weights.rs:21-36): `weights` holds
                                    UNSIGNED bytes q (QuantWeights::codes, U32
                                    [rows, hidden / 4], low byte first, is the
                                    same memory), w = scale * q + bias, and
                                    this is device bf16 [rows, hidden / group];
                                    hidden <= 8192 */
    uint32_t code_bits;          /* 0 or 8: a byte per weight, as above. 4 (with
                                    biases set): MLX affine 4-bit storage, the
                                    format gemv_q4_bf16 reads
                                    (src/kernels/metal/quant.metal:44-66): `weights`
                                    is QuantWeights::codes, U32 [rows, hidden / 8],
                                    eight codes to a word, low nibble first;
                                    w = scale * q + bias with q in 0..15 */
    uint32_t reserved;
} lily_lmhead_t;

/* out_logits: device F32 [tokens, out_ld >= rows]. Needs no handle state
 * beyond the status word; any handle of the device serves. */
int32_t lily_lmhead_logits(lily_sampler_t *h, void *stream, const lily_lmhead_t *head,
                           const void *hidden_bf16, uint64_t hidden_ld, uint32_t tokens,
                           float *out_logits, uint64_t out_ld);

/*
 * Vocabulary shards (no counterpart in the reference, which keeps the whole
 * head on one GPU; its two-phase select, src/kernels/metal/sample.metal:
 * 664-701, is the same idea inside one device). Shard s holds the logits of
 * ids [first_id, first_id + vocab) and runs lily_shard_candidates: per row it
 * keeps its best LILY_SHARD_CANDIDATES candidates (a greedy row: 1), sorted,
 * with the shard's largest adjusted logit and sum of exponentials, as one
 * 520-byte record. The caller gathers all shards' records onto every rank
 * (an all-gather of tokens * 520 bytes per rank) and calls lily_merge_draw,
 * which selects, cuts and draws over the union: the same token on every
 * rank, and the token one pass over the whole vocabulary draws, because the
 * global top-k lies inside the union of the shards' top-64.
 *
 * Limits: params are HOST arrays; sampled rows need 1 <= top_k <= 64; no
 * penalties, bias, ban or forced ids (their ids would be global, the shard's
 * logits are local): refused with LILY_ERR_ARG.
 */
#define LILY_SHARD_CANDIDATES 64u
#define LILY_SHARD_RECORD_BYTES 520u

/*
 * args: logits (this shard's, [rows, ld >= handle vocab]), logits_dtype,
 * rows, params; everything else must be NULL / 0. records: device
 * [rows] x 520 bytes. want_sums != 0 also fills each record's sum of
 * exponentials (one more pass over the logits).
 */
int32_t lily_shard_candidates(lily_sampler_t *h, void *stream, const lily_sample_args_t *args,
                              uint32_t first_id, int32_t want_sums, void *records);

/* lily_lmhead_logits into the handle's own logits scratch (created with
 * LILY_FLAG_LMHEAD: F32 [64, vocab]) followed by lily_shard_candidates on it.
 * head->rows must equal the handle's vocab. */
#define LILY_FLAG_LMHEAD 4u
int32_t lily_lmhead_shard_candidates(lily_sampler_t *h, void *stream, const lily_lmhead_t *head,
                                     const void *hidden_bf16, uint64_t hidden_ld,
                                     const lily_sample_args_t *args, uint32_t first_id,
                                     int32_t want_sums, void *records);

/*
 * gathered: device [n_shards, shard_stride >= rows] records, shard-major.
 * args: rows, params, uniforms or steps, out_ids, and optionally out_status
 * and kept_*; logits and lists NULL. out_lse: optional device [rows], the log
 * of the sum over the whole vocabulary of exp(adjusted logit), valid when the
 * records were made with want_sums. n_shards <= 64.
 */
int32_t lily_merge_draw(lily_sampler_t *h, void *stream, const void *gathered, uint32_t n_shards,
                        uint64_t shard_stride, const lily_sample_args_t *args, float *out_lse);

/*
 * The same exchange without a collective library: every rank writes its records
 * straight into every rank's memory (peer stores over NVLink) and raises a
 * flag there; the merge waits for the flags. No counterpart in the reference.
 *
 * A rank owns one exchange buffer (lily_peer_buffer_create: device memory of
 * lily_peer_buffer_bytes, zeroed, and its 64-byte inter-process handle): a flag
 * word per (rank, row), then two slots of n_shards x max_rows records. The
 * ranks pass the handles around by any means, open each other's buffers
 * (lily_peer_buffer_open: the buffer as THIS process sees it; peer access is
 * enabled on the way) and fill a lily_peer_exchange_t, own buffer included.
 * Per step, with `step` counting 1, 2, 3, ... on every rank alike, ONE call and
 * one kernel, lily_merge_draw_peer: the block of row r writes this rank's record
 * of the row (`records`, as lily_shard_candidates left them) into slot
 * (step & 1, rank) of every buffer, fences system-wide and sets flag[rank][r] :=
 * step there; then it waits until the n_shards flags of row r in the OWN buffer
 * have reached `step` (bounded by lily_sampler_set_wait_limit; on time-out the
 * status becomes LILY_ERR_TIMEOUT and the draw is not valid) and merges the
 * row as lily_merge_draw does. Rows wait for nothing but their own records, so
 * the exchange of one row overlaps the merge of another.
 * lily_shard_publish does the first half alone, for all rows at once (a rank
 * that publishes apart from its merge then passes records = NULL to
 * lily_merge_draw_peer).
 *
 * Two slots suffice: a rank cannot publish step n + 2 before it has merged step
 * n + 1, which every rank publishes only after it has merged step n. All ranks
 * must be single GPUs of one node with peer access to each other, one process
 * per GPU; a rank must not skip a step.
 */
#define LILY_PEER_MAX 16u
#define LILY_IPC_HANDLE_BYTES 64u
typedef struct lily_peer_exchange {
    uint32_t struct_size;             /* sizeof(lily_peer_exchange_t) */
    uint32_t n_shards;                /* ranks, <= LILY_PEER_MAX */
    uint32_t rank;                    /* this rank */
    uint32_t max_rows;                /* as given to lily_peer_buffer_create, the same on every rank */
    void *buffers[LILY_PEER_MAX];     /* rank r's exchange buffer as this process sees it */
} lily_peer_exchange_t;

uint64_t lily_peer_buffer_bytes(uint32_t n_shards, uint32_t max_rows);
int32_t lily_peer_buffer_create(int32_t device, uint32_t n_shards, uint32_t max_rows, void **buffer,
                                void *ipc_handle);
int32_t lily_peer_buffer_open(int32_t device, const void *ipc_handle, void **buffer);
int32_t lily_peer_buffer_close(int32_t device, void *buffer);
int32_t lily_peer_buffer_destroy(int32_t device, void *buffer);
int32_t lily_shard_publish(lily_sampler_t *h, void *stream, const lily_peer_exchange_t *x,
                           const void *records, uint32_t rows, uint32_t step);
int32_t lily_merge_draw_peer(lily_sampler_t *h, void *stream, const lily_peer_exchange_t *x,
                             const void *records, uint32_t step, const lily_sample_args_t *args,
                             float *out_lse);

/* ------------------------------------------------------------------ test -- */

/*
 * out[i] = the kernels' exp(in[i]) (device pointers). The reference calls the
 * platform's f32::exp (tests/unit/kernels/sample.rs:37); this library uses
 * one fixed sequence of binary32 operations instead so that results do not
 * depend on the platform. Exposed so that a checker can compare it.
 */
int32_t lily_debug_exp(void *stream, const float *in, float *out, uint64_t n);

#ifdef __cplusplus
}
#endif
#endif /* LILY_SAMPLER_H */
