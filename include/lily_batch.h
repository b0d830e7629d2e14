/*
 * lily_batch.h -- C ABI of the scheduler-side bookkeeping around the sampler
 * when requests decode as rows of a batch: which histogram slot holds a
 * request's penalty counts and when they move, the draw index of a row of a
 * committed or parked step, and the host decisions that keep a parked step
 * from getting ahead of a row that must rest.
 *
 * Replaces, for the sampling path only:
 *   src/serve/batch.rs:74-102    Slots (take / give / in_use)
 *   src/serve/batch.rs:110-139   admits, Next, next_action
 *   src/serve/batch.rs:141-189   RowAhead, park_next
 *   src/serve/batch.rs:191-226   SoloStop
 *   src/serve/batch.rs:228-264   BatchStats::record_step / mean_rows
 *   src/serve/batch.rs:421-438   batch_of: step = generated.len() + ahead
 *   src/engine.rs:588-596        CountsSlot
 *   src/engine.rs:983-994, src/qwen4exp/batch.rs:137-162  move_sampler_counts
 *
 * Host logic, except lily_move_counts, which enqueues device copies.
 */
#ifndef LILY_BATCH_H
#define LILY_BATCH_H

#include <stdint.h>

#include "lily_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ slots -- */

/* src/serve/batch.rs:74-102. Each batch slot owns one histogram slot of the
 * batch sampler handle (slot i of a handle created with max_rows >= n). */
typedef struct lily_slots lily_slots_t;

int32_t lily_slots_create(uint32_t n, lily_slots_t **out);
void lily_slots_destroy(lily_slots_t *s);
/* The lowest free slot, now taken; -1 when every slot is taken. */
int32_t lily_slots_take(lily_slots_t *s);
/* Gives a slot back. A slot outside the table is ignored rather than growing
 * it; giving back a free slot changes nothing and returns LILY_ERR_ARG (the
 * reference asserts in debug builds). */
int32_t lily_slots_give(lily_slots_t *s, uint32_t slot);
uint32_t lily_slots_in_use(const lily_slots_t *s);
uint32_t lily_slots_capacity(const lily_slots_t *s);

/* ------------------------------------------------------------ counts slot -- */

/* src/engine.rs:588-596 CountsSlot: LILY_COUNTS_ENGINE is the engine's own
 * sampler (prefill draws, the single-session loop, speculation); any other
 * value i is CountsSlot::Batch(i). */
#define LILY_COUNTS_ENGINE 0xFFFFFFFFu

/*
 * move_sampler_counts (src/qwen4exp/batch.rs:137-162): copies a request's
 * penalty counts between the engine's handle (its histogram slot 0) and slot i
 * of the batch handle, or between two batch slots. from == to is a no-op that
 * touches neither handle. A batch slot outside the batch handle is refused
 * with LILY_ERR_ARG ("batch slot i of n"). Stream-ordered on `stream`; the
 * caller keeps both handles' draws ordered against it (the reference: "The
 * GPU must be idle on both"). `engine` and `batch` may be the same handle
 * only if no batch slot is 0.
 */
int32_t lily_move_counts(lily_sampler_t *engine, lily_sampler_t *batch, void *stream,
                         uint32_t from, uint32_t to);

/* ------------------------------------------------------------- draw index -- */

/* src/serve/batch.rs:421-438: the draw index of a row in the step that feeds
 * its last draw (`ahead` 0) or in the step parked behind that one (`ahead`
 * 1): generated + ahead. It is the `step` of lily_uniform_for. */
uint32_t lily_row_draw_step(uint64_t generated, uint32_t ahead);

/* -------------------------------------------------------------- decisions -- */

/* src/serve/batch.rs:110-118. Sizes saturate instead of overflowing. */
int32_t lily_admits(uint64_t rows, uint64_t max_rows, uint64_t in_flight, uint64_t estimate,
                    uint64_t budget);

/* src/serve/batch.rs:120-139. */
enum lily_next { LILY_NEXT_DONE = 0, LILY_NEXT_SOLO = 1, LILY_NEXT_STEP = 2 };
/* *preempt (may be NULL) is written for LILY_NEXT_SOLO: !held. */
int32_t lily_next_action(uint64_t rows, int32_t held, int32_t *preempt);

/* src/serve/batch.rs:141-160 RowAhead. */
typedef struct lily_row_ahead {
    uint64_t pos;           /* where the committed step leaves the row */
    uint64_t capacity;      /* tokens its caches hold before they grow */
    uint8_t checkpoint_due; /* a decode checkpoint is due at pos */
    uint8_t ending;         /* the committed step's draw ends the row */
    uint8_t may_insert;     /* its thinking control may act on that draw */
    uint8_t reserved[5];
} lily_row_ahead_t;

/* src/serve/batch.rs:162-189: whether the next step may be committed behind
 * the one just committed, before that one's draws are read. */
int32_t lily_park_next(const lily_row_ahead_t *rows, uint32_t n, int32_t another_step,
                       int32_t admission, int32_t cancel);

/* src/serve/batch.rs:191-226 SoloStop. Zero-initialise. */
typedef struct lily_solo_stop {
    uint8_t yielded;
    uint8_t terminal;
} lily_solo_stop_t;
/* Records one callback; returns whether the loop goes on. */
int32_t lily_solo_stop_observe(lily_solo_stop_t *s, int32_t terminal, int32_t waiting);
int32_t lily_solo_stop_yielded_only(const lily_solo_stop_t *s);

/* src/serve/batch.rs:228-264 BatchStats (the counters; the log line is the
 * server's). `peers` is caller storage of `peers_cap` sequence numbers. */
typedef struct lily_batch_stats {
    uint64_t batched_tokens;
    uint64_t rows_sum;
    uint64_t max_rows;
    uint64_t *peers;
    uint32_t n_peers;
    uint32_t peers_cap;
} lily_batch_stats_t;
/* One batched step of the rows `members`, `own` among them. LILY_ERR_ARG when
 * a new peer does not fit `peers_cap` (the counters are still updated). */
int32_t lily_batch_stats_record_step(lily_batch_stats_t *s, uint64_t own, const uint64_t *members,
                                     uint32_t n);
/* rows_sum / batched_tokens, or a negative value before the first step. */
double lily_batch_stats_mean_rows(const lily_batch_stats_t *s);

#ifdef __cplusplus
}
#endif

#endif /* LILY_BATCH_H */
