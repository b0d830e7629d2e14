// Scheduler-side bookkeeping around the sampler for requests that decode as
// rows of a batch (include/lily_batch.h): the slot table, the draw index of a
// row, and the host decisions about parking the next step. Host logic only;
// lily_move_counts, which enqueues device copies, lives beside the handle.
#include <cstdint>
#include <new>
#include <vector>

#include "lily_batch.h"

struct lily_slots {
    std::vector<uint8_t> free_;
};

namespace {

uint64_t saturating_add(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    return s < a ? UINT64_MAX : s;
}

}  // namespace

extern "C" {

int32_t lily_slots_create(uint32_t n, lily_slots_t **out) {
    if (out == nullptr) {
        return LILY_ERR_ARG;
    }
    lily_slots *s = new (std::nothrow) lily_slots;
    if (s == nullptr) {
        return LILY_ERR_ARG;
    }
    s->free_.assign(n, 1);
    *out = s;
    return LILY_OK;
}

void lily_slots_destroy(lily_slots_t *s) { delete s; }

int32_t lily_slots_take(lily_slots_t *s) {
    if (s == nullptr) {
        return -1;
    }
    for (size_t i = 0; i < s->free_.size(); ++i) {
        if (s->free_[i]) {
            s->free_[i] = 0;
            return static_cast<int32_t>(i);
        }
    }
    return -1;
}

int32_t lily_slots_give(lily_slots_t *s, uint32_t slot) {
    if (s == nullptr) {
        return LILY_ERR_ARG;
    }
    if (slot >= s->free_.size()) {
        return LILY_OK;  // ignored, the table does not grow
    }
    if (s->free_[slot]) {
        return LILY_ERR_ARG;  // given back twice
    }
    s->free_[slot] = 1;
    return LILY_OK;
}

uint32_t lily_slots_in_use(const lily_slots_t *s) {
    uint32_t n = 0;
    if (s != nullptr) {
        for (uint8_t f : s->free_) {
            n += f ? 0u : 1u;
        }
    }
    return n;
}

uint32_t lily_slots_capacity(const lily_slots_t *s) {
    return s ? static_cast<uint32_t>(s->free_.size()) : 0u;
}

uint32_t lily_row_draw_step(uint64_t generated, uint32_t ahead) {
    return static_cast<uint32_t>(generated + ahead);
}

int32_t lily_admits(uint64_t rows, uint64_t max_rows, uint64_t in_flight, uint64_t estimate,
                    uint64_t budget) {
    return rows == 0 || (rows < max_rows && saturating_add(in_flight, estimate) <= budget);
}

int32_t lily_next_action(uint64_t rows, int32_t held, int32_t *preempt) {
    if (rows == 0) {
        return LILY_NEXT_DONE;
    }
    if (rows == 1) {
        if (preempt != nullptr) {
            *preempt = held ? 0 : 1;
        }
        return LILY_NEXT_SOLO;
    }
    return LILY_NEXT_STEP;
}

int32_t lily_park_next(const lily_row_ahead_t *rows, uint32_t n, int32_t another_step,
                       int32_t admission, int32_t cancel) {
    if (!another_step || admission || cancel || (rows == nullptr && n != 0)) {
        return 0;
    }
    for (uint32_t i = 0; i < n; ++i) {
        const lily_row_ahead_t &r = rows[i];
        // Room for the parked step and the one after it: pos + 1 < capacity.
        if (r.checkpoint_due || r.ending || r.may_insert ||
            saturating_add(r.pos, 1) >= r.capacity) {
            return 0;
        }
    }
    return 1;
}

int32_t lily_solo_stop_observe(lily_solo_stop_t *s, int32_t terminal, int32_t waiting) {
    if (terminal) {
        s->terminal = 1;
        return 0;
    }
    if (waiting) {
        s->yielded = 1;
        return 0;
    }
    return 1;
}

int32_t lily_solo_stop_yielded_only(const lily_solo_stop_t *s) {
    return s->yielded && !s->terminal;
}

int32_t lily_batch_stats_record_step(lily_batch_stats_t *s, uint64_t own, const uint64_t *members,
                                     uint32_t n) {
    if (s == nullptr || (members == nullptr && n != 0)) {
        return LILY_ERR_ARG;
    }
    s->batched_tokens += 1;
    s->rows_sum += n;
    if (n > s->max_rows) {
        s->max_rows = n;
    }
    int32_t st = LILY_OK;
    for (uint32_t i = 0; i < n; ++i) {
        const uint64_t m = members[i];
        if (m == own) {
            continue;
        }
        bool known = false;
        for (uint32_t j = 0; j < s->n_peers && !known; ++j) {
            known = s->peers[j] == m;
        }
        if (known) {
            continue;
        }
        if (s->peers == nullptr || s->n_peers >= s->peers_cap) {
            st = LILY_ERR_ARG;
            continue;
        }
        s->peers[s->n_peers++] = m;
    }
    return st;
}

double lily_batch_stats_mean_rows(const lily_batch_stats_t *s) {
    if (s == nullptr || s->batched_tokens == 0) {
        return -1.0;
    }
    return static_cast<double>(s->rows_sum) / static_cast<double>(s->batched_tokens);
}

}  // extern "C"
