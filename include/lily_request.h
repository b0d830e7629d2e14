/*
 * lily_request.h -- C ABI of the layer between an OpenAI-style request and
 * the sampler: the request's sampling fields over the server's defaults
 * (src/serve/api.rs:436-457, 798-834), the checkpoint's defaults
 * (src/serve.rs:1762-1835) and the thinking controls' fields, budgets and
 * defaults (src/serve/api.rs:498-708, 861-888), resolved into the
 * lily_sampling_params_t the sampler takes and the lily_thinking_settings_t
 * the thinking control takes.
 *
 * Pure host logic. Errors: nonzero return, reason written to err[0..err_cap).
 */
#ifndef LILY_REQUEST_H
#define LILY_REQUEST_H

#include <stdint.h>

#include "lily_sampler.h"
#include "lily_thinking.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Bits of `present` in the structs below. */
enum lily_field_bits {
    LILY_HAS_TEMPERATURE = 1u << 0,
    LILY_HAS_TOP_P = 1u << 1,
    LILY_HAS_TOP_K = 1u << 2,
    LILY_HAS_MIN_P = 1u << 3,
    LILY_HAS_SEED = 1u << 4,
    LILY_HAS_PRESENCE = 1u << 5,
    LILY_HAS_FREQUENCY = 1u << 6,
    LILY_HAS_REPETITION = 1u << 7,
    LILY_HAS_THINKING_BUDGET = 1u << 8,
    LILY_HAS_THINKING_NUDGES = 1u << 9,
    LILY_HAS_TOOL_CALL_ENDS_THINKING = 1u << 10
};

/* src/serve.rs SamplingOverrides (the command-line overrides): the fields
 * whose bit is set in `present` replace the checkpoint's value. */
typedef struct lily_sampling_overrides {
    uint32_t present;
    float temperature;
    uint64_t top_k;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
} lily_sampling_overrides_t;

/*
 * src/serve.rs:1762-1835 sampling_defaults / sampling_unvalidated: OpenAI's
 * defaults (T 1, top_k off, top_p 1, no penalties), then the checkpoint's
 * generation_config.json (do_sample false -> T 0; temperature, top_p, top_k,
 * min_p, repetition_penalty, presence_penalty), then the overrides.
 * `generation_config_json` may be NULL (no such file). `validate` != 0 adds
 * SamplingParams::validate.
 */
int32_t lily_sampling_defaults(const char *generation_config_json, uint32_t len,
                               const lily_sampling_overrides_t *overrides, int32_t validate,
                               lily_sampling_params_t *out, char *err, uint32_t err_cap);

/* src/serve/api.rs:436-457 SamplingFields and :498-512 ThinkingFields, the
 * two groups a request flattens into its top level. */
typedef struct lily_request_fields {
    uint32_t present;
    float temperature;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
    int64_t top_k;
    int64_t seed;
    int64_t thinking_budget;
    int32_t thinking_nudges;
    int32_t tool_call_ends_thinking;
} lily_request_fields_t;

/*
 * The two groups read from a request body (any other member is ignored, as
 * serde's flatten does; `logit_bias` too: the reference parses and ignores
 * it, tests/unit/serve.rs:152). A chat request's `chat_template_kwargs` win
 * over the top-level thinking fields (src/serve/api.rs:525-563 from_kwargs,
 * or). A thinking_budget of 0 is refused wherever it comes from (:516-523).
 */
int32_t lily_request_fields_from_json(const char *body, uint32_t len, lily_request_fields_t *out,
                                      char *err, uint32_t err_cap);

/*
 * src/serve/api.rs:798-834 resolve_sampling: the request's fields over
 * `defaults`; a negative top_k means off; without a seed the caller's
 * `entropy` is the seed (the reference mixes the clock and the process id);
 * then SamplingParams::validate.
 */
int32_t lily_resolve_sampling(const lily_request_fields_t *fields,
                              const lily_sampling_params_t *defaults, uint64_t entropy,
                              lily_sampling_params_t *out, char *err, uint32_t err_cap);

/* src/serve/api.rs:591-600 ThinkingBudgets; a level without a budget is < 0. */
typedef struct lily_thinking_budgets {
    int64_t low;
    int64_t medium;
    int64_t xhigh;
} lily_thinking_budgets_t;

#define LILY_MAX_THINKING_TOKENS (1u << 20) /* src/serve/api.rs:605 */
#define LILY_MAX_TOOL_TURN_FACTOR 100.0     /* :606 */

/* :608-650 ThinkingBudgets::parse: "off", one number for every level, or
 * level=tokens pairs ("high" is "xhigh"). */
int32_t lily_thinking_budgets_parse(const char *text, lily_thinking_budgets_t *out, char *err,
                                    uint32_t err_cap);
/* :654-660 ThinkingBudgets::at; effort NULL = the template's default (xhigh).
 * Returns the budget or -1. */
int64_t lily_thinking_budgets_at(const lily_thinking_budgets_t *b, const char *effort);
/* :881-888 template_effort: "low", "medium", "xhigh" ("high", "max") or NULL. */
const char *lily_template_effort(const char *value);

/* :666-689 ThinkingDefaults (and its Default). */
typedef struct lily_thinking_defaults {
    lily_thinking_budgets_t budgets;
    double tool_turn_factor;
    int32_t nudges;
    int32_t tool_call_ends_thinking;
    uint64_t grace;
} lily_thinking_defaults_t;

void lily_thinking_defaults_init(lily_thinking_defaults_t *d);
/* :692-698 validate (check_tool_turn_factor :861, check_grace :870). */
int32_t lily_thinking_defaults_validate(const lily_thinking_defaults_t *d, char *err, uint32_t err_cap);
/* :700-708 budget: the server's budget for a chat turn, -1 for none. */
int64_t lily_thinking_defaults_budget(const lily_thinking_defaults_t *d, const char *effort,
                                      int32_t tool_turn);

/* :568-589 ThinkingFields::resolve; default_budget < 0 = none. */
void lily_thinking_resolve(const lily_request_fields_t *fields, const lily_thinking_defaults_t *defaults,
                           int64_t default_budget, uint64_t seed, lily_thinking_settings_t *out);

#ifdef __cplusplus
}
#endif
#endif /* LILY_REQUEST_H */
