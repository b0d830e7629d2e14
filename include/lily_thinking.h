/*
 * lily_thinking.h -- C ABI of the host half of the sampling path: the
 * thinking-budget control that decides WHEN tokens are forced into, or kept
 * out of, the stream the sampler draws (src/thinking.rs of the reference),
 * and the helpers that emit the groups it asks for (src/generate.rs:121-169).
 *
 * Pure host logic: no CUDA, no allocation visible to the caller beyond the
 * opaque objects. The tokenizer stays with the caller, exactly as in the
 * reference, where ThinkingTokens::new takes an `encode` closure
 * (src/thinking.rs:247-254): here it is a callback.
 */
#ifndef LILY_THINKING_H
#define LILY_THINKING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* src/thinking.rs:109 DEFAULT_GRACE */
#define LILY_THINKING_DEFAULT_GRACE 128u

/* src/thinking.rs:113-131 NudgeLevel / ThinkingTexts (UTF-8, NUL-terminated). */
typedef struct lily_nudge_level {
    double at;
    const char *const *texts;
    uint32_t n_texts;
} lily_nudge_level_t;

typedef struct lily_thinking_texts {
    const char *const *close;
    uint32_t n_close;
    const lily_nudge_level_t *nudges;
    uint32_t n_nudges;
} lily_thinking_texts_t;

/*
 * The tokenizer's plain encoding of `utf8[0..len)`: writes up to `cap` ids
 * and returns how many the text has (call again with more room if that is
 * above `cap`), or a negative value on failure.
 */
typedef int32_t (*lily_encode_fn)(void *user, const char *utf8, uint32_t len, uint32_t *out_ids,
                                  uint32_t cap);
/* Whether `id` is one of the vocabulary's added tokens (special or not). */
typedef int32_t (*lily_is_added_fn)(void *user, uint32_t id);

typedef struct lily_thinking_tokens lily_thinking_tokens_t;
typedef struct lily_thinking_control lily_thinking_control_t;

/*
 * src/thinking.rs:247-325 ThinkingTokens::new. `texts` NULL = the built-in
 * set (src/thinking.rs:133-170). On failure returns nonzero and writes the
 * reason to err[0..err_cap).
 */
int32_t lily_thinking_tokens_create(uint32_t think_end, uint32_t tool_call, uint32_t tool_call_end,
                                    const lily_thinking_texts_t *texts, lily_encode_fn encode,
                                    lily_is_added_fn is_added, void *user,
                                    lily_thinking_tokens_t **out, char *err, uint32_t err_cap);
/*
 * The same with the texts read from JSON of the shape the reference's
 * --thinking-texts file has (src/thinking.rs:120-131, unknown fields
 * refused): {"close": ["..."], "nudges": [{"at": 0.5, "texts": ["..."]}]}.
 */
int32_t lily_thinking_tokens_create_json(uint32_t think_end, uint32_t tool_call,
                                         uint32_t tool_call_end, const char *json, uint32_t json_len,
                                         lily_encode_fn encode, lily_is_added_fn is_added,
                                         void *user, lily_thinking_tokens_t **out, char *err,
                                         uint32_t err_cap);
void lily_thinking_tokens_destroy(lily_thinking_tokens_t *t);

/* src/thinking.rs:329-352 ThinkingSettings; budget < 0 = none. */
typedef struct lily_thinking_settings {
    int64_t budget;
    uint64_t grace;
    int32_t nudges;
    int32_t tool_call_ends_thinking;
    uint64_t seed;
} lily_thinking_settings_t;

/* src/thinking.rs:349-351 ThinkingSettings::any */
int32_t lily_thinking_settings_any(const lily_thinking_settings_t *s);

/* src/thinking.rs:356-367 Action */
enum lily_action { LILY_ACTION_KEEP = 0, LILY_ACTION_BEFORE = 1, LILY_ACTION_AFTER = 2,
                   LILY_ACTION_REPLACE = 3 };
/* src/thinking.rs:371-376 ClosedBy */
enum lily_closed_by { LILY_CLOSED_TOOL_CALL = 0, LILY_CLOSED_BUDGET = 1,
                      LILY_CLOSED_END_OF_TURN = 2 };

/* src/thinking.rs:421-436 ThinkingControl::new. The control keeps a reference
 * to `tokens`, which must outlive it. */
lily_thinking_control_t *lily_thinking_control_create(const lily_thinking_tokens_t *tokens,
                                                      const lily_thinking_settings_t *settings,
                                                      int32_t opens_thinking);
void lily_thinking_control_destroy(lily_thinking_control_t *c);

/* src/thinking.rs:439-466 */
int32_t lily_thinking_is_open(const lily_thinking_control_t *c);
int32_t lily_thinking_closed(const lily_thinking_control_t *c, int32_t *by,
                             uint64_t *thinking_tokens); /* 1 if a close was asked for */
int32_t lily_thinking_close_emitted(const lily_thinking_control_t *c, const uint32_t *generated,
                                    uint64_t n);
uint64_t lily_thinking_nudged(const lily_thinking_control_t *c);
uint64_t lily_thinking_tokens_counted(const lily_thinking_control_t *c);
/* src/thinking.rs:485-487 may_act_next */
int32_t lily_thinking_may_act_next(const lily_thinking_control_t *c);

/*
 * src/thinking.rs:516-584 decide / :596-608 decide_stop. Return an
 * enum lily_action; the tokens to insert (for anything but KEEP) stay valid
 * until the next call on this control: lily_thinking_action_ids.
 */
int32_t lily_thinking_decide(lily_thinking_control_t *c, uint32_t token, const char *text_utf8,
                             uint32_t len);
int32_t lily_thinking_decide_stop(lily_thinking_control_t *c);
void lily_thinking_action_ids(const lily_thinking_control_t *c, const uint32_t **ids, uint32_t *n);

/* src/thinking.rs:848-850 opens_thinking */
int32_t lily_opens_thinking(const char *prompt_tail, uint32_t len);

/* src/generate.rs FinishReason, as far as the helpers below produce it. */
enum lily_finish { LILY_FINISH_NONE = 0, LILY_FINISH_CALLBACK = 1, LILY_FINISH_LENGTH = 2 };
/* Delivers one token; returns 1 to go on, 0 to ask for a stop, < 0 on error. */
typedef int32_t (*lily_on_token_fn)(void *user, uint32_t token);

/*
 * src/generate.rs:121-142 push_group: appends `group` to tokens[0..*n) (room
 * for `cap`), each delivered to on_token; emitted whole even when the
 * callback asks to stop; only max_tokens cuts it short. *finish receives an
 * enum lily_finish. Returns 0, or nonzero on a callback error / lack of room.
 */
int32_t lily_push_group(uint32_t *tokens, uint64_t *n, uint64_t cap, const uint32_t *group,
                        uint64_t n_group, uint64_t max_tokens, lily_on_token_fn on_token,
                        void *user, int32_t *finish);
/* src/generate.rs:144-169 emit_acted: `action` must not be KEEP. */
int32_t lily_emit_acted(int32_t action, const uint32_t *group, uint64_t n_group, uint32_t drawn,
                        uint32_t *tokens, uint64_t *n, uint64_t cap, uint64_t max_tokens,
                        lily_on_token_fn on_token, void *user, int32_t *finish);

#ifdef __cplusplus
}
#endif
#endif /* LILY_THINKING_H */
