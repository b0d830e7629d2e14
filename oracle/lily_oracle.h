/*
 * CPU oracle for the token-sampling path. TEST INFRASTRUCTURE ONLY: nothing
 * that ships (the CUDA library, its host-side mirror) may include, link or
 * call this file; only the tests, the smoke check and the benchmark's CPU
 * baseline leg do, and only as the checker / the timed CPU baseline.
 *
 * It restates, in plain C, the reference's own CPU sampler code (paths are
 * relative to the reference project):
 *   tests/unit/kernels/sample.rs:8-54    cpu_sample
 *   tests/unit/kernels/sample.rs:251-260 cpu_kept
 *   tests/unit/kernels/sample.rs:264-283 cpu_spec
 *   src/kernels/sample.rs:47-55,83-94    is_greedy / uses_penalties / effective
 *   src/kernels/sample.rs:57-79          validate
 *   src/kernels/sample.rs:435-441        uniform_for
 *   src/kernels/sample.rs:220-222        draft_step
 *   src/kernels/metal/sample.metal:649-651 residual-draw domain and fallback
 *   src/kernels/metal/elementwise.metal:145-150 argmax tie rule
 *   src/kernels/metal/spec.metal:26-29   accepted count
 *
 * Parity status. The reference keeps no stored golden vectors for the
 * sampler (its tests draw inputs from an RNG crate that is not available
 * here); the restatement is pinned by the deterministic known-answer cases
 * of the reference's tests (greedy tie, penalty arithmetic, accept-count
 * table, uniform_for) which tests/test_oracle_pins.py replays. The logit
 * bias, the ban list and forced ids have no counterpart in the reference:
 * for those three features parity is unpinned and this file defines them.
 */
#ifndef LILY_ORACLE_H
#define LILY_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LO_K_CAP 1024u

enum {
    LO_OK = 0,
    LO_ERR_NAN = 1,        /* a NaN among the adjusted logits */
    LO_ERR_NONFINITE = 2,  /* the largest adjusted logit is not finite */
    LO_ERR_PARAMS = -1,    /* SamplingParams::validate failed */
    LO_ERR_ARG = -2
};

/* src/kernels/sample.rs:19-31 (top_k as u32, seed last, 40 bytes). */
typedef struct {
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
    uint32_t reserved;
    uint64_t seed;
} lo_params_t;

/* The exponential both sides use (see lily_oracle.c for the algorithm). */
float lo_expf(float x);

float lo_uniform_for(uint64_t seed, uint32_t step);
uint32_t lo_draft_step(uint32_t step);
uint32_t lo_residual_step(uint32_t step);

int lo_validate(const lo_params_t *p);
int lo_is_greedy(const lo_params_t *p);
int lo_uses_penalties(const lo_params_t *p);
/* effective(): greedy -> (1.0, 1); top_k 0 -> 1024; else min(top_k, 1024). */
void lo_effective(const lo_params_t *p, float *temperature, uint32_t *k);

/* counts[id] = multiplicity of id in history[0..n); ids >= vocab ignored. */
void lo_counts_from_history(const uint32_t *history, uint32_t n, uint32_t vocab,
                            uint32_t *counts);

/* bf16 bit patterns widened to f32 (exact). */
void lo_widen_bf16(const uint16_t *src, uint64_t n, float *dst);

/*
 * adjusted[i] = ((logit[i] + bias) penalised, banned -> -inf) / temperature.
 * counts may be NULL (no penalties applied). Returns LO_OK or LO_ERR_NAN.
 */
int lo_adjust(const float *logits, uint32_t vocab, const lo_params_t *p,
              const uint32_t *counts,
              const uint32_t *bias_ids, const float *bias_vals, uint32_t n_bias,
              const uint32_t *ban_ids, uint32_t n_ban,
              float *adjusted);

/*
 * One draw (cpu_sample + cpu_kept). `uniform` replaces uniform_for(seed,
 * step). kept_* hold LO_K_CAP entries: ids in rank order, w = exp(adj -
 * top), cum = sequential prefix of w, prob = w / cum[n_keep-1].
 * mode 0 = full sort (the faithful restatement), 1 = partial selection
 * (identical results, faster; the tests assert the identity).
 */
int lo_sample(const float *logits, uint32_t vocab, const lo_params_t *p,
              const uint32_t *counts,
              const uint32_t *bias_ids, const float *bias_vals, uint32_t n_bias,
              const uint32_t *ban_ids, uint32_t n_ban,
              float uniform, int mode,
              uint32_t *out_id,
              uint32_t *kept_ids, float *kept_w, float *kept_cum,
              float *kept_prob, uint32_t *n_keep,
              uint32_t *near_tie);

/* Exact argmax with the lowest index on ties; NaN never wins. */
uint32_t lo_argmax(const float *x, uint32_t n);

/*
 * Speculative draw for one row (cpu_spec + the kernel's no-residual-mass
 * fallback). The trunk's kept set is (p_ids, p_w, p_cum, n_p) as lo_sample
 * returns it. The draft distribution is dense (q_dense[vocab]) when
 * q_dense != NULL, else the sparse list (q_ids, q_probs, n_q).
 */
uint32_t lo_spec_draw(const uint32_t *p_ids, const float *p_w, const float *p_cum,
                      uint32_t n_p,
                      const float *q_dense,
                      const uint32_t *q_ids, const float *q_probs, uint32_t n_q,
                      uint32_t draft, float u_accept, float u_resid);

/*
 * One speculative verify step over m target rows. Rows j < m-1 check
 * draft_ids[j] against draft distribution j; the last row is a plain draw.
 * With penalties on, counts (may be NULL = all zero, then a scratch table
 * is used) see the earlier rows' draws, as the rows of the reference share
 * one histogram. out_accepted = leading rows with out_ids[j] ==
 * draft_ids[j]. A greedy sampler without penalties is the exact argmax on
 * every row. Returns the first non-OK row status.
 */
int lo_spec_verify(const float *target, uint32_t m, uint64_t ld, uint32_t vocab,
                   const lo_params_t *p, uint32_t *counts,
                   const uint32_t *draft_ids,
                   const float *q_dense, uint64_t q_ld,
                   const uint32_t *q_ids, const float *q_probs,
                   const uint32_t *q_n,
                   const float *u_accept, const float *u_resid,
                   uint32_t *out_ids, uint32_t *out_accepted);

/* a = 0; while a+1 < m && draws[a] == ids[a+1]: a++ */
uint32_t lo_spec_accept(const uint32_t *draws, const uint32_t *ids, uint32_t m);

/*
 * The 8-bit LM head of the vocab-sharded configuration:
 * logits[t, n] = sum_g scale[n, g] * sum_{c in group g} w[n, c] * h[t, c],
 * h widened from bf16, inner sums and the group sum in fp32 in index order.
 */
void lo_lmhead_int8(const uint16_t *hidden_bf16, uint32_t tokens, uint32_t hidden,
                    const int8_t *w, const uint16_t *scales_bf16, uint32_t group,
                    uint32_t n_begin, uint32_t n_end, float *logits, uint64_t ld);

/*
 * The head in the reference's own storage (MLX affine, src/weights.rs:21-36):
 * the dequantisation the reference's tests pin bit for bit against MLX
 * (tests/unit/kernels/quant.rs:39-63) and the fp32 product they compare
 * gemv_quant with (tests/unit/kernels/quant.rs:418-434).
 */
void lo_dequant_affine(const uint32_t *codes, const float *scales, const float *biases,
                       uint32_t rows, uint32_t cols, uint32_t group, uint32_t bits, float *out);
void lo_gemm_nt(const float *a, const float *b, uint32_t m, uint32_t k, uint32_t n, float *c);

#ifdef __cplusplus
}
#endif
#endif
