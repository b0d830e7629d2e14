/*
 * CPU oracle for the token-sampling path (see lily_oracle.h for what it
 * restates and for its parity status). TEST INFRASTRUCTURE ONLY.
 *
 * Build with -ffp-contract=off: every float operation below is one IEEE
 * binary32 operation, rounded to nearest even, exactly as written.
 */
#include "lily_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- bits -- */

static inline uint32_t f2u(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static inline float u2f(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* Monotone float -> uint key; its order is Rust's f32::total_cmp
 * (src/kernels/metal/sample.metal:29-32). */
static inline uint32_t sample_key(float v) {
    uint32_t u = f2u(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/* ----------------------------------------------------------------- exp -- */

/*
 * exp(x) in binary32. The reference calls Rust's f32::exp, the platform
 * libm, whose bits differ between platforms; the sampler under test and
 * this oracle instead both use the algorithm below, so that token ids can be
 * compared exactly. Its distance from glibc's expf is measured by the tests.
 *
 *   n = rint(x * log2(e))            by the 1.5*2^23 add/subtract trick
 *   r = x - n*ln2                    two-term Cody-Waite, with fused mul-add
 *   e^r = 1 + r + r^2 * P(r)         degree-5 polynomial (Cephes expf), fma
 *   result = e^r * 2^n               exact power-of-two scaling, in two steps
 *                                    where 2^n alone is not a normal float
 */
float lo_expf(float x) {
    if (x != x) {
        return x;
    }
    if (x > 88.72283935546875f) {
        return u2f(0x7F800000u);
    }
    if (x < -103.97208404541015625f) {
        return 0.0f;
    }
    const float log2e = 1.44269502162933349609375f;
    const float ln2_hi = 0.693145751953125f;
    const float ln2_lo = 1.428606765330187045037746429443359375e-06f;
    const float magic = 12582912.0f;
    float t = x * log2e;
    float nf = (t + magic) - magic;
    float r = fmaf(nf, -ln2_hi, x);
    r = fmaf(nf, -ln2_lo, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float z = r * r;
    float y = fmaf(p, z, r);
    y = y + 1.0f;
    int n = (int)nf;
    if (n > 127) {
        y = y * u2f(0x7F000000u); /* 2^127 */
        return y * u2f((uint32_t)(n - 127 + 127) << 23);
    }
    if (n < -126) {
        y = y * u2f((uint32_t)(n + 100 + 127) << 23);
        return y * u2f((uint32_t)(-100 + 127) << 23);
    }
    return y * u2f((uint32_t)(n + 127) << 23);
}

/* ------------------------------------------------------------ uniforms -- */

/* src/kernels/sample.rs:435-441 */
float lo_uniform_for(uint64_t seed, uint32_t step) {
    uint64_t z = seed + (uint64_t)step * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
}

/* src/kernels/sample.rs:220-222 */
uint32_t lo_draft_step(uint32_t step) {
    return step | 0x40000000u;
}

/* src/kernels/metal/sample.metal:649 */
uint32_t lo_residual_step(uint32_t step) {
    return step | 0x80000000u;
}

/* -------------------------------------------------------------- params -- */

/* src/kernels/sample.rs:57-79 */
int lo_validate(const lo_params_t *p) {
    if (!(isfinite(p->temperature) && p->temperature >= 0.0f)) {
        return LO_ERR_PARAMS;
    }
    if (!(isfinite(p->top_p) && p->top_p > 0.0f && p->top_p <= 1.0f)) {
        return LO_ERR_PARAMS;
    }
    if (!(isfinite(p->min_p) && p->min_p >= 0.0f && p->min_p <= 1.0f)) {
        return LO_ERR_PARAMS;
    }
    if (!(isfinite(p->repetition_penalty) && p->repetition_penalty > 0.0f)) {
        return LO_ERR_PARAMS;
    }
    if (!(isfinite(p->presence_penalty) && isfinite(p->frequency_penalty))) {
        return LO_ERR_PARAMS;
    }
    return LO_OK;
}

/* src/kernels/sample.rs:47-49 */
int lo_is_greedy(const lo_params_t *p) {
    return p->temperature <= 0.0f || p->top_k == 1u;
}

/* src/kernels/sample.rs:51-55 */
int lo_uses_penalties(const lo_params_t *p) {
    return p->presence_penalty != 0.0f || p->frequency_penalty != 0.0f ||
           p->repetition_penalty != 1.0f;
}

/* src/kernels/sample.rs:83-94 */
void lo_effective(const lo_params_t *p, float *temperature, uint32_t *k) {
    if (lo_is_greedy(p)) {
        *temperature = 1.0f;
        *k = 1u;
    } else {
        *temperature = p->temperature;
        *k = p->top_k == 0u ? LO_K_CAP : (p->top_k < LO_K_CAP ? p->top_k : LO_K_CAP);
    }
}

void lo_counts_from_history(const uint32_t *history, uint32_t n, uint32_t vocab,
                            uint32_t *counts) {
    memset(counts, 0, (size_t)vocab * sizeof(uint32_t));
    for (uint32_t i = 0; i < n; ++i) {
        if (history[i] < vocab) {
            counts[history[i]] += 1u;
        }
    }
}

void lo_widen_bf16(const uint16_t *src, uint64_t n, float *dst) {
    for (uint64_t i = 0; i < n; ++i) {
        dst[i] = u2f((uint32_t)src[i] << 16);
    }
}

/* -------------------------------------------------------------- adjust -- */

/*
 * tests/unit/kernels/sample.rs:15-30, with the three extensions in front of
 * and behind the penalties: bias entries add in list order (duplicates add),
 * then the penalties, then banned ids drop to -inf, then the division by the
 * temperature. Out-of-range bias / ban ids are ignored.
 */
int lo_adjust(const float *logits, uint32_t vocab, const lo_params_t *p,
              const uint32_t *counts,
              const uint32_t *bias_ids, const float *bias_vals, uint32_t n_bias,
              const uint32_t *ban_ids, uint32_t n_ban,
              float *adjusted) {
    float temperature;
    uint32_t k;
    lo_effective(p, &temperature, &k);
    const int pen = lo_uses_penalties(p) && counts != NULL;
    memcpy(adjusted, logits, (size_t)vocab * sizeof(float));
    for (uint32_t j = 0; j < n_bias; ++j) {
        if (bias_ids[j] < vocab) {
            adjusted[bias_ids[j]] = adjusted[bias_ids[j]] + bias_vals[j];
        }
    }
    int status = LO_OK;
    for (uint32_t i = 0; i < vocab; ++i) {
        float l = adjusted[i];
        if (pen && counts[i] > 0u) {
            l = l > 0.0f ? l / p->repetition_penalty : l * p->repetition_penalty;
            float f = p->frequency_penalty * (float)counts[i];
            float s = p->presence_penalty + f;
            l = l - s;
        }
        adjusted[i] = l;
    }
    for (uint32_t j = 0; j < n_ban; ++j) {
        if (ban_ids[j] < vocab) {
            adjusted[ban_ids[j]] = u2f(0xFF800000u);
        }
    }
    for (uint32_t i = 0; i < vocab; ++i) {
        float q = adjusted[i] / temperature;
        if (q != q) {
            status = LO_ERR_NAN;
        }
        adjusted[i] = q;
    }
    return status;
}

/* -------------------------------------------------------------- select -- */

static int cmp_u64_desc(const void *a, const void *b) {
    uint64_t x = *(const uint64_t *)a, y = *(const uint64_t *)b;
    return x < y ? 1 : (x > y ? -1 : 0);
}

/* Moves the k largest of a[0..n) to a[0..k) (any order); three-way
 * partition around a median-of-three pivot. */
static void select_top(uint64_t *a, uint32_t n, uint32_t k) {
    uint32_t lo = 0, hi = n;
    while (hi - lo > 1u && lo < k && k < hi) {
        uint64_t x = a[lo], y = a[lo + (hi - lo) / 2u], z = a[hi - 1u];
        uint64_t pivot = x > y ? (y > z ? y : (x > z ? z : x))
                               : (x > z ? x : (y > z ? z : y));
        uint32_t gt = lo, i = lo, lt = hi;
        while (i < lt) {
            if (a[i] > pivot) {
                uint64_t t = a[gt];
                a[gt] = a[i];
                a[i] = t;
                ++gt;
                ++i;
            } else if (a[i] < pivot) {
                --lt;
                uint64_t t = a[lt];
                a[lt] = a[i];
                a[i] = t;
            } else {
                ++i;
            }
        }
        /* a[lo..gt) > pivot, a[gt..lt) == pivot, a[lt..hi) < pivot */
        if (k <= gt) {
            hi = gt;
        } else if (k <= lt) {
            return;
        } else {
            lo = lt;
        }
    }
}

/*
 * tests/unit/kernels/sample.rs:31-53 on already adjusted logits: candidates
 * = the first k of the order (value descending by total_cmp, id ascending),
 * w = exp(adj - top), total and the keep loop's running sum both sequential
 * in rank order.
 */
static int sample_adjusted(const float *adjusted, uint32_t vocab, uint32_t k,
                           float top_p, float min_p, float uniform, int mode,
                           uint32_t *out_id, uint32_t *kept_ids, float *kept_w,
                           float *kept_cum, float *kept_prob, uint32_t *n_keep_out,
                           uint32_t *near_tie) {
    uint64_t *order = (uint64_t *)malloc((size_t)vocab * sizeof(uint64_t));
    if (order == NULL) {
        return LO_ERR_ARG;
    }
    for (uint32_t i = 0; i < vocab; ++i) {
        order[i] = ((uint64_t)sample_key(adjusted[i]) << 32) | (uint64_t)(0xFFFFFFFFu - i);
    }
    if (k > vocab) {
        k = vocab;
    }
    if (k == 0u) {
        free(order);
        return LO_ERR_ARG;
    }
    uint32_t tie = 0;
    if (mode == 0) {
        qsort(order, vocab, sizeof(uint64_t), cmp_u64_desc);
    } else {
        select_top(order, vocab, k);
        qsort(order, k, sizeof(uint64_t), cmp_u64_desc);
    }
    uint32_t ids[LO_K_CAP];
    float w[LO_K_CAP];
    for (uint32_t i = 0; i < k; ++i) {
        ids[i] = 0xFFFFFFFFu - (uint32_t)(order[i] & 0xFFFFFFFFu);
    }
    if (k < vocab) {
        uint64_t best = 0;
        for (uint32_t i = k; i < vocab; ++i) {
            best = order[i] > best ? order[i] : best;
            if (mode == 0) {
                break;
            }
        }
        uint32_t next = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu);
        float a = adjusted[ids[k - 1u]], b = adjusted[next];
        float big = fabsf(a) > fabsf(b) ? fabsf(a) : fabsf(b);
        if (fabsf(a - b) <= 1e-6f * big) {
            tie |= 1u;
        }
    }
    free(order);
    const float top = adjusted[ids[0]];
    if (!isfinite(top)) {
        return top != top ? LO_ERR_NAN : LO_ERR_NONFINITE;
    }
    float total = 0.0f;
    for (uint32_t i = 0; i < k; ++i) {
        w[i] = lo_expf(adjusted[ids[i]] - top);
        total = total + w[i];
    }
    const float limit = top_p * total;
    float cum = 0.0f;
    uint32_t n_keep = 0;
    for (uint32_t rank = 0; rank < k; ++rank) {
        if (rank > 0u) {
            if (fabsf(cum - limit) <= 1e-6f * limit ||
                (min_p > 0.0f && fabsf(w[rank] - min_p) <= 1e-6f * min_p)) {
                tie |= 2u;
            }
            if (!(cum < limit && w[rank] >= min_p)) {
                break;
            }
        }
        cum = cum + w[rank];
        kept_ids[n_keep] = ids[rank];
        kept_w[n_keep] = w[rank];
        kept_cum[n_keep] = cum;
        ++n_keep;
    }
    const float mass = kept_cum[n_keep - 1u];
    for (uint32_t i = 0; i < n_keep; ++i) {
        kept_prob[i] = kept_w[i] / mass;
    }
    const float target = uniform * mass;
    uint32_t chosen = n_keep - 1u;
    for (uint32_t i = 0; i < n_keep; ++i) {
        if (target < kept_cum[i]) {
            chosen = i;
            break;
        }
    }
    for (uint32_t i = 0; i < n_keep; ++i) {
        if (fabsf(target - kept_cum[i]) <= 1e-6f * kept_cum[i]) {
            tie |= 4u;
        }
    }
    *out_id = kept_ids[chosen];
    *n_keep_out = n_keep;
    if (near_tie != NULL) {
        *near_tie = tie;
    }
    return LO_OK;
}

int lo_sample(const float *logits, uint32_t vocab, const lo_params_t *p,
              const uint32_t *counts,
              const uint32_t *bias_ids, const float *bias_vals, uint32_t n_bias,
              const uint32_t *ban_ids, uint32_t n_ban,
              float uniform, int mode,
              uint32_t *out_id,
              uint32_t *kept_ids, float *kept_w, float *kept_cum,
              float *kept_prob, uint32_t *n_keep,
              uint32_t *near_tie) {
    if (vocab == 0u) {
        return LO_ERR_ARG;
    }
    if (lo_validate(p) != LO_OK) {
        return LO_ERR_PARAMS;
    }
    if (lo_is_greedy(p) && !lo_uses_penalties(p) && n_bias == 0u && n_ban == 0u) {
        /* src/kernels/sample.rs:382-385: not a sampled draw, the exact argmax. */
        *out_id = lo_argmax(logits, vocab);
        kept_ids[0] = *out_id;
        kept_w[0] = 1.0f;
        kept_cum[0] = 1.0f;
        kept_prob[0] = 1.0f;
        *n_keep = 1u;
        if (near_tie != NULL) {
            *near_tie = 0u;
        }
        return LO_OK;
    }
    float *adjusted = (float *)malloc((size_t)vocab * sizeof(float));
    if (adjusted == NULL) {
        return LO_ERR_ARG;
    }
    int status = lo_adjust(logits, vocab, p, counts, bias_ids, bias_vals, n_bias,
                           ban_ids, n_ban, adjusted);
    if (status == LO_OK) {
        float temperature;
        uint32_t k;
        lo_effective(p, &temperature, &k);
        status = sample_adjusted(adjusted, vocab, k, p->top_p, p->min_p, uniform, mode,
                                 out_id, kept_ids, kept_w, kept_cum, kept_prob, n_keep,
                                 near_tie);
    }
    free(adjusted);
    return status;
}

/* src/kernels/metal/elementwise.metal:145-150 */
uint32_t lo_argmax(const float *x, uint32_t n) {
    float bv = u2f(0xFF800000u);
    uint32_t bi = 0;
    for (uint32_t i = 0; i < n; ++i) {
        if (x[i] > bv || (x[i] == bv && i < bi)) {
            bv = x[i];
            bi = i;
        }
    }
    return bi;
}

/* ---------------------------------------------------------------- spec -- */

static float q_at(const float *q_dense, const uint32_t *q_ids, const float *q_probs,
                  uint32_t n_q, uint32_t id) {
    if (q_dense != NULL) {
        return q_dense[id];
    }
    for (uint32_t j = 0; j < n_q; ++j) {
        if (q_ids[j] == id) {
            return q_probs[j];
        }
    }
    return 0.0f;
}

/*
 * tests/unit/kernels/sample.rs:264-283, on the probabilities p_i = w_i /
 * mass, plus src/kernels/metal/sample.metal:650-651: a residual without
 * mass falls back to a plain draw from p on the second uniform.
 */
uint32_t lo_spec_draw(const uint32_t *p_ids, const float *p_w, const float *p_cum,
                      uint32_t n_p,
                      const float *q_dense,
                      const uint32_t *q_ids, const float *q_probs, uint32_t n_q,
                      uint32_t draft, float u_accept, float u_resid) {
    const float mass = p_cum[n_p - 1u];
    float p_d = 0.0f;
    for (uint32_t i = 0; i < n_p; ++i) {
        if (p_ids[i] == draft) {
            p_d = p_w[i] / mass;
            break;
        }
    }
    const float q_d = q_at(q_dense, q_ids, q_probs, n_q, draft);
    if (u_accept * q_d < p_d) {
        return draft;
    }
    float r[LO_K_CAP];
    float total = 0.0f;
    for (uint32_t i = 0; i < n_p; ++i) {
        float x = p_w[i] / mass - q_at(q_dense, q_ids, q_probs, n_q, p_ids[i]);
        r[i] = x > 0.0f ? x : 0.0f;
        total = total + r[i];
    }
    if (total > 0.0f) {
        const float target = u_resid * total;
        float cum = 0.0f;
        for (uint32_t i = 0; i < n_p; ++i) {
            cum = cum + r[i];
            if (target < cum) {
                return p_ids[i];
            }
        }
        return p_ids[n_p - 1u];
    }
    const float target = u_resid * mass;
    for (uint32_t i = 0; i < n_p; ++i) {
        if (target < p_cum[i]) {
            return p_ids[i];
        }
    }
    return p_ids[n_p - 1u];
}

/* src/kernels/metal/spec.metal:26-29 */
uint32_t lo_spec_accept(const uint32_t *draws, const uint32_t *ids, uint32_t m) {
    uint32_t a = 0;
    while (a + 1u < m && draws[a] == ids[a + 1u]) {
        ++a;
    }
    return a;
}

/*
 * src/qwen4exp/model.rs:3013-3040: row j draws with the request's sampler
 * (penalties included, counts shared and updated row by row); rows before
 * the last are speculative draws against proposal j.
 */
int lo_spec_verify(const float *target, uint32_t m, uint64_t ld, uint32_t vocab,
                   const lo_params_t *p, uint32_t *counts,
                   const uint32_t *draft_ids,
                   const float *q_dense, uint64_t q_ld,
                   const uint32_t *q_ids, const float *q_probs,
                   const uint32_t *q_n,
                   const float *u_accept, const float *u_resid,
                   uint32_t *out_ids, uint32_t *out_accepted) {
    if (m == 0u || lo_validate(p) != LO_OK) {
        return LO_ERR_PARAMS;
    }
    const int pen = lo_uses_penalties(p);
    uint32_t *own = NULL;
    if (pen && counts == NULL) {
        own = (uint32_t *)calloc(vocab, sizeof(uint32_t));
        counts = own;
    }
    uint32_t kept_ids[LO_K_CAP];
    float kept_w[LO_K_CAP], kept_cum[LO_K_CAP], kept_prob[LO_K_CAP];
    int status = LO_OK;
    for (uint32_t j = 0; j < m; ++j) {
        const float *row = target + (uint64_t)j * ld;
        uint32_t out;
        if (lo_is_greedy(p) && !pen) {
            out = lo_argmax(row, vocab);
        } else {
            uint32_t n_keep = 0, chosen = 0;
            int s = lo_sample(row, vocab, p, pen ? counts : NULL, NULL, NULL, 0, NULL, 0,
                              u_accept[j], 1, &chosen, kept_ids, kept_w, kept_cum,
                              kept_prob, &n_keep, NULL);
            if (s != LO_OK) {
                status = status == LO_OK ? s : status;
                out_ids[j] = 0xFFFFFFFFu;
                continue;
            }
            if (j + 1u < m) {
                out = lo_spec_draw(kept_ids, kept_w, kept_cum, n_keep,
                                   q_dense ? q_dense + (uint64_t)j * q_ld : NULL,
                                   q_ids ? q_ids + (uint64_t)j * LO_K_CAP : NULL,
                                   q_probs ? q_probs + (uint64_t)j * LO_K_CAP : NULL,
                                   q_n ? q_n[j] : 0u, draft_ids[j], u_accept[j],
                                   u_resid[j]);
            } else {
                out = chosen;
            }
        }
        out_ids[j] = out;
        if (pen && out < vocab) {
            counts[out] += 1u;
        }
    }
    uint32_t a = 0;
    while (a + 1u < m && out_ids[a] == draft_ids[a]) {
        ++a;
    }
    *out_accepted = a;
    free(own);
    return status;
}

/* ------------------------------------------------------------- LM head -- */

void lo_lmhead_int8(const uint16_t *hidden_bf16, uint32_t tokens, uint32_t hidden,
                    const int8_t *w, const uint16_t *scales_bf16, uint32_t group,
                    uint32_t n_begin, uint32_t n_end, float *logits, uint64_t ld) {
    const uint32_t groups = hidden / group;
    for (uint32_t t = 0; t < tokens; ++t) {
        const uint16_t *h = hidden_bf16 + (uint64_t)t * hidden;
        for (uint32_t n = n_begin; n < n_end; ++n) {
            const int8_t *wr = w + (uint64_t)n * hidden;
            float acc = 0.0f;
            for (uint32_t g = 0; g < groups; ++g) {
                float part = 0.0f;
                for (uint32_t c = g * group; c < (g + 1u) * group; ++c) {
                    part = part + (float)wr[c] * u2f((uint32_t)h[c] << 16);
                }
                float s = u2f((uint32_t)scales_bf16[(uint64_t)n * groups + g] << 16);
                acc = acc + s * part;
            }
            logits[(uint64_t)t * ld + n] = acc;
        }
    }
}

/* ---------------------------------------------- MLX affine 4/8-bit head -- */

/* tests/support/cpu_ref.rs:402-430 dequant_affine: element c of row r is bits
 * bits*(c % per_word) of codes[r][c / per_word], low element first;
 * w = scale * q + bias, two roundings. */
void lo_dequant_affine(const uint32_t *codes, const float *scales, const float *biases,
                       uint32_t rows, uint32_t cols, uint32_t group, uint32_t bits, float *out) {
    const uint32_t per_word = 32u / bits;
    const uint32_t mask = (1u << bits) - 1u;
    const uint32_t words = cols / per_word, groups = cols / group;
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t c = 0; c < cols; ++c) {
            const uint32_t word = codes[(uint64_t)r * words + c / per_word];
            const uint32_t q = (word >> (bits * (c % per_word))) & mask;
            const uint64_t g = (uint64_t)r * groups + c / group;
            const float scaled = scales[g] * (float)q;
            out[(uint64_t)r * cols + c] = scaled + biases[g];
        }
    }
}

/* tests/support/cpu_ref.rs:50-62 gemm_nt: c[m, n] = sum_i a[m, i] * b[n, i],
 * one fp32 accumulator in index order. */
void lo_gemm_nt(const float *a, const float *b, uint32_t m, uint32_t k, uint32_t n, float *c) {
    for (uint32_t row = 0; row < m; ++row) {
        for (uint32_t col = 0; col < n; ++col) {
            float sum = 0.0f;
            for (uint32_t i = 0; i < k; ++i) {
                const float prod = a[(uint64_t)row * k + i] * b[(uint64_t)col * k + i];
                sum = sum + prod;
            }
            c[(uint64_t)row * n + col] = sum;
        }
    }
}
