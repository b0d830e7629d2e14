// Host side of the CPU stand-in for the reference's Metal sampler: the
// dispatches that src/kernels/sample.rs:250-372 (encode_draw) encodes, made as
// plain calls of the shader's entry points, one threadgroup after another.
// Appended to the shader's translation unit by the build recipe, so the entry
// points (static functions there) are in scope. TEST INFRASTRUCTURE.
//
// Mirrors, and cites:
//   effective()        src/kernels/sample.rs:83-95   greedy -> (T = 1, k = 1); k capped at 1024
//   samples()          src/kernels/sample.rs:238-240 an exact argmax otherwise (another shader;
//                                                    refused here with status 2)
//   prepare dispatch   src/kernels/sample.rs:266-286 64 threadgroups x 256 threads
//   two-phase rule     src/kernels/sample.rs:289-291 k <= 64 and V > 4 * groups * k
//   local top-k        src/kernels/sample.rs:292-305 `groups` threadgroups x 1024 threads
//   the draw           src/kernels/sample.rs:306-371 1 threadgroup x 1024 threads; seed split
//                                                    into its low and high words
#pragma once

namespace metal_shim {

enum Mode : int { MODE_PLAIN = 0, MODE_DRAFT = 1, MODE_SPEC = 2 };

struct Ids {
    uint32_t tid, sg, lane;
    explicit Ids(uint32_t t) : tid(t), sg(t / SIMD_WIDTH), lane(t % SIMD_WIDTH) {}
};

}  // namespace metal_shim

// Status: 0 a draw was made; 1 bad argument; 2 the parameters take the
// reference's exact-argmax route, which this shader does not serve; 3 the
// emulated threads deadlocked at a barrier.
extern "C" int lily_metal_shim_draw(const float* logits, uint32_t vocab, uint32_t* counts,
                                    float temperature, uint32_t top_k, float top_p, float min_p,
                                    float presence, float frequency, float repetition,
                                    uint64_t seed, uint32_t step, int two_phase_on,
                                    uint32_t local_groups, int mode, uint32_t* q_ids,
                                    float* q_probs, uint32_t* q_n, const uint32_t* draft,
                                    uint32_t* out, float* adjusted_out, int* used_two_phase) {
    using namespace metal_shim;
    if (!logits || !counts || !out || vocab == 0 || local_groups == 0 || local_groups > 256) {
        return 1;
    }
    if (mode != MODE_PLAIN && (!q_ids || !q_probs || !q_n)) {
        return 1;
    }
    if (mode == MODE_SPEC && !draft) {
        return 1;
    }
    const bool greedy = temperature <= 0.0f || top_k == 1;
    const bool penalties = presence != 0.0f || frequency != 0.0f || repetition != 1.0f;
    if (greedy && !penalties) {
        return 2;
    }
    const float t_eff = greedy ? 1.0f : temperature;
    const uint32_t k_eff = greedy ? 1u : (top_k == 0 ? uint32_t(SAMPLE_K_CAP)
                                                     : metal::min(top_k, uint32_t(SAMPLE_K_CAP)));
    const uint32_t use_penalties = penalties ? 1u : 0u;

    static std::vector<float> adjusted;
    static std::vector<uint32_t> local_ids(256 * SAMPLE_LOCAL_K_MAX);
    float maxima[SAMPLE_PREP_GROUPS];
    adjusted.assign(vocab, 0.0f);

    for (uint32_t g = 0; g < SAMPLE_PREP_GROUPS; ++g) {
        const bool ok = run_threadgroup(SAMPLE_PREP_TG, [&](uint32_t t) {
            const Ids i(t);
            sample_prepare_f32(logits, adjusted.data(), counts, maxima, t_eff, presence, frequency,
                               repetition, vocab, use_penalties, g, i.tid, i.sg, i.lane);
        });
        if (!ok) {
            return 3;
        }
    }
    if (adjusted_out) {
        std::memcpy(adjusted_out, adjusted.data(), size_t(vocab) * sizeof(float));
    }

    const bool two_phase = k_eff <= SAMPLE_LOCAL_K_MAX
        && uint64_t(vocab) > 4ull * local_groups * k_eff && two_phase_on != 0;
    if (used_two_phase) {
        *used_two_phase = two_phase ? 1 : 0;
    }
    uint32_t select_v = vocab;
    uint32_t mapped = 0;
    if (two_phase) {
        for (uint32_t g = 0; g < local_groups; ++g) {
            const bool ok = run_threadgroup(SAMPLE_TG, [&](uint32_t t) {
                const Ids i(t);
                sample_local_topk_f32(adjusted.data(), maxima, local_ids.data(), k_eff, vocab,
                                      local_groups, g, i.tid, i.sg, i.lane);
            });
            if (!ok) {
                return 3;
            }
        }
        select_v = local_groups * k_eff;
        mapped = 1;
    }

    const uint32_t seed_lo = uint32_t(seed & 0xffffffffull);
    const uint32_t seed_hi = uint32_t(seed >> 32);
    const bool ok = run_threadgroup(SAMPLE_TG, [&](uint32_t t) {
        const Ids i(t);
        if (mode == MODE_PLAIN) {
            sample_f32(adjusted.data(), maxima, counts, out, local_ids.data(), top_p, min_p, k_eff,
                       select_v, seed_lo, seed_hi, step, use_penalties, mapped, i.tid, i.sg,
                       i.lane);
        } else if (mode == MODE_DRAFT) {
            sample_draft_f32(adjusted.data(), maxima, counts, out, q_ids, q_probs, q_n,
                             local_ids.data(), top_p, min_p, k_eff, select_v, seed_lo, seed_hi,
                             step, use_penalties, mapped, i.tid, i.sg, i.lane);
        } else {
            sample_spec_f32(adjusted.data(), maxima, counts, out, q_ids, q_probs, q_n, draft,
                            local_ids.data(), top_p, min_p, k_eff, select_v, seed_lo, seed_hi, step,
                            use_penalties, mapped, i.tid, i.sg, i.lane);
        }
    });
    return ok ? 0 : 3;
}

// The shader's uniform for (seed, step), src/kernels/metal/sample.metal:93-101.
extern "C" float lily_metal_shim_uniform(uint64_t seed, uint32_t step) {
    return sample_uniform(uint32_t(seed & 0xffffffffull), uint32_t(seed >> 32), step);
}
