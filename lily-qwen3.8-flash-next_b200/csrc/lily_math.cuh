// Device arithmetic of the sampler. Every float operation that reaches a
// token decision is written with an explicit round-to-nearest intrinsic so
// that the compiler can neither contract it into an fma nor reassociate it:
// the results have to match a sequential binary32 evaluation bit for bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lily {

// Monotone float -> uint key whose unsigned order is the total order of the
// floats (-NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN): the order Rust's
// f32::total_cmp gives the reference's CPU sampler and the key the
// reference's shader sorts by (src/kernels/metal/sample.metal:29-32).
__device__ __forceinline__ uint32_t key_of(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float float_of_key(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) {
    return __uint_as_float(packed << 16);
}

__device__ __forceinline__ float bf16_hi(uint32_t packed) {
    return __uint_as_float(packed & 0xFFFF0000u);
}

// max that returns NaN when either operand is NaN, on two packed bf16.
__device__ __forceinline__ uint32_t max_nan_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ float max_nan_f32(float a, float b) {
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// exp(x) in binary32: n = rint(x*log2 e) by the 1.5*2^23 trick, two-term
// Cody-Waite reduction with fma, the degree-5 Cephes polynomial with fma,
// exact power-of-two scaling (two steps outside the normal range). Within
// 1 ulp of the correctly rounded value; what matters is that the CPU
// checker evaluates the same operations in the same order.
__device__ __forceinline__ float exp_f32(float x) {
    if (x != x) {
        return x;
    }
    if (x > 88.72283935546875f) {
        return __uint_as_float(0x7F800000u);
    }
    if (x < -103.97208404541015625f) {
        return 0.0f;
    }
    const float log2e = 1.44269502162933349609375f;
    const float ln2_hi = 0.693145751953125f;
    const float ln2_lo = 1.428606765330187045037746429443359375e-06f;
    const float magic = 12582912.0f;
    const float t = __fmul_rn(x, log2e);
    const float nf = __fsub_rn(__fadd_rn(t, magic), magic);
    float r = __fmaf_rn(nf, -ln2_hi, x);
    r = __fmaf_rn(nf, -ln2_lo, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    const float z = __fmul_rn(r, r);
    float y = __fmaf_rn(p, z, r);
    y = __fadd_rn(y, 1.0f);
    const int n = (int)nf;
    if (n > 127) {
        y = __fmul_rn(y, __uint_as_float(0x7F000000u));
        return __fmul_rn(y, __uint_as_float((uint32_t)(n - 127 + 127) << 23));
    }
    if (n < -126) {
        y = __fmul_rn(y, __uint_as_float((uint32_t)(n + 100 + 127) << 23));
        return __fmul_rn(y, __uint_as_float((uint32_t)(-100 + 127) << 23));
    }
    return __fmul_rn(y, __uint_as_float((uint32_t)(n + 127) << 23));
}

// src/kernels/sample.rs:435-441 / src/kernels/metal/sample.metal:93-101.
__host__ __device__ __forceinline__ float uniform_for(uint64_t seed, uint32_t step) {
    uint64_t z = seed + (uint64_t)step * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
}

}  // namespace lily
