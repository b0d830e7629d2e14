// The 8-bit LM head that feeds the sampler: logits[t, n] = sum over column
// groups g of scale[n, g] * (sum over the group's 64 columns of w[n, c] * h[t, c]),
// w int8 (symmetric), scale bf16 per 64 columns, h bf16, everything summed in
// binary32. It stands where the reference projects the hidden state through
// its quantised head before sampling (gemv_quant, src/kernels/quant.rs:141-175,
// called from src/qwen4exp/model.rs:2999-3006); the reference's format is
// affine 4/8-bit, this one is the symmetric int8 layout of the vocab-sharded
// configuration, so parity here is by tolerance against a binary32 CPU sum.
// The same kernel (VARIANT bit 5) takes the reference's own 8-bit storage, MLX
// affine (src/weights.rs:21-36; gemv_q8, src/kernels/metal/quant.metal:
// 124-160): w = scale * q + bias with q an unsigned byte. The converters widen
// q - 128 (again exact in bf16, and for the same three instructions); the
// term that leaves out, (128 * scale + bias) * (sum of the group's 64 hidden
// values) summed over the groups, is written to the output by a small kernel
// that runs first (affine_bias_term_kernel); the epilogue's sums start from it.
//
// sm_100a only. The weights are the only large operand (1 byte per
// multiply-add), so the kernel is a stream of them through the tensor cores,
// one persistent block per SM, warps specialised:
//
//   * a tile is 256 vocabulary rows. One thread asks the copy engine (TMA,
//     128-byte swizzle) for 256 rows x 128 bytes of int8 per stage, four
//     stages deep, and for each group's 64 x 64 slice of the hidden states,
//     which lands in the swizzled K-major layout the multiplier's B operand
//     descriptor names;
//   * eight warps own one tile row per thread: per 64-column group a thread
//     widens its row's 64 bytes to bf16 exactly (every int8 is a bf16) and
//     stores them with tcgen05.st into TENSOR MEMORY, where the multiplier
//     reads its A operand (lane = row, two bf16 per column): the widened
//     weights never touch shared memory;
//   * two threads (one per 128 rows) issue, per group, 4 tcgen05.mma each
//     (M = 128 rows, N = 64 tokens, K = 16) into a TMEM accumulator that
//     starts from zero: products of two bf16 are exact in binary32, so only
//     the order of the 64 adds differs from a sequential sum. One commit per
//     thread and group completes the group's "done" barrier, which frees the
//     group's operand slots and hands its sums to the epilogue;
//   * sixteen warps read each group's sums back with tcgen05.ld, multiply by
//     the row's scale of that group and add into registers: the group sums
//     cannot stay in TMEM across groups because each has its own scale;
//   * after the last group the tile's 256 x 64 logits go to global memory.
//
// Tensor memory: 3 accumulators of 128 columns, 2 operand slots of 64.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out sets an
// abort word, after which no wait blocks any more: the block runs to its end
// (results are garbage, TMEM is freed) and the status word tells the host.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lily_head {

constexpr int TILE_ROWS = 256;   // two M = 128 accumulators
constexpr int TOK = 64;          // MMA N: the most hidden rows per launch
constexpr int GROUP_K = 64;      // columns per scale group = one 128-byte bf16 atom
constexpr int RAW_GROUPS = 2;    // groups per stage of int8 bytes
constexpr int RAW_STAGES = 4;
constexpr int H_SLOTS = 8;       // hidden slices in shared memory: as many groups as the stages hold
static_assert(H_SLOTS == 8, "the hidden ring and the done ring share their indexing");
constexpr int A_SLOTS = 2;       // bf16 weight tiles in tensor memory
constexpr int ACC_BUFS = 3;      // accumulators in tensor memory
constexpr uint32_t RAW_STAGE_BYTES = TILE_ROWS * GROUP_K * RAW_GROUPS;  // 32 KB
constexpr uint32_t H_BYTES = TOK * 128;                                 // 8 KB
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 128;           // two row halves x 64 tokens, binary32
constexpr uint32_t A_COLS = 64;              // two row halves x 64 bf16 = 32 columns each
constexpr uint32_t A_COL0 = ACC_BUFS * ACC_COLS;
static_assert(A_COL0 + A_SLOTS * A_COLS <= TMEM_COLS, "tensor memory columns");

constexpr int WARP_MMA = 0;
constexpr int WARP_LOAD = 1;
constexpr int WARP_CONV0 = 2;
constexpr int N_CONV_WARPS = 8;
constexpr int WARP_EPI0 = WARP_CONV0 + N_CONV_WARPS;
constexpr int N_EPI_WARPS = 16;  // a row's 64 tokens are split between two warps
constexpr int WARP_MMA1 = WARP_EPI0 + N_EPI_WARPS;  // issues the multiplies of rows 128..255
constexpr int THREADS = 32 * (WARP_MMA1 + 1);  // 864 (registers are granted as for 896)
constexpr int DONE_SLOTS = 8;    // ring of "group q has been multiplied" barriers
constexpr int CONV_THREADS = 32 * N_CONV_WARPS;
constexpr int EPI_THREADS = 32 * N_EPI_WARPS;
static_assert(CONV_THREADS == TILE_ROWS && EPI_THREADS == 2 * TILE_ROWS, "threads per tile row");
static_assert(WARP_CONV0 % 2 == 0 && WARP_EPI0 % 2 == 0, "warp % 4 must cover all four lane quarters");

constexpr uint32_t STATUS_TIMEOUT_BIT = 30;  // bit of the handle's status word

struct Smem {
    // Offsets from a 1024-byte aligned base.
    static constexpr uint32_t HID = 0;
    static constexpr uint32_t RAW = HID + H_SLOTS * H_BYTES;
    static constexpr uint32_t BARS = RAW + RAW_STAGES * RAW_STAGE_BYTES;
    static constexpr uint32_t RAW_FULL = BARS;                      // [RAW_STAGES]
    static constexpr uint32_t RAW_EMPTY = RAW_FULL + 8 * RAW_STAGES;  // [RAW_STAGES]
    static constexpr uint32_t A_FULL = RAW_EMPTY + 8 * RAW_STAGES;  // [A_SLOTS]
    static constexpr uint32_t H_FULL = A_FULL + 8 * A_SLOTS;        // [H_SLOTS]
    // DONE[q % 8] completes when both halves of group q have been multiplied:
    // one commit per issuing thread tells the converters (slot of q free for
    // q + 2), the loader (slot free for q + 8) and the epilogue (sums ready).
    static constexpr uint32_t DONE = H_FULL + 8 * H_SLOTS;          // [DONE_SLOTS]
    static constexpr uint32_t ACC_EMPTY = DONE + 8 * DONE_SLOTS;    // [ACC_BUFS]
    static constexpr uint32_t FINAL = ACC_EMPTY + 8 * ACC_BUFS;     // [2] an issuing thread's last commit
    static constexpr uint32_t TMEM_ADDR = FINAL + 8 * 2;
    static constexpr uint32_t ABORT = TMEM_ADDR + 4;
    static constexpr uint32_t END = ABORT + 4;
    static constexpr uint32_t BYTES = END + 1024;  // room to align the base
};
static_assert(Smem::BYTES <= 227 * 1024, "shared memory of one block");

struct Args {
    // Tiled copies (TMA), both with the 128-byte swizzle: the weights as uint8
    // [rows, k] in boxes of 256 rows x 128 bytes, the hidden states as bf16
    // [tokens, k] in boxes of 64 rows x 64 columns. Rows past the end read 0.
    CUtensorMap w_map;
    CUtensorMap h_map;
    const __nv_bfloat16 *scales;  // [rows, hidden / 64]
    uint32_t tokens;            // <= 64
    uint32_t k;                 // hidden size, a multiple of 512
    uint32_t rows;              // vocabulary rows of this shard
    float *out;                 // [tokens, ldo]
    uint64_t ldo;
    uint32_t *status_word;
    uint64_t wait_ns;           // the bound of every wait inside the kernel
    // Test hook: block 0 does not ask for the weights of this stage (~0: none),
    // so that the wait of their consumers runs out.
    uint32_t lost_stage;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity to complete, for at most
// `limit_ns`; once any wait of the block has run out, none blocks any more.
// Returns true if it gave up (this wait ran out, or another had): the caller
// then leaves its loop. A phase that is complete at the first look returns
// false without reading the abort word, so the path that never waits pays
// nothing for the bound.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_word,
                                          uint64_t limit_ns) {
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) {
            return false;
        }
        if ((spin & 15u) == 15u) {
            if (*abort_word) {
                return true;
            }
            const uint64_t now = global_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort_word = 1u;
                return true;
            }
        }
    }
}

// The same wait for the way out of a block that has given up: it does not look
// at the abort word (which is set by then), only at its own clock. Used to let
// copies and multiplies that are still in flight land before the block frees
// its tensor memory and returns.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t t0 = global_ns();
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done || ((spin & 15u) == 15u && global_ns() - t0 > limit_ns)) {
            return;
        }
    }
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One tile of a 2-D tensor map into shared memory; its bytes complete `bar`.
// x (the inner coordinate) times the element size is a multiple of 16 bytes
// at every call site.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x,
                                            int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// K-major operand in shared memory, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart; the start address may be advanced by 32
// bytes per K = 16 step inside the (1024-byte aligned) atom.
__device__ __forceinline__ uint64_t operand_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

// kind::f16: D binary32, A and B bf16, both K-major, N = 64, M = 128.
constexpr uint32_t INSTR_DESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) |
                                ((128u >> 4) << 24);

// D[tmem] (+)= A[tmem] * B[smem]^T.
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(INSTR_DESC), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Four int8 in a word -> two words of bf16 pairs, exactly. With c = 0x43 in
// the high byte, (0x4300 | b) & 0xFF7F is 128 + (b & 127) and
// (0x4300 | b) & 0xFF80 is 128 or 256: their difference is the signed byte.
// (A variant that trades the two masks for two bf16 fused multiply-adds and a
// minimum was measured slower.)
template <bool UNSIGNED>
__device__ __forceinline__ void widen4(uint32_t x, uint32_t &lo, uint32_t &hi) {
    const uint32_t t01 = __byte_perm(x, 0x43434343u, 0x5140);
    const uint32_t t23 = __byte_perm(x, 0x43434343u, 0x5342);
    // An unsigned byte q widens to q - 128: the same subtraction with the
    // byte's top bit flipped in the subtrahend.
    constexpr uint32_t FLIP = UNSIGNED ? 0x00800080u : 0u;
    const uint32_t a01 = t01 & 0xFF7FFF7Fu, b01 = (t01 ^ FLIP) & 0xFF80FF80u;
    const uint32_t a23 = t23 & 0xFF7FFF7Fu, b23 = (t23 ^ FLIP) & 0xFF80FF80u;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(a01), "r"(b01));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(a23), "r"(b23));
}

// The same for four bytes below 128 (4-bit codes): 0x4300 | b is 128 + b as it
// stands, and one subtraction of 128 per pair is all that is left.
__device__ __forceinline__ void widen4_small(uint32_t x, uint32_t &lo, uint32_t &hi) {
    const uint32_t t01 = __byte_perm(x, 0x43434343u, 0x5140);
    const uint32_t t23 = __byte_perm(x, 0x43434343u, 0x5342);
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(t01), "r"(0x43004300u));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(t23), "r"(0x43004300u));
}

// Two binary32 values in one 64-bit register, and the packed fused
// multiply-add on them (each half rounds as a scalar fma does).
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void fma2(uint64_t &acc, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}

#define LM_T0() do {} while (0)
#define LM_ACC(var) do {} while (0)

// VARIANT is 0 in the product; debug builds instantiate others that leave
// out the epilogue's math (bit 0), the conversion (bit 1), the hidden-state
// copies (bit 3) or the weight copies (bit 4) to time the rest. Bit 5 selects
// the affine storage (unsigned bytes, a bias per group).
constexpr int VARIANT_AFFINE = 32;
// Bit 6 (with bit 5): the affine storage in 4 bits, eight codes to a 32-bit word,
// low nibble first (src/kernels/metal/quant.metal:44-66, src/weights.rs:20-36). A
// stage's 128 bytes per row are then four groups, not two; a thread splits a word
// into its low and high nibbles, interleaves them back into code order with two
// byte permutes and widens the eight small bytes as it widens int8 (a code is at
// most 15: no shift by 128, the bias term is bias * sum of the hidden values).
constexpr int VARIANT_Q4 = 64;
template <int VARIANT>
__global__ void __launch_bounds__(THREADS, 1) lmhead_int8_kernel(const __grid_constant__ Args a) {
    constexpr bool AFFINE = (VARIANT & VARIANT_AFFINE) != 0;
    constexpr bool Q4 = (VARIANT & VARIANT_Q4) != 0;
    static_assert(!Q4 || AFFINE, "4-bit codes come with a bias per group");
    constexpr uint32_t RG = Q4 ? 2u * RAW_GROUPS : (uint32_t)RAW_GROUPS;  // groups per stage
    extern __shared__ uint8_t smem_unaligned[];
    const uint32_t base = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_unaligned + (base - smem_u32(smem_unaligned));
    volatile uint32_t *abort_word = reinterpret_cast<volatile uint32_t *>(base_ptr + Smem::ABORT);
    volatile uint32_t *tmem_word = reinterpret_cast<volatile uint32_t *>(base_ptr + Smem::TMEM_ADDR);

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5;
    const uint32_t lane = tid & 31u;

    const uint32_t groups = a.k / GROUP_K;
    const uint32_t n_tiles = (a.rows + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const uint32_t total_groups = my_tiles * groups;
    const uint64_t wait_ns = a.wait_ns;

    if (tid == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) {
            mbar_init(base + Smem::RAW_FULL + 8 * s, 1);
            mbar_init(base + Smem::RAW_EMPTY + 8 * s, N_CONV_WARPS);
        }
        for (int s = 0; s < A_SLOTS; ++s) {
            mbar_init(base + Smem::A_FULL + 8 * s, N_CONV_WARPS);
        }
        for (int s = 0; s < H_SLOTS; ++s) {
            mbar_init(base + Smem::H_FULL + 8 * s, 1);
        }
        for (int s = 0; s < DONE_SLOTS; ++s) {
            mbar_init(base + Smem::DONE + 8 * s, 2);
        }
        for (int b = 0; b < ACC_BUFS; ++b) {
            mbar_init(base + Smem::ACC_EMPTY + 8 * b, N_EPI_WARPS);
        }
        mbar_init(base + Smem::FINAL, 1);
        mbar_init(base + Smem::FINAL + 8, 1);
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         base + Smem::TMEM_ADDR),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_word;

    if (warp == WARP_MMA || warp == WARP_MMA1) {
        // ---- two issuing threads, one per 128 rows of the tile (issuing a
        // multiply costs its thread some 60 clocks: one thread cannot keep up)
        if (lane == 0) {
            const uint32_t half = warp == WARP_MMA ? 0u : 1u;
            long long tw_h = 0, tw_acc = 0, tw_a = 0, t_issue = 0, t_commit = 0;
            LM_T0();
            for (uint32_t q = 0; q < total_groups; ++q) {
                const uint32_t as = q % A_SLOTS, hs = q % H_SLOTS, b = q % ACC_BUFS;
                if (mbar_wait(base + Smem::H_FULL + 8 * hs, (q / H_SLOTS) & 1u, abort_word, wait_ns)) {
                    break;
                }
                LM_ACC(tw_h);
                if (mbar_wait(base + Smem::ACC_EMPTY + 8 * b, ((q / ACC_BUFS) & 1u) ^ 1u, abort_word, wait_ns)) {
                    break;
                }
                LM_ACC(tw_acc);
                if (mbar_wait(base + Smem::A_FULL + 8 * as, (q / A_SLOTS) & 1u, abort_word, wait_ns)) {
                    break;
                }
                LM_ACC(tw_a);
                tc_fence_after();
                const uint32_t h_addr = base + Smem::HID + hs * H_BYTES;
#pragma unroll
                for (uint32_t k4 = 0; k4 < 4; ++k4) {
                    mma_bf16_ts(tmem + b * ACC_COLS + half * TOK,
                                tmem + A_COL0 + as * A_COLS + half * (A_COLS / 2) + k4 * 8u,
                                operand_desc(h_addr + k4 * 32u), k4);
                }
                LM_ACC(t_issue);
                mma_commit(base + Smem::DONE + 8 * (q % DONE_SLOTS));
                LM_ACC(t_commit);
            }
            // The multiplies this thread has issued must have run before the tensor
            // memory they use is freed. On the normal way out the epilogue has seen
            // to that already and this wait finds its phase complete; it matters
            // when the block has given up.
            mma_commit(base + Smem::FINAL + 8 * half);
            mbar_drain(base + Smem::FINAL + 8 * half, 0u, wait_ns);
        }
        __syncwarp();
    } else if (warp == WARP_LOAD) {
        // ---- one thread asks the copy engine for every stage of weights and
        // every group's slice of the hidden states, as far ahead as slots are free
        if (lane == 0) {
            const uint32_t stages_per_tile = groups / RG;
            const uint32_t n_stages = my_tiles * stages_per_tile;
            long long tw_re = 0, tw_he = 0;
            // The copies asked for last, per slot (bit s: slot s has one; its phase's
            // parity beside it): what the way out has to wait for if the block gives up.
            uint32_t raw_asked = 0, raw_parity = 0, h_asked = 0, h_parity = 0;
            bool gave_up = false;
            LM_T0();
            for (uint32_t i = 0; i < n_stages && !gave_up; ++i) {
                const uint32_t st = i % RAW_STAGES;
                const uint32_t tile = blockIdx.x + (i / stages_per_tile) * gridDim.x;
                const uint32_t kb = (i % stages_per_tile) * (GROUP_K * RG);  // first column of the stage
                if (mbar_wait(base + Smem::RAW_EMPTY + 8 * st, ((i / RAW_STAGES) & 1u) ^ 1u, abort_word, wait_ns)) {
                    break;
                }
                LM_ACC(tw_re);
                if (i == a.lost_stage && blockIdx.x == 0) {
                    // test hook: nothing is asked for, the stage never fills
                } else if (!(VARIANT & 16)) {
                    raw_asked |= 1u << st;
                    raw_parity = (raw_parity & ~(1u << st)) | (((i / RAW_STAGES) & 1u) << st);
                    mbar_expect_tx(base + Smem::RAW_FULL + 8 * st, RAW_STAGE_BYTES);
                    tma_load_2d(base + Smem::RAW + st * RAW_STAGE_BYTES, &a.w_map, base + Smem::RAW_FULL + 8 * st,
                                (int32_t)(Q4 ? kb / 2u : kb), (int32_t)(tile * TILE_ROWS));  // (a byte offset)
                } else {
                    mbar_arrive(base + Smem::RAW_FULL + 8 * st);
                }
#pragma unroll
                for (uint32_t gg = 0; gg < RG; ++gg) {
                    const uint32_t q = i * RG + gg;
                    const uint32_t hs = q % H_SLOTS;
                    if (q >= (uint32_t)H_SLOTS) {  // the slot's previous group has been multiplied
                        if (mbar_wait(base + Smem::DONE + 8 * hs, ((q / H_SLOTS) & 1u) ^ 1u, abort_word, wait_ns)) {
                            gave_up = true;
                            break;
                        }
                    }
                    LM_ACC(tw_he);
                    if (!(VARIANT & 8)) {
                        h_asked |= 1u << hs;
                        h_parity = (h_parity & ~(1u << hs)) | (((q / H_SLOTS) & 1u) << hs);
                        mbar_expect_tx(base + Smem::H_FULL + 8 * hs, H_BYTES);
                        tma_load_2d(base + Smem::HID + hs * H_BYTES, &a.h_map, base + Smem::H_FULL + 8 * hs,
                                    (int32_t)(kb + gg * GROUP_K), 0);
                    } else {
                        mbar_arrive(base + Smem::H_FULL + 8 * hs);
                    }
                }
            }
            if (*abort_word) {
                // The block has given up: the copies asked for land in this block's
                // shared memory, so it stays until they have.
#pragma unroll
                for (uint32_t s2 = 0; s2 < (uint32_t)RAW_STAGES; ++s2) {
                    if ((raw_asked >> s2) & 1u) {
                        mbar_drain(base + Smem::RAW_FULL + 8 * s2, (raw_parity >> s2) & 1u, wait_ns);
                    }
                }
#pragma unroll
                for (uint32_t s2 = 0; s2 < (uint32_t)H_SLOTS; ++s2) {
                    if ((h_asked >> s2) & 1u) {
                        mbar_drain(base + Smem::H_FULL + 8 * s2, (h_parity >> s2) & 1u, wait_ns);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp < WARP_EPI0) {
        // ---- int8 bytes in; one thread per tile row widens them into tensor memory
        const uint32_t ct = tid - 32u * WARP_CONV0;
        const uint32_t quad = warp & 3u;                    // the TMEM lanes this warp may write
        const uint32_t half = (warp - WARP_CONV0) >> 2;     // which 128 rows of the tile
        const uint32_t trow = half * 128u + quad * 32u + lane;
        const uint32_t t_lane = (quad * 32u) << 16;
        const uint32_t stages_per_tile = groups / RG;
        const uint32_t n_stages = my_tiles * stages_per_tile;
        long long tw_raw = 0, tw_ae = 0, t_conv = 0, t_st = 0;
        bool conv_gave_up = false;
        LM_T0();
        for (uint32_t i = 0; i < n_stages; ++i) {
            const uint32_t st = i % RAW_STAGES;
            // (the vote takes the place of a __syncwarp: the lanes leave together)
            if (__any_sync(0xFFFFFFFFu, mbar_wait(base + Smem::RAW_FULL + 8 * st, (i / RAW_STAGES) & 1u, abort_word,
                                                  wait_ns))) {
                break;
            }
            LM_ACC(tw_raw);
            const uint32_t raw_row = base + Smem::RAW + st * RAW_STAGE_BYTES + trow * 128u;
#pragma unroll 1
            for (uint32_t gg = 0; gg < RG; ++gg) {
                const uint32_t q = i * RG + gg;
                const uint32_t as = q % A_SLOTS;
                // Widen first (it needs no slot), then wait for the slot: the
                // conversion overlaps the multiplies still reading the slot.
                uint32_t o[2][16];
#pragma unroll
                for (uint32_t part = 0; part < 2; ++part) {
                    if (Q4) {
                        // 16 bytes = 32 codes of the group's 64.
                        uint32_t x[4];
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3])
                                     : "r"(raw_row + (((gg * 2u + part) ^ (trow & 7u)) << 4)));
#pragma unroll
                        for (uint32_t w = 0; w < 4; ++w) {
                            const uint32_t lo = x[w] & 0x0F0F0F0Fu, hi = (x[w] >> 4) & 0x0F0F0F0Fu;
                            const uint32_t c0123 = __byte_perm(lo, hi, 0x5140);  // codes 0..3 of the word, a byte each
                            const uint32_t c4567 = __byte_perm(lo, hi, 0x7362);
                            widen4_small(c0123, o[part][4 * w + 0], o[part][4 * w + 1]);
                            widen4_small(c4567, o[part][4 * w + 2], o[part][4 * w + 3]);
                        }
                    } else if (!(VARIANT & 2)) {
#pragma unroll
                        for (uint32_t c = 0; c < 2; ++c) {
                            uint32_t x0, x1, x2, x3;
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                                         : "r"(raw_row + (((gg * 4u + part * 2u + c) ^ (trow & 7u)) << 4)));
                            widen4<AFFINE>(x0, o[part][8 * c + 0], o[part][8 * c + 1]);
                            widen4<AFFINE>(x1, o[part][8 * c + 2], o[part][8 * c + 3]);
                            widen4<AFFINE>(x2, o[part][8 * c + 4], o[part][8 * c + 5]);
                            widen4<AFFINE>(x3, o[part][8 * c + 6], o[part][8 * c + 7]);
                        }
                    } else {
#pragma unroll
                        for (uint32_t c = 0; c < 16; ++c) {
                            o[part][c] = 0x3F803F80u;
                        }
                    }
                }
                LM_ACC(t_conv);
                bool gave_up = false;
                if (q >= (uint32_t)A_SLOTS) {  // group q - 2, the slot's last user, has been multiplied
                    gave_up = mbar_wait(base + Smem::DONE + 8 * ((q - A_SLOTS) % DONE_SLOTS),
                                        ((q - A_SLOTS) / DONE_SLOTS) & 1u, abort_word, wait_ns);
                }
                LM_ACC(tw_ae);
                if (__any_sync(0xFFFFFFFFu, gave_up)) {
                    conv_gave_up = true;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = tmem + t_lane + A_COL0 + as * A_COLS + half * (A_COLS / 2);
                tmem_st16(a_addr, o[0]);
                tmem_st16(a_addr + 16u, o[1]);
                tmem_st_wait();
                tc_fence_before();
                // One arrival per warp: arrivals on one barrier are serialised.
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(base + Smem::A_FULL + 8 * as);
                }
                LM_ACC(t_st);
            }
            if (conv_gave_up) {
                break;
            }
            // The stage's bytes are in registers or tensor memory: the slot may be refilled.
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(base + Smem::RAW_EMPTY + 8 * st);
            }
        }
    } else {
        // ---- scale each group's sums and add them up; write the tile
        const uint32_t e = warp - WARP_EPI0;
        const uint32_t quad = warp & 3u;   // the TMEM lanes this warp may read
        const uint32_t half = (e >> 2) & 1u;  // which 128 rows of the tile
        const uint32_t tok0 = (e >> 3) * (TOK / 2);  // which 32 tokens of the row
        const uint32_t t_lane = (quad * 32u) << 16;
        uint32_t q = 0;
        long long tw_af = 0, t_math = 0, t_store = 0;
        LM_T0();
        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t row = tile * TILE_ROWS + half * 128u + quad * 32u + lane;
            const uint32_t rowc = min(row, a.rows - 1u);
            const uint4 *srow = reinterpret_cast<const uint4 *>(a.scales + (uint64_t)rowc * groups);
            uint64_t acc[TOK / 4];  // 32 tokens, two per register
#pragma unroll
            for (int m = 0; m < TOK / 4; ++m) {
                acc[m] = 0ull;
            }
            if (AFFINE && row < a.rows) {
                // The sums start from the term the bias kernel left in `out`; the
                // loads complete while the first groups are multiplied.
#pragma unroll
                for (int m = 0; m < TOK / 4; ++m) {
                    uint32_t lo = 0u, hi = 0u;
                    if (tok0 + 2u * m < a.tokens) {
                        lo = __float_as_uint(__ldcg(a.out + (uint64_t)(tok0 + 2 * m) * a.ldo + row));
                    }
                    if (tok0 + 2u * m + 1u < a.tokens) {
                        hi = __float_as_uint(__ldcg(a.out + (uint64_t)(tok0 + 2 * m + 1) * a.ldo + row));
                    }
                    acc[m] = pack2(lo, hi);
                }
            }
            uint4 sc_next = __ldg(srow);
            for (uint32_t g8 = 0; g8 < groups; g8 += 8) {
                const uint4 sc = sc_next;
                if (g8 + 8u < groups) {
                    sc_next = __ldg(srow + (g8 >> 3) + 1u);
                }
                const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (uint32_t gi = 0; gi < 8; ++gi, ++q) {
                    const uint32_t b = q % ACC_BUFS;
                    const float s = __uint_as_float((gi & 1u) ? (sw[gi >> 1] & 0xFFFF0000u) : (sw[gi >> 1] << 16));
                    const uint64_t s2 = pack2(__float_as_uint(s), __float_as_uint(s));
                    if (__any_sync(0xFFFFFFFFu, mbar_wait(base + Smem::DONE + 8 * (q % DONE_SLOTS),
                                                          (q / DONE_SLOTS) & 1u, abort_word, wait_ns))) {
                        goto epilogue_out;  // the block has given up: nothing more is read or written
                    }
                    LM_ACC(tw_af);
                    tc_fence_after();
                    const uint32_t taddr = tmem + t_lane + b * ACC_COLS + half * TOK + tok0;
                    if (!(VARIANT & 1)) {
#pragma unroll
                        for (int c = 0; c < TOK / 32; ++c) {
                            uint32_t v[16];
                            tmem_ld16(taddr + 16u * c, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int m = 0; m < 8; ++m) {
                                fma2(acc[8 * c + m], s2, pack2(v[2 * m], v[2 * m + 1]));
                            }
                        }
                    } else {
                        acc[gi] += (uint64_t)__float_as_uint(s) + taddr;
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(base + Smem::ACC_EMPTY + 8 * b);
                    }
                    LM_ACC(t_math);
                }
            }
            if (row < a.rows) {
#pragma unroll
                for (int m = 0; m < TOK / 4; ++m) {
                    float lo, hi;
                    unpack2(acc[m], lo, hi);
                    if (tok0 + 2u * m < a.tokens) {
                        a.out[(uint64_t)(tok0 + 2 * m) * a.ldo + row] = lo;
                    }
                    if (tok0 + 2u * m + 1u < a.tokens) {
                        a.out[(uint64_t)(tok0 + 2 * m + 1) * a.ldo + row] = hi;
                    }
                }
            }
            LM_ACC(t_store);
        }
    epilogue_out:;
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && *abort_word) {
        atomicOr(a.status_word, 1u << STATUS_TIMEOUT_BIT);
    }
}

// Affine storage, the term the multiplier does not see: with the converters
// widening q - 128,
//   sum_c (scale * q + bias) * h = scale * sum_c (q - 128) * h + (128 * scale + bias) * sum_c h
// per group, and this kernel writes out[t, n] = sum_g (128 * scale[n, g] +
// bias[n, g]) * hsum[g, t]; the head kernel then adds its own sums to it.
// A thread owns 4 vocabulary rows x 16 tokens, their partial results in registers;
// the group sums of the hidden states (binary32, index order; [group][token],
// tokens past the last: 0) come from hidden_group_sums_kernel, which runs
// before it, one block per group and one thread per token.
__global__ void __launch_bounds__(TOK) hidden_group_sums_kernel(const __nv_bfloat16 *hidden, uint64_t ld,
                                                                uint32_t tokens, float *out) {
    const uint32_t g = blockIdx.x, t = threadIdx.x;
    float sum = 0.0f;
    if (t < tokens) {
        const uint4 *src = reinterpret_cast<const uint4 *>(hidden + (uint64_t)t * ld + (uint64_t)g * GROUP_K);
#pragma unroll
        for (int i = 0; i < GROUP_K / 8; ++i) {
            const uint4 v = __ldg(src + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sum += __uint_as_float(w[j] << 16);
                sum += __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
    }
    out[(uint64_t)g * TOK + t] = sum;
}

constexpr int BIAS_THREADS = 128;
constexpr uint32_t BIAS_ROWS = BIAS_THREADS * 4 / 4;  // a warp covers 32 rows x 64 tokens
constexpr uint32_t BIAS_MAX_GROUPS = 128;             // hidden <= 8192

// Dynamic shared memory: the group sums, then the block's scales and biases,
// each row padded by 16 bytes so that rows four apart fall into different banks.
__host__ __device__ constexpr uint32_t bias_row_bytes(uint32_t groups) { return groups * 2u + 16u; }
__host__ __device__ constexpr uint32_t bias_smem_bytes(uint32_t groups) {
    return groups * TOK * 4u + 2u * BIAS_ROWS * bias_row_bytes(groups);
}

__global__ void __launch_bounds__(BIAS_THREADS) affine_bias_term_kernel(
    const float *group_sums, uint32_t tokens, const __nv_bfloat16 *scales, const __nv_bfloat16 *biases,
    uint32_t groups, uint32_t rows, float *out, uint64_t ldo, float code_offset) {
    extern __shared__ __align__(16) uint8_t bias_smem[];
    float *hsum = reinterpret_cast<float *>(bias_smem);  // [group][token]
    uint8_t *sc_s = bias_smem + groups * TOK * 4u;
    const uint32_t row_bytes = bias_row_bytes(groups);
    uint8_t *bi_s = sc_s + BIAS_ROWS * row_bytes;
    const uint32_t block_row0 = blockIdx.x * BIAS_ROWS;
    for (uint32_t i = threadIdx.x; i < groups * TOK / 4u; i += BIAS_THREADS) {
        reinterpret_cast<float4 *>(hsum)[i] = __ldg(reinterpret_cast<const float4 *>(group_sums) + i);
    }
    {
        const uint32_t per_row = groups / 8u;  // 16-byte pieces of a row
        for (uint32_t i = threadIdx.x; i < BIAS_ROWS * per_row; i += BIAS_THREADS) {
            const uint32_t r = i / per_row, piece = i % per_row;
            const uint32_t rowc = min(block_row0 + r, rows - 1u);
            const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(scales + (uint64_t)rowc * groups) + piece);
            const uint4 bv = __ldg(reinterpret_cast<const uint4 *>(biases + (uint64_t)rowc * groups) + piece);
            *reinterpret_cast<uint4 *>(sc_s + r * row_bytes + piece * 16u) = sv;
            *reinterpret_cast<uint4 *>(bi_s + r * row_bytes + piece * 16u) = bv;
        }
    }
    __syncthreads();
    // A thread owns 4 rows x 16 tokens: a group's 16 sums are read once from
    // shared memory for 64 multiply-adds.
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    // Its rows are 8 apart, so that the eight threads that read scales at
    // once read consecutive (padded) rows: no bank conflicts, and the stores
    // of one token fill whole sectors.
    const uint32_t lrow0 = warp * 32u + (lane >> 2);
    const uint32_t row0 = block_row0 + lrow0;
    const uint32_t tok0 = (lane & 3u) * 16u;
    const uint4 *srow[4], *brow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        srow[r] = reinterpret_cast<const uint4 *>(sc_s + (lrow0 + 8u * r) * row_bytes);
        brow[r] = reinterpret_cast<const uint4 *>(bi_s + (lrow0 + 8u * r) * row_bytes);
    }
    uint64_t acc[4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            acc[r][m] = 0ull;
        }
    }
    for (uint32_t g8 = 0; g8 < groups; g8 += 8) {
        uint32_t sw[4][4], bw[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint4 sc = srow[r][g8 >> 3];
            const uint4 bi = brow[r][g8 >> 3];
            sw[r][0] = sc.x, sw[r][1] = sc.y, sw[r][2] = sc.z, sw[r][3] = sc.w;
            bw[r][0] = bi.x, bw[r][1] = bi.y, bw[r][2] = bi.z, bw[r][3] = bi.w;
        }
#pragma unroll
        for (uint32_t gi = 0; gi < 8; ++gi) {
            const ulonglong2 *hs = reinterpret_cast<const ulonglong2 *>(hsum + (g8 + gi) * TOK + tok0);
            ulonglong2 h2[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                h2[m] = hs[m];
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float s = __uint_as_float((gi & 1u) ? (sw[r][gi >> 1] & 0xFFFF0000u) : (sw[r][gi >> 1] << 16));
                const float b = __uint_as_float((gi & 1u) ? (bw[r][gi >> 1] & 0xFFFF0000u) : (bw[r][gi >> 1] << 16));
                const float shift = fmaf(code_offset, s, b);  // (8-bit codes are widened less 128, 4-bit ones as they are)
                const uint64_t shift2 = pack2(__float_as_uint(shift), __float_as_uint(shift));
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    fma2(acc[r][2 * m], shift2, h2[m].x);
                    fma2(acc[r][2 * m + 1], shift2, h2[m].y);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t row = row0 + 8u * r;
        if (row < rows) {
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                float lo, hi;
                unpack2(acc[r][m], lo, hi);
                if (tok0 + 2u * m < tokens) {
                    out[(uint64_t)(tok0 + 2 * m) * ldo + row] = lo;
                }
                if (tok0 + 2u * m + 1u < tokens) {
                    out[(uint64_t)(tok0 + 2 * m + 1) * ldo + row] = hi;
                }
            }
        }
    }
}

}  // namespace lily_head
