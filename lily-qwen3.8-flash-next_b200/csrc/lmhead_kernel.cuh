// The 8-bit LM head that feeds the sampler: logits[t, n] = sum over column
// groups g of scale[n, g] * (sum over the group's 64 columns of w[n, c] * h[t, c]),
// w int8 (symmetric), scale bf16 per 64 columns, h bf16, everything summed in
// binary32. It stands where the reference projects the hidden state through
// its quantised head before sampling (gemv_quant, src/kernels/quant.rs:141-175,
// called from src/qwen4exp/model.rs:2999-3006); the reference's format is
// affine 4/8-bit, this one is the symmetric int8 layout of the vocab-sharded
// configuration, so parity here is by tolerance against a binary32 CPU sum.
//
// sm_100a only. The weights are the only large operand (1 byte per
// multiply-add), so the kernel is a stream of them through the tensor cores:
//
//   * a tile is 256 vocabulary rows; per 64-column group the int8 bytes of
//     the tile (16 KB) arrive by cp.async, are widened to bf16 exactly (every
//     int8 is a bf16) and stored in the 128-byte-swizzled K-major layout;
//   * one thread issues, per group, 2 x 4 tcgen05.mma (M = 128 rows, N = 64
//     tokens, K = 16) into a TMEM accumulator that starts from zero: products
//     of two bf16 are exact in binary32, so only the order of the 64 adds
//     differs from a sequential sum;
//   * eight warps read each group's accumulator back with tcgen05.ld, multiply
//     by the row's scale of that group and add into registers: the group sums
//     cannot stay in TMEM across groups because each has its own scale;
//   * after the last group the tile's 256 x 64 logits go to global memory.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out sets an
// abort word, after which no wait blocks any more: the block runs to its end
// (results are garbage, TMEM is freed) and the status word tells the host.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lily_head {

constexpr int TILE_ROWS = 256;   // two M = 128 accumulators
constexpr int TOK = 64;          // MMA N: the most hidden rows per launch
constexpr int GROUP_K = 64;      // columns per scale group = one 128-byte bf16 atom
constexpr int RAW_GROUPS = 2;    // groups per stage of int8 bytes
constexpr int RAW_STAGES = 3;
constexpr int OP_SLOTS = 3;      // bf16 operand slots (A tile + hidden slice)
constexpr int ACC_BUFS = 4;      // TMEM accumulators in flight
constexpr uint32_t RAW_STAGE_BYTES = TILE_ROWS * GROUP_K * RAW_GROUPS;  // 32 KB
constexpr uint32_t A_BYTES = TILE_ROWS * 128;                           // 32 KB
constexpr uint32_t H_BYTES = TOK * 128;                                 // 8 KB
constexpr uint32_t OP_BYTES = A_BYTES + H_BYTES;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 128;  // two row halves x 64 tokens

constexpr int WARP_MMA = 0;
constexpr int WARP_HIDDEN = 1;
constexpr int WARP_CONV0 = 2;
constexpr int N_CONV_WARPS = 4;
constexpr int WARP_EPI0 = 6;
constexpr int N_EPI_WARPS = 8;
constexpr int THREADS = 32 * (WARP_EPI0 + N_EPI_WARPS);  // 448
constexpr int CONV_THREADS = 32 * N_CONV_WARPS;
constexpr int EPI_THREADS = 32 * N_EPI_WARPS;

constexpr uint32_t STATUS_TIMEOUT_BIT = 30;  // bit of the handle's status word

struct Smem {
    // Offsets from a 1024-byte aligned base.
    static constexpr uint32_t OPS = 0;
    static constexpr uint32_t RAW = OPS + OP_SLOTS * OP_BYTES;
    static constexpr uint32_t BARS = RAW + RAW_STAGES * RAW_STAGE_BYTES;
    static constexpr uint32_t FULL = BARS;                       // [OP_SLOTS]
    static constexpr uint32_t EMPTY = FULL + 8 * OP_SLOTS;       // [OP_SLOTS]
    static constexpr uint32_t ACC_FULL = EMPTY + 8 * OP_SLOTS;   // [ACC_BUFS]
    static constexpr uint32_t ACC_EMPTY = ACC_FULL + 8 * ACC_BUFS;
    static constexpr uint32_t TMEM_ADDR = ACC_EMPTY + 8 * ACC_BUFS;
    static constexpr uint32_t ABORT = TMEM_ADDR + 4;
    static constexpr uint32_t END = ABORT + 4;
    static constexpr uint32_t BYTES = END + 1024;  // room to align the base
};
static_assert(Smem::BYTES <= 227 * 1024, "shared memory of one block");

struct Args {
    const int8_t *w;            // [rows, ldw]
    uint64_t ldw;               // = hidden
    const __nv_bfloat16 *scales;  // [rows, hidden / 64]
    const __nv_bfloat16 *hidden;  // [tokens, ldh]
    uint64_t ldh;
    uint32_t tokens;            // <= 64
    uint32_t k;                 // hidden size, a multiple of 512
    uint32_t rows;              // vocabulary rows of this shard
    float *out;                 // [tokens, ldo]
    uint64_t ldo;
    uint32_t *status_word;
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

// Waits for the phase with the given parity to complete, for at most about a
// second; once any wait of the block has run out, none blocks any more.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_word) {
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
            return;
        }
        if ((spin & 15u) == 15u) {
            if (*abort_word) {
                return;
            }
            const uint64_t now = global_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > 1000000000ull) {
                *abort_word = 1u;
                return;
            }
        }
    }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// K-major operand, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024
// bytes apart; the start address may be advanced by 32 bytes per K = 16 step
// inside the (1024-byte aligned) atom.
__device__ __forceinline__ uint64_t operand_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

// kind::f16: D binary32, A and B bf16, both K-major, N = 64, M = 128.
constexpr uint32_t INSTR_DESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) |
                                ((128u >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(INSTR_DESC), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
__device__ __forceinline__ void widen4(uint32_t x, uint32_t &lo, uint32_t &hi) {
    const uint32_t t01 = __byte_perm(x, 0x43434343u, 0x5140);
    const uint32_t t23 = __byte_perm(x, 0x43434343u, 0x5342);
    const uint32_t a01 = t01 & 0xFF7FFF7Fu, b01 = t01 & 0xFF80FF80u;
    const uint32_t a23 = t23 & 0xFF7FFF7Fu, b23 = t23 & 0xFF80FF80u;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(a01), "r"(b01));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(a23), "r"(b23));
}

__global__ void __launch_bounds__(THREADS, 1) lmhead_int8_kernel(const __grid_constant__ Args a) {
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

    if (tid == 0) {
        for (int s = 0; s < OP_SLOTS; ++s) {
            mbar_init(base + Smem::FULL + 8 * s, CONV_THREADS + 1);
            mbar_init(base + Smem::EMPTY + 8 * s, 1);
        }
        for (int b = 0; b < ACC_BUFS; ++b) {
            mbar_init(base + Smem::ACC_FULL + 8 * b, 1);
            mbar_init(base + Smem::ACC_EMPTY + 8 * b, EPI_THREADS);
        }
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

    if (warp == WARP_MMA) {
        // ---- the issuing thread
        if (lane == 0) {
            for (uint32_t q = 0; q < total_groups; ++q) {
                const uint32_t s = q % OP_SLOTS, b = q % ACC_BUFS;
                mbar_wait(base + Smem::FULL + 8 * s, (q / OP_SLOTS) & 1u, abort_word);
                mbar_wait(base + Smem::ACC_EMPTY + 8 * b, ((q / ACC_BUFS) & 1u) ^ 1u, abort_word);
                fence_async_proxy();
                tc_fence_after();
                const uint32_t a_addr = base + Smem::OPS + s * OP_BYTES;
                const uint32_t h_addr = a_addr + A_BYTES;
#pragma unroll
                for (uint32_t half = 0; half < 2; ++half) {
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4) {
                        mma_bf16(tmem + b * ACC_COLS + half * TOK,
                                 operand_desc(a_addr + half * (A_BYTES / 2) + k4 * 32u),
                                 operand_desc(h_addr + k4 * 32u), k4);
                    }
                }
                mma_commit(base + Smem::EMPTY + 8 * s);
                mma_commit(base + Smem::ACC_FULL + 8 * b);
            }
        }
        __syncwarp();
    } else if (warp == WARP_HIDDEN) {
        // ---- the hidden slice of each group, straight into the swizzled layout
        for (uint32_t q = 0; q <= total_groups; ++q) {
            if (q < total_groups) {
                const uint32_t s = q % OP_SLOTS;
                mbar_wait(base + Smem::EMPTY + 8 * s, ((q / OP_SLOTS) & 1u) ^ 1u, abort_word);
                const uint32_t g = q % groups;
                const uint32_t h_addr = base + Smem::OPS + s * OP_BYTES + A_BYTES;
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) {
                    const uint32_t chunk = lane + 32u * j;
                    const uint32_t m = chunk >> 3, c = chunk & 7u;
                    const bool live = m < a.tokens;
                    const __nv_bfloat16 *src =
                        a.hidden + (live ? (uint64_t)m * a.ldh + (uint64_t)g * GROUP_K + c * 8u : 0u);
                    cp_async16(h_addr + (m >> 3) * 1024u + (m & 7u) * 128u + ((c ^ (m & 7u)) << 4), src,
                               live ? 16u : 0u);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (q >= 1) {
                asm volatile("cp.async.wait_group 1;" ::: "memory");
                fence_async_proxy();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(base + Smem::FULL + 8 * ((q - 1) % OP_SLOTS));
                }
            }
        }
    } else if (warp < WARP_EPI0) {
        // ---- int8 bytes in, bf16 operand tiles out
        const uint32_t ct = tid - 32u * WARP_CONV0;
        const uint32_t stages_per_tile = groups / RAW_GROUPS;
        const uint32_t n_stages = my_tiles * stages_per_tile;
        auto issue_raw = [&](uint32_t i) {
            if (i < n_stages) {
                const uint32_t tile = blockIdx.x + (i / stages_per_tile) * gridDim.x;
                const uint32_t row0 = tile * TILE_ROWS;
                const uint32_t kb = (i % stages_per_tile) * (GROUP_K * RAW_GROUPS);
                const uint32_t dst0 = base + Smem::RAW + (i % RAW_STAGES) * RAW_STAGE_BYTES;
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) {
                    const uint32_t chunk = ct + CONV_THREADS * j;
                    const uint32_t r = chunk >> 3, col = chunk & 7u;
                    const uint32_t grow = min(row0 + r, a.rows - 1u);
                    const int8_t *src = a.w + (uint64_t)grow * a.ldw + kb + col * 16u;
                    // Odd rows swap their two 64-byte halves: the reads below stay free of
                    // bank conflicts.
                    cp_async16(dst0 + r * 128u + ((col ^ ((r & 1u) << 2)) << 4), src, 16u);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        issue_raw(0);
        issue_raw(1);
        for (uint32_t i = 0; i < n_stages; ++i) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            __syncwarp();
            asm volatile("bar.sync 1, %0;" ::"n"(CONV_THREADS) : "memory");
            issue_raw(i + 2);
            const uint32_t raw0 = base + Smem::RAW + (i % RAW_STAGES) * RAW_STAGE_BYTES;
#pragma unroll 1
            for (uint32_t gg = 0; gg < RAW_GROUPS; ++gg) {
                const uint32_t q = i * RAW_GROUPS + gg;
                const uint32_t s = q % OP_SLOTS;
                mbar_wait(base + Smem::EMPTY + 8 * s, ((q / OP_SLOTS) & 1u) ^ 1u, abort_word);
                const uint32_t a_addr = base + Smem::OPS + s * OP_BYTES;
                const uint32_t j4 = ct & 3u;
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t r = (ct >> 2) + 32u * j;
                    const uint32_t pcol = (gg * 4u + j4) ^ ((r & 1u) << 2);
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                                 : "r"(raw0 + r * 128u + (pcol << 4)));
                    uint32_t o[8];
                    widen4(x0, o[0], o[1]);
                    widen4(x1, o[2], o[3]);
                    widen4(x2, o[4], o[5]);
                    widen4(x3, o[6], o[7]);
                    const uint32_t line = a_addr + (r >> 3) * 1024u + (r & 7u) * 128u;
                    // The swizzle already separates an even row from the odd row below it.
                    const uint32_t ca = 2u * j4, cb = 2u * j4 + 1u;
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(line + ((ca ^ (r & 7u)) << 4)),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                 : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(line + ((cb ^ (r & 7u)) << 4)),
                                 "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                                 : "memory");
                }
                fence_async_proxy();
                mbar_arrive(base + Smem::FULL + 8 * s);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ---- scale each group's sums and add them up; write the tile
        const uint32_t e = warp - WARP_EPI0;
        const uint32_t quad = warp & 3u;   // the TMEM lanes this warp may read
        const uint32_t half = e >> 2;      // which 128 rows of the tile
        const uint32_t t_lane = (quad * 32u) << 16;
        uint32_t q = 0;
        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t row = tile * TILE_ROWS + half * 128u + quad * 32u + lane;
            const uint32_t rowc = min(row, a.rows - 1u);
            const uint4 *srow = reinterpret_cast<const uint4 *>(a.scales + (uint64_t)rowc * groups);
            float acc[TOK];
#pragma unroll
            for (int m = 0; m < TOK; ++m) {
                acc[m] = 0.0f;
            }
            for (uint32_t g8 = 0; g8 < groups; g8 += 8) {
                const uint4 sc = __ldg(srow + (g8 >> 3));
                const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (uint32_t gi = 0; gi < 8; ++gi, ++q) {
                    const uint32_t b = q % ACC_BUFS;
                    const float s = __uint_as_float((gi & 1u) ? (sw[gi >> 1] & 0xFFFF0000u) : (sw[gi >> 1] << 16));
                    mbar_wait(base + Smem::ACC_FULL + 8 * b, (q / ACC_BUFS) & 1u, abort_word);
                    __syncwarp();
                    tc_fence_after();
                    const uint32_t taddr = tmem + t_lane + b * ACC_COLS + half * TOK;
                    uint32_t v[32];
                    tmem_ld32(taddr, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int m = 0; m < 32; ++m) {
                        acc[m] = __fadd_rn(acc[m], __fmul_rn(s, __uint_as_float(v[m])));
                    }
                    tmem_ld32(taddr + 32u, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int m = 0; m < 32; ++m) {
                        acc[32 + m] = __fadd_rn(acc[32 + m], __fmul_rn(s, __uint_as_float(v[m])));
                    }
                    tc_fence_before();
                    mbar_arrive(base + Smem::ACC_EMPTY + 8 * b);
                }
            }
            if (row < a.rows) {
#pragma unroll
                for (int m = 0; m < TOK; ++m) {
                    if ((uint32_t)m < a.tokens) {
                        a.out[(uint64_t)m * a.ldo + row] = acc[m];
                    }
                }
            }
        }
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

}  // namespace lily_head
