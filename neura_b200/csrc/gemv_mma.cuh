// Decode product: out[r][c] = chain(sum_k W[c][k] x[r][k]) for r <= 16 activation rows,
// W streamed once from HBM in the tiled layout (layout.cuh), x staged as int8 digit
// planes (prep.cuh), the dot products on mma.sync.m16n8k32 (u8|s8 x s8 -> s32).
//
// This stands in for template_run_matmul_folded and its per-format dots
// (crates/neura-kernel/src/task/matmul.rs:376-517, dot.rs:471-542, :583-619).
//
// Work split.  A "unit" is one 32-row tile x one block of K (a Q4_K super-block or a
// Q8_0 block); units are contiguous in memory in (tile, block) order.  Every warp of
// the grid takes one contiguous, equally long run of units, so all SMs stream the same
// number of bytes whatever N and K are.  A run may start or end inside a tile; such a
// tile is finished by the last of its contributing warps to arrive (a counter per
// tile, no waiting), which adds the partial sums in warp order, so results do not
// depend on timing.
//
// Data movement.  Each warp owns a ring of shared-memory stages that one lane fills
// with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier), several
// stages ahead of the MMA work, so the bytes in flight per SM do not depend on
// registers.  Waits on those barriers are bounded: a warp that gives up raises the
// status word, drains its own copies and leaves.
#pragma once
#include "common.cuh"
#include "prep.cuh"

namespace nc {

#ifndef NC_GEMV_WARPS
#define NC_GEMV_WARPS 8   // warps a CTA; two such CTAs share an SM
#endif
constexpr int kGemvWarps = NC_GEMV_WARPS;            // warps per CTA (they never synchronise with each other)
constexpr uint32_t kQ4kStage = 2 * kQ4kUnit;       // one 32-row unit: 4608 B
constexpr uint32_t kQ8Group = 4;                   // 32-row units per stage
constexpr uint32_t kQ8Stage = kQ8Group * 2 * kQ8Unit;  // 4352 B
constexpr unsigned long long kWaitNanos = 2000000000ull;  // a warp gives up on a copy after two seconds

struct GemvParams {
    const uint8_t *w;     // tiled weights
    const uint8_t *dig;   // activation digit planes
    const float *cs;      // digit scales
    const uint8_t *sums;  // Q4_K: MMA fragments of the per-sub-block digit sums
    float *out;
    float *partial;       // [tile][slot][rows][32] split-tile partial sums
    unsigned int *counters;  // [tile], zero between launches
    unsigned int *status;    // raised when a bounded wait ran out
    uint64_t out_stride;
    uint32_t n, rows, ncols;  // output features; activation rows of this launch and their 3 * rows digit columns
    uint32_t col_stride, col0;  // the staged tables hold col_stride columns a block; this launch reads [col0, col0 + ncols)
    uint32_t upt;         // units per tile (blocks along K)
    uint32_t nwarps;      // warps that take work
    uint32_t q, r;        // every warp takes q units, the first r one more
    uint32_t maxp;        // slots per tile in `partial`
    uint32_t pair;        // 1: a tile is 16 rows of one matrix over the same 16 rows of a second one, and
                          //    output c is silu(first row c) * (second row c): the SwiGLU of a gate and an up projection
    Chain chain;
    StageAfter then;          // has_then: finished tiles are counted and full chunks digitised for the next product
    uint32_t has_then;
    const float *sumsq;       // not null: [rows][sumsq_chunks] sums of squares of the input rows, whose rms_norm
    uint32_t sumsq_chunks;    //           scalar 1 / sqrt(sum / k + floor) multiplies the outputs
    float floor, inv_k;
};

// D = A * B with a zero accumulator (the zeros are immediates, not registers).
__device__ __forceinline__ void mma_u8s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// ---- shared-memory ring plumbing ----------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ unsigned long long global_nanos() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits for a stage with a time limit; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long start = global_nanos();
    for (;;) {
#pragma unroll 1
        for (int tries = 0; tries < 64; ++tries)
            if (mbar_try(bar, parity)) return true;
        if (global_nanos() - start > kWaitNanos) return false;
    }
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds4(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Which warp owns unit u under the (q, r) split (the host keeps the unit count below 2^32).
__device__ __forceinline__ uint32_t owner_of(uint32_t u, uint32_t q, uint32_t r) {
    const uint32_t head = r * (q + 1);
    return u < head ? u / (q + 1) : r + (u - head) / q;
}

// Ends a warp's stretch [first_blk, end_blk) of the 32-row tile `tile`: either finishes the
// tile or leaves a partial for the last contributor to add up.  acc[h] holds, for rows
// 16h..16h+15 and per 8-column MMA tile, (row g, col 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).
// `scale0` and `scale1` multiply the sums of rows 0 and 1 (an rms_norm's scalar; 1 otherwise).  Returns
// whether this warp wrote the tile's final outputs.
// With HOOKS false (the one-launch-per-product kernel) the scales and `p.after` are not looked at.
template <int NT, bool HOOKS>
__device__ __forceinline__ bool flush_tile(const GemvParams &p, float (&acc)[2][NT][4], float *patch, uint32_t warp,
                                        uint32_t tile, uint32_t first_blk, uint32_t end_blk, float scale0_, float scale1_) {
    const float scale0 = HOOKS ? scale0_ : 1.0f, scale1 = HOOKS ? scale1_ : 1.0f;
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int W = NT * 8 + 1;  // padded row of the per-warp patch
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            patch[(16 * h + g) * W + nt * 8 + 2 * t] = acc[h][nt][0];
            patch[(16 * h + g) * W + nt * 8 + 2 * t + 1] = acc[h][nt][1];
            patch[(16 * h + g + 8) * W + nt * 8 + 2 * t] = acc[h][nt][2];
            patch[(16 * h + g + 8) * W + nt * 8 + 2 * t + 1] = acc[h][nt][3];
            acc[h][nt][0] = acc[h][nt][1] = acc[h][nt][2] = acc[h][nt][3] = 0.0f;
        }
    __syncwarp();
    const uint32_t cells = p.rows * 32;
    const bool whole = first_blk == 0 && end_blk == p.upt;
    bool final = whole;
    if (whole && p.pair) {
        for (uint32_t idx = lane; idx < p.rows * 16; idx += 32) {
            const uint32_t rr = idx & 15, b = idx >> 4, col = tile * 16 + rr, up = rr + 16;
            const float rs = b == 0 ? scale0 : scale1;
            const float gate = ((patch[rr * W + 3 * b] + patch[rr * W + 3 * b + 1]) + patch[rr * W + 3 * b + 2]) * rs;
            const float other = ((patch[up * W + 3 * b] + patch[up * W + 3 * b + 1]) + patch[up * W + 3 * b + 2]) * rs;
            if (col < p.n)
                p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, gate * sigmoid_f(gate) * other);
        }
    } else if (whole) {
        for (uint32_t idx = lane; idx < cells; idx += 32) {
            const uint32_t rr = idx & 31, b = idx >> 5, col = tile * 32 + rr;
            const float v = ((patch[rr * W + 3 * b] + patch[rr * W + 3 * b + 1]) + patch[rr * W + 3 * b + 2]) * (b == 0 ? scale0 : scale1);
            if (col < p.n) p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, v);
        }
    } else {
        const uint32_t base = tile * p.upt;
        const uint32_t first = owner_of(base, p.q, p.r), last = owner_of(base + p.upt - 1, p.q, p.r);
        const uint32_t count = last - first + 1, slot = warp - first;
        float *mine = p.partial + ((uint64_t)tile * p.maxp + slot) * cells;
        for (uint32_t idx = lane; idx < cells; idx += 32) {
            const uint32_t rr = idx & 31, b = idx >> 5;
            __stcg(mine + idx, (patch[rr * W + 3 * b] + patch[rr * W + 3 * b + 1]) + patch[rr * W + 3 * b + 2]);
        }
        // the warp's stores are ordered before lane 0's fence by the warp barrier, and the fence
        // makes them visible to the GPU before the arrival is counted
        __syncwarp();
        unsigned int seen = 0;
        if (lane == 0) {
            seen = arrive_on(p.counters + tile);
        }
        seen = __shfl_sync(0xffffffffu, seen, 0);
        final = seen == count - 1;
        if (seen == count - 1 && p.pair) {
            const float *all = p.partial + (uint64_t)tile * p.maxp * cells;
            for (uint32_t idx = lane; idx < p.rows * 16; idx += 32) {
                const uint32_t rr = idx & 15, b = idx >> 4, col = tile * 16 + rr;
                float gate = 0.0f, other = 0.0f;
                for (uint32_t s = 0; s < count; ++s) {
                    gate += __ldcg(all + (uint64_t)s * cells + b * 32 + rr);
                    other += __ldcg(all + (uint64_t)s * cells + b * 32 + rr + 16);
                }
                gate *= b == 0 ? scale0 : scale1;
                other *= b == 0 ? scale0 : scale1;
                if (col < p.n)
                    p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, gate * sigmoid_f(gate) * other);
            }
            if (lane == 0) p.counters[tile] = 0u;
        } else if (seen == count - 1) {
            const float *all = p.partial + (uint64_t)tile * p.maxp * cells;
            for (uint32_t idx = lane; idx < cells; idx += 32) {
                const uint32_t rr = idx & 31, b = idx >> 5, col = tile * 32 + rr;
                float v = 0.0f;
                for (uint32_t s = 0; s < count; ++s) v += __ldcg(all + (uint64_t)s * cells + idx);
                v *= b == 0 ? scale0 : scale1;
                if (col < p.n) p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, v);
            }
            if (lane == 0) p.counters[tile] = 0u;
        }
    }
    __syncwarp();
    if constexpr (HOOKS) {
        if (final && p.has_then) stage_after_piece(p.then, tile * p.then.piece);
    }
    return final;
}

// ---- Q4_K: one 16-row half of a unit ---------------------------------------------------
// dg[nt][i] holds the digit fragments of sub-blocks 2i (.x,.y) and 2i+1 (.z,.w); sf[nt] the
// fragments of the per-sub-block digit sums, low byte (.x,.y) and high byte (.z,.w).
//
// Low nibbles are used as they are and high nibbles in place (16 * q, no shift), so the two
// kinds are summed apart and joined as 16 * low + high with the 1/16 folded into d.
// The min term sum_k m * x_k = m * (sum of the sub-block's digits) takes two MMAs for the whole
// super-block: K slot 4t holds sub-block t (and 16 + 4t sub-block 4 + t), A = the 6-bit mins,
// B = the low and the high byte of the digit sums (prep.cuh).
template <int NT>
__device__ __forceinline__ void q4k_half(uint32_t half_addr, const uint4 (&dg)[NT][4], const uint4 (&sf)[NT],
                                         const float (&c)[NT][2], float (&acc)[NT][4]) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint4 h0 = lds16(half_addr + g * 16), h1 = lds16(half_addr + (g + 8) * 16);
    uint4 q[4];
#pragma unroll
    for (int G = 0; G < 4; ++G) q[G] = lds16(half_addr + 256 + G * 512 + lane * 16);
    uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
    q4k_scales(h0.y, h0.z, h0.w, sc0, mn0);
    q4k_scales(h1.y, h1.z, h1.w, sc1, mn1);
    int lo[NT][4], hi[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) lo[nt][i] = hi[nt][i] = 0;
#pragma unroll
    for (int G = 0; G < 4; ++G) {
        {
            const int sub = G * 2;
            const int s0 = (int)__byte_perm(sc0[sub >> 2], 0u, 0x4440u + (sub & 3));
            const int s1 = (int)__byte_perm(sc1[sub >> 2], 0u, 0x4440u + (sub & 3));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                mma_u8s8_zero(d, q[G].x & 0x0f0f0f0fu, q[G].z & 0x0f0f0f0fu, q[G].y & 0x0f0f0f0fu,
                              q[G].w & 0x0f0f0f0fu, dg[nt][G].x, dg[nt][G].y);
                lo[nt][0] += d[0] * s0;
                lo[nt][1] += d[1] * s0;
                lo[nt][2] += d[2] * s1;
                lo[nt][3] += d[3] * s1;
            }
        }
        {
            const int sub = G * 2 + 1;
            const int s0 = (int)__byte_perm(sc0[sub >> 2], 0u, 0x4440u + (sub & 3));
            const int s1 = (int)__byte_perm(sc1[sub >> 2], 0u, 0x4440u + (sub & 3));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                mma_u8s8_zero(d, q[G].x & 0xf0f0f0f0u, q[G].z & 0xf0f0f0f0u, q[G].y & 0xf0f0f0f0u,
                              q[G].w & 0xf0f0f0f0u, dg[nt][G].z, dg[nt][G].w);
                hi[nt][0] += d[0] * s0;
                hi[nt][1] += d[1] * s0;
                hi[nt][2] += d[2] * s1;
                hi[nt][3] += d[3] * s1;
            }
        }
    }
    // A of the min MMAs: byte 0 of each register is the min of this lane's sub-block; the other
    // bytes meet zero bytes of B
    const uint32_t a0 = mn0[0] >> (8 * t), a2 = mn0[1] >> (8 * t);
    const uint32_t a1 = mn1[0] >> (8 * t), a3 = mn1[1] >> (8 * t);
    // value = (d*sc)*q - dmin*m  (ggml.rs:341-346)  ->  sum = d*sum(sc*q*x) - dmin*sum(m*x)
    const float d0 = half_bits_to_float(h0.x & 0xffffu) * 0.0625f, n0 = half_bits_to_float(h0.x >> 16);
    const float d1 = half_bits_to_float(h1.x & 0xffffu) * 0.0625f, n1 = half_bits_to_float(h1.x >> 16);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int ml[4], mh[4];
        mma_u8s8_zero(ml, a0, a1, a2, a3, sf[nt].x, sf[nt].y);
        mma_u8s8_zero(mh, a0, a1, a2, a3, sf[nt].z, sf[nt].w);
        float qf[4], mf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qf[i] = (float)(lo[nt][i] * 16 + hi[nt][i]);
            mf[i] = (float)(mh[i] * 256 + ml[i]);
        }
        acc[nt][0] = fmaf(d0 * qf[0] - n0 * mf[0], c[nt][0], acc[nt][0]);
        acc[nt][1] = fmaf(d0 * qf[1] - n0 * mf[1], c[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf(d1 * qf[2] - n1 * mf[2], c[nt][0], acc[nt][2]);
        acc[nt][3] = fmaf(d1 * qf[3] - n1 * mf[3], c[nt][1], acc[nt][3]);
    }
}

// ---- Q8_0: one 16-row half of a unit ---------------------------------------------------
template <int NT>
__device__ __forceinline__ void q8_half(uint32_t half_addr, const uint2 (&dg)[NT], const float (&c)[NT][2],
                                        float (&acc)[NT][4]) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2;
    const uint4 q = lds16(half_addr + lane * 16);   // (.x,.y) row g, (.z,.w) row g+8
    const uint32_t dd = lds4(half_addr + 512 + g * 4);
    const float d0 = half_bits_to_float(dd & 0xffffu), d1 = half_bits_to_float(dd >> 16);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int d[4];
        mma_s8s8_zero(d, q.x, q.z, q.y, q.w, dg[nt].x, dg[nt].y);
        acc[nt][0] = fmaf((float)d[0], d0 * c[nt][0], acc[nt][0]);
        acc[nt][1] = fmaf((float)d[1], d0 * c[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf((float)d[2], d1 * c[nt][0], acc[nt][2]);
        acc[nt][3] = fmaf((float)d[3], d1 * c[nt][1], acc[nt][3]);
    }
}

// ---- the streaming kernel ----------------------------------------------------------------
// Activation fragments of one stage (kGroup units): B operands of the MMAs and the digit scales.
template <bool Q4K, int NT>
struct StageFrags {
    static constexpr int kUnits = Q4K ? 1 : (int)kQ8Group;
    uint4 wide[Q4K ? NT : 1][4];          // Q4_K: sub-blocks 2i (.x,.y) and 2i+1 (.z,.w) of 8-column tile nt
    uint4 sums[Q4K ? NT : 1];             // Q4_K: digit sums per sub-block, low and high byte
    uint2 narrow[Q4K ? 1 : kUnits][NT];   // Q8_0: one block per unit
    float c[kUnits][NT][2];
};

// Loads the fragments of the `have` units that start at block `blk` of K (wrapping at the tile end).
template <bool Q4K, int NT>
__device__ __forceinline__ void load_frags(StageFrags<Q4K, NT> &f, const GemvParams &p, uint32_t blk, uint32_t have) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int j = 0; j < StageFrags<Q4K, NT>::kUnits; ++j) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t col = nt * 8 + 2 * t;
            f.c[j][nt][0] = col < p.ncols ? __ldg(p.cs + blk * p.col_stride + p.col0 + col) : 0.0f;
            f.c[j][nt][1] = col + 1 < p.ncols ? __ldg(p.cs + blk * p.col_stride + p.col0 + col + 1) : 0.0f;
            const uint32_t mine = nt * 8 + g;
            const bool live = mine < p.ncols;
            if constexpr (Q4K) {
                const uint32_t entry = (blk * p.col_stride + p.col0 + mine) * 4 + t;
                const uint4 *from = reinterpret_cast<const uint4 *>(p.dig) + entry * 4u;
#pragma unroll
                for (int i = 0; i < 4; ++i) f.wide[nt][i] = live ? __ldg(from + i) : make_uint4(0u, 0u, 0u, 0u);
                f.sums[nt] = live ? __ldg(reinterpret_cast<const uint4 *>(p.sums) + entry) : make_uint4(0u, 0u, 0u, 0u);
            } else {
                f.narrow[j][nt] = live
                    ? __ldg(reinterpret_cast<const uint2 *>(p.dig + (blk * p.col_stride + p.col0 + mine) * 32u + t * 8u))
                    : make_uint2(0u, 0u);
            }
        }
        // units past the warp's run re-read its last block; nothing uses them
        if ((uint32_t)(j + 1) < have && ++blk == p.upt) blk = 0;
    }
}

template <bool Q4K, int NT, int STAGES, bool HOOKS = false>
struct GemvWarp {
    static constexpr uint32_t kStage = Q4K ? kQ4kStage : kQ8Stage;
    static constexpr uint32_t kGroup = Q4K ? 1 : kQ8Group;
    const GemvParams &p;
    uint32_t ring, bars;
    float *patch;
    const uint8_t *src;
    uint64_t bytes;
    uint32_t warp, units, steps;
    uint32_t tile, blk, first_blk, done;
    float acc[2][NT][4];
    uint32_t base = 0;   // fills of this warp's ring before this product (a persistent kernel runs many on one ring)
    float scale0 = 1.0f, scale1 = 1.0f;   // the rms_norm scalars of rows 0 and 1 of the input (GemvParams::sumsq)

    // Unit J of the stage at `buf`.
    template <int J>
    __device__ __forceinline__ void unit(uint32_t buf, const StageFrags<Q4K, NT> &f) {
        if (done >= units) return;
        if constexpr (Q4K) {
            q4k_half<NT>(buf, f.wide, f.sums, f.c[0], acc[0]);
            q4k_half<NT>(buf + kQ4kUnit, f.wide, f.sums, f.c[0], acc[1]);
        } else {
            q8_half<NT>(buf + J * 2 * kQ8Unit, f.narrow[J], f.c[J], acc[0]);
            q8_half<NT>(buf + J * 2 * kQ8Unit + kQ8Unit, f.narrow[J], f.c[J], acc[1]);
        }
        ++done;
        if (++blk == p.upt || done == units) {
            flush_tile<NT, HOOKS>(p, acc, patch, warp, tile, first_blk, blk, scale0, scale1);
            if (blk == p.upt) { blk = 0; ++tile; }
            first_blk = blk;
        }
    }

    // One stage: wait for its bytes, multiply, finish tiles that end in it, refill it.
    // Returns false when the bounded wait ran out.
    __device__ __forceinline__ bool run(uint32_t step, const StageFrags<Q4K, NT> &f) {
        const uint32_t stage = (base + step) % STAGES, parity = ((base + step) / STAGES) & 1u;
        if (!mbar_wait(bars + stage * 8, parity)) return false;
        const uint32_t buf = ring + stage * kStage;
        unit<0>(buf, f);
        if constexpr (kGroup > 1) {
            unit<1>(buf, f);
            unit<2>(buf, f);
            unit<3>(buf, f);
        }
        __syncwarp();  // every lane has read this stage: it may be refilled
        if ((threadIdx.x & 31) == 0 && step + STAGES < steps) {
            const uint64_t at = (uint64_t)(step + STAGES) * kStage;
            const uint32_t len = (uint32_t)min((uint64_t)kStage, bytes - at);
            mbar_expect(bars + stage * 8, len);
            bulk_load(buf, src + at, len, bars + stage * 8);
        }
        return true;
    }

    // The block of K at which the stage after the current one starts.
    __device__ __forceinline__ uint32_t block_after(uint32_t from) const {
        uint32_t next = from + kGroup;
        while (next >= p.upt) next -= p.upt;
        return next;
    }
};

// HOOKS: the product also applies the rms_norm scalar of its input rows (GemvParams::sumsq, at most two rows) and
// stages its own output for the next product (GemvParams::then).
template <bool Q4K, int NT, int STAGES, bool HOOKS = false>
__global__ void __launch_bounds__(kGemvWarps * 32, NT <= 1 ? 16 / kGemvWarps : 1) qlinear_stream_kernel(const __grid_constant__ GemvParams p) {
    static_assert(STAGES >= 2 && kQ8Group == 4, "the four units of a Q8_0 stage are unrolled by hand");
    constexpr uint32_t kStage = Q4K ? kQ4kStage : kQ8Stage;
    constexpr uint32_t kUnit = Q4K ? kQ4kStage : 2 * kQ8Unit;  // bytes of one 32-row unit
    constexpr uint32_t kGroup = Q4K ? 1 : kQ8Group;            // units per stage
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const uint32_t warp = blockIdx.x * kGemvWarps + wib;
    if (warp >= p.nwarps) return;
    GemvWarp<Q4K, NT, STAGES, HOOKS> w{p};
    w.ring = smem_addr(smem) + wib * STAGES * kStage;
    w.bars = smem_addr(smem) + kGemvWarps * STAGES * kStage + wib * STAGES * 8;
    w.patch = reinterpret_cast<float *>(smem + kGemvWarps * STAGES * (kStage + 8)) + wib * 32 * (NT * 8 + 1);
    const uint32_t u0 = warp * p.q + min(warp, p.r);
    w.warp = warp;
    w.units = p.q + (warp < p.r ? 1u : 0u);
    w.steps = (w.units + kGroup - 1) / kGroup;
    w.src = p.w + (uint64_t)u0 * kUnit;
    w.bytes = (uint64_t)w.units * kUnit;

    // The weights do not depend on the kernel before this one: start streaming them at once.
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(w.bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            if ((uint32_t)s < w.steps) {
                const uint64_t at = (uint64_t)s * kStage;
                const uint32_t len = (uint32_t)min((uint64_t)kStage, w.bytes - at);
                mbar_expect(w.bars + s * 8, len);
                bulk_load(w.ring + s * kStage, w.src + at, len, w.bars + s * 8);
            }
        }
    }
    __syncwarp();
    // Programmatic dependent launch: let the next kernel of the stream start its own
    // prologue, then wait until the kernel before this one (the activation staging) is
    // complete and visible.  Both are no-ops in a plain launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    w.tile = u0 / p.upt;
    w.blk = u0 % p.upt;
    w.first_blk = w.blk;
    w.done = 0;
    if constexpr (HOOKS) {
        if (p.sumsq) {   // the chunks' sums of squares, added in chunk order
            float total0 = 0.0f, total1 = 0.0f;
            for (uint32_t c = 0; c < p.sumsq_chunks; ++c) {
                total0 += __ldcg(p.sumsq + c);
                if (p.rows > 1) total1 += __ldcg(p.sumsq + p.sumsq_chunks + c);
            }
            w.scale0 = 1.0f / sqrtf(total0 * p.inv_k + p.floor);
            w.scale1 = 1.0f / sqrtf(total1 * p.inv_k + p.floor);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) w.acc[h][nt][0] = w.acc[h][nt][1] = w.acc[h][nt][2] = w.acc[h][nt][3] = 0.0f;

    // Two fragment sets take turns: the set of the following stage travels while this one is multiplied.
    StageFrags<Q4K, NT> even, odd;
    load_frags<Q4K, NT>(even, p, w.blk, min(w.units, kGroup));
    uint32_t failed = 0xffffffffu;
    for (uint32_t step = 0; step < w.steps; step += 2) {
        const bool second = step + 1 < w.steps;
        if (second) load_frags<Q4K, NT>(odd, p, w.block_after(w.blk), min(w.units - (step + 1) * kGroup, kGroup));
        if (!w.run(step, even)) { failed = step; break; }
        if (second) {
            if (step + 2 < w.steps)
                load_frags<Q4K, NT>(even, p, w.block_after(w.blk), min(w.units - (step + 2) * kGroup, kGroup));
            if (!w.run(step + 1, odd)) { failed = step + 1; break; }
        }
    }
    if (failed != 0xffffffffu) {
        // a copy never landed: say so, then give the copies still in flight a bounded time to
        // land before the shared memory is handed back
        if (lane == 0) atomicOr(p.status, 1u);
        const uint32_t pending = min((uint32_t)STAGES, w.steps - failed);
        for (uint32_t s = 0; s < pending; ++s)
            mbar_wait(w.bars + ((failed + s) % STAGES) * 8, ((failed + s) / STAGES) & 1u);
    }
}

}  // namespace nc
