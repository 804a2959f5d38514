// Decode product: out[r][c] = chain(sum_k W[c][k] x[r][k]) for r <= 16 activation rows,
// W streamed once from HBM in the tiled layout (layout.cuh), x staged as int8 digit
// planes (prep.cuh), the dot products on mma.sync.m16n8k32 (u8|s8 x s8 -> s32).
//
// This stands in for template_run_matmul_folded and its per-format dots
// (crates/neura-kernel/src/task/matmul.rs:376-517, dot.rs:471-542, :583-619).
//
// Work split.  A "unit" is one 16-row tile x one block of K (a Q4_K super-block or a
// Q8_0 block); units are contiguous in memory in (tile, block) order.  Every warp of
// the grid takes one contiguous, equally long run of units, so all SMs stream the same
// number of bytes whatever N and K are.  A run may start or end inside a tile; such a
// tile is finished by the last of its contributing warps to arrive (a counter per
// tile, no waiting), which adds the partial sums in warp order, so results do not
// depend on timing.
#pragma once
#include "common.cuh"

namespace nc {

struct GemvParams {
    const uint8_t *w;     // tiled weights
    const int8_t *dig;    // activation digit planes
    const float *cs;      // digit scales
    float *out;
    float *partial;       // [tile][slot][rows][16] split-tile partial sums
    unsigned int *counters;  // [tile], zero between launches
    uint64_t out_stride;
    uint32_t n, rows, ncols;
    uint32_t upt;         // units per tile (blocks along K)
    uint32_t nwarps;      // warps that take work
    uint32_t q, r;        // every warp takes q units, the first r one more
    uint32_t maxp;        // slots per tile in `partial`
    Chain chain;
};

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Which warp owns unit u under the (q, r) split.
__device__ __forceinline__ uint32_t owner_of(uint64_t u, uint32_t q, uint32_t r) {
    const uint64_t head = (uint64_t)r * (q + 1);
    return u < head ? (uint32_t)(u / (q + 1)) : r + (uint32_t)((u - head) / q);
}

// Ends a warp's stretch [first_blk, end_blk) of tile `tile`: either finishes the tile
// or leaves a partial for the last contributor to add up.  acc holds, per 8-column
// MMA tile, (row g, col 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).
template <int NT>
__device__ __forceinline__ void flush_tile(const GemvParams &p, float (&acc)[NT][4], float *patch, uint32_t warp,
                                           uint32_t tile, uint32_t first_blk, uint32_t end_blk) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int W = NT * 8 + 1;  // padded row of the per-warp patch
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        patch[g * W + nt * 8 + 2 * t] = acc[nt][0];
        patch[g * W + nt * 8 + 2 * t + 1] = acc[nt][1];
        patch[(g + 8) * W + nt * 8 + 2 * t] = acc[nt][2];
        patch[(g + 8) * W + nt * 8 + 2 * t + 1] = acc[nt][3];
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    }
    __syncwarp();
    const uint32_t cells = p.rows * 16;
    const bool whole = first_blk == 0 && end_blk == p.upt;
    if (whole) {
        for (uint32_t idx = lane; idx < cells; idx += 32) {
            const uint32_t rr = idx & 15, b = idx >> 4, col = tile * 16 + rr;
            const float v = (patch[rr * W + 3 * b] + patch[rr * W + 3 * b + 1]) + patch[rr * W + 3 * b + 2];
            if (col < p.n) p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, v);
        }
    } else {
        const uint64_t base = (uint64_t)tile * p.upt;
        const uint32_t first = owner_of(base, p.q, p.r), last = owner_of(base + p.upt - 1, p.q, p.r);
        const uint32_t count = last - first + 1, slot = warp - first;
        float *mine = p.partial + ((uint64_t)tile * p.maxp + slot) * cells;
        for (uint32_t idx = lane; idx < cells; idx += 32) {
            const uint32_t rr = idx & 15, b = idx >> 4;
            __stcg(mine + idx, (patch[rr * W + 3 * b] + patch[rr * W + 3 * b + 1]) + patch[rr * W + 3 * b + 2]);
        }
        __threadfence();
        __syncwarp();
        unsigned int seen = 0;
        if (lane == 0) seen = atomicAdd(p.counters + tile, 1u);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (seen == count - 1) {
            __threadfence();
            const float *all = p.partial + (uint64_t)tile * p.maxp * cells;
            for (uint32_t idx = lane; idx < cells; idx += 32) {
                const uint32_t rr = idx & 15, b = idx >> 4, col = tile * 16 + rr;
                float v = 0.0f;
                for (uint32_t s = 0; s < count; ++s) v += __ldcg(all + (uint64_t)s * cells + idx);
                if (col < p.n) p.out[(uint64_t)b * p.out_stride + col] = chained(p.chain, b, col, v);
            }
            if (lane == 0) p.counters[tile] = 0u;
        }
    }
    __syncwarp();
}

// ---------------------------------------------------------------------------------
// Q4_K
// ---------------------------------------------------------------------------------
struct Q4kRegs {
    uint4 h0, h1;  // headers of rows g and g+8
    uint4 q[4];    // nibble groups: (.x,.y) row g, (.z,.w) row g+8
};

__device__ __forceinline__ void q4k_load(Q4kRegs &regs, const uint8_t *unit, uint32_t lane) {
    const uint32_t g = lane >> 2;
    regs.h0 = ld_stream16(unit + g * 16);
    regs.h1 = ld_stream16(unit + (g + 8) * 16);
#pragma unroll
    for (int G = 0; G < 4; ++G) regs.q[G] = ld_stream16(unit + 256 + G * 512 + lane * 16);
}

template <int NT>
__device__ __forceinline__ void q4k_unit(const GemvParams &p, const Q4kRegs &regs, uint32_t sb, float (&acc)[NT][4]) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
    q4k_scales(regs.h0.y, regs.h0.z, regs.h0.w, sc0, mn0);
    q4k_scales(regs.h1.y, regs.h1.z, regs.h1.w, sc1, mn1);
    int qa[NT][4], ma[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) qa[nt][i] = ma[nt][i] = 0;
    const int8_t *dig = p.dig + ((uint64_t)sb * 8 * p.ncols + g) * 32 + t * 8;
#pragma unroll
    for (int G = 0; G < 4; ++G) {
#pragma unroll
        for (int seat = 0; seat < 2; ++seat) {
            const int sub = G * 2 + seat;
            const uint32_t a0 = (regs.q[G].x >> (4 * seat)) & 0x0f0f0f0fu;
            const uint32_t a2 = (regs.q[G].y >> (4 * seat)) & 0x0f0f0f0fu;
            const uint32_t a1 = (regs.q[G].z >> (4 * seat)) & 0x0f0f0f0fu;
            const uint32_t a3 = (regs.q[G].w >> (4 * seat)) & 0x0f0f0f0fu;
            const int s0 = (int)((sc0[sub >> 2] >> (8 * (sub & 3))) & 0xffu);
            const int s1 = (int)((sc1[sub >> 2] >> (8 * (sub & 3))) & 0xffu);
            // the sub-block's min, replicated over the four bytes of an A register
            const uint32_t m0 = __byte_perm(mn0[sub >> 2], 0u, 0x1111u * (sub & 3));
            const uint32_t m1 = __byte_perm(mn1[sub >> 2], 0u, 0x1111u * (sub & 3));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint2 b = make_uint2(0u, 0u);
                if (nt * 8 + g < p.ncols)
                    b = __ldg(reinterpret_cast<const uint2 *>(dig + ((uint64_t)sub * p.ncols + nt * 8) * 32));
                int d[4] = {0, 0, 0, 0};
                mma_u8s8(d, a0, a1, a2, a3, b.x, b.y);
                qa[nt][0] += d[0] * s0;
                qa[nt][1] += d[1] * s0;
                qa[nt][2] += d[2] * s1;
                qa[nt][3] += d[3] * s1;
                mma_u8s8(ma[nt], m0, m1, m0, m1, b.x, b.y);
            }
        }
    }
    // value = (d*sc)*q - dmin*m  (ggml.rs:341-346)  ->  sum = d*sum(sc*q*x) - dmin*sum(m*x)
    const float d0 = half_bits_to_float(regs.h0.x & 0xffffu), n0 = half_bits_to_float(regs.h0.x >> 16);
    const float d1 = half_bits_to_float(regs.h1.x & 0xffffu), n1 = half_bits_to_float(regs.h1.x >> 16);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const uint32_t col = nt * 8 + 2 * t;
        const float c0 = col < p.ncols ? __ldg(p.cs + (uint64_t)sb * p.ncols + col) : 0.0f;
        const float c1 = col + 1 < p.ncols ? __ldg(p.cs + (uint64_t)sb * p.ncols + col + 1) : 0.0f;
        acc[nt][0] = fmaf(d0 * (float)qa[nt][0] - n0 * (float)ma[nt][0], c0, acc[nt][0]);
        acc[nt][1] = fmaf(d0 * (float)qa[nt][1] - n0 * (float)ma[nt][1], c1, acc[nt][1]);
        acc[nt][2] = fmaf(d1 * (float)qa[nt][2] - n1 * (float)ma[nt][2], c0, acc[nt][2]);
        acc[nt][3] = fmaf(d1 * (float)qa[nt][3] - n1 * (float)ma[nt][3], c1, acc[nt][3]);
    }
}

template <int NT>
__global__ void __launch_bounds__(256) gemv_q4k_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ float patches[];
    const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const uint32_t warp = blockIdx.x * (blockDim.x >> 5) + wib;
    if (warp >= p.nwarps) return;
    float *patch = patches + wib * 16 * (NT * 8 + 1);
    const uint64_t u0 = (uint64_t)warp * p.q + min(warp, p.r);
    const uint64_t u1 = u0 + p.q + (warp < p.r ? 1u : 0u);
    uint32_t tile = (uint32_t)(u0 / p.upt), blk = (uint32_t)(u0 % p.upt), first_blk = blk;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    const uint8_t *unit = p.w + u0 * kQ4kUnit;
    Q4kRegs bufa, bufb;
    q4k_load(bufa, unit, lane);
    for (uint64_t u = u0; u < u1; u += 2) {
        if (u + 1 < u1) q4k_load(bufb, unit + kQ4kUnit, lane);
        q4k_unit<NT>(p, bufa, blk, acc);
        if (++blk == p.upt || u + 1 == u1) {
            flush_tile<NT>(p, acc, patch, warp, tile, first_blk, blk);
            if (blk == p.upt) { blk = 0; ++tile; }
            first_blk = blk;
        }
        if (u + 1 < u1) {
            if (u + 2 < u1) q4k_load(bufa, unit + 2 * kQ4kUnit, lane);
            q4k_unit<NT>(p, bufb, blk, acc);
            if (++blk == p.upt || u + 2 == u1) {
                flush_tile<NT>(p, acc, patch, warp, tile, first_blk, blk);
                if (blk == p.upt) { blk = 0; ++tile; }
                first_blk = blk;
            }
        }
        unit += 2 * kQ4kUnit;
    }
}

// ---------------------------------------------------------------------------------
// Q8_0: four blocks of K per step
// ---------------------------------------------------------------------------------
constexpr int kQ8Group = 4;

struct Q8Regs {
    uint4 q[kQ8Group];      // (.x,.y) row g, (.z,.w) row g+8
    uint32_t d[kQ8Group];   // fp16 scales of rows g (low half) and g+8 (high half)
};

// Loads the group of units starting at `u`; units past `last` (the matrix's final
// unit) are clamped onto it, so every lane register is defined by an in-bounds load.
__device__ __forceinline__ void q8_load(Q8Regs &regs, const uint8_t *w, uint64_t u, uint64_t last, uint32_t lane) {
#pragma unroll
    for (int i = 0; i < kQ8Group; ++i) {
        const uint8_t *unit = w + min(u + i, last) * kQ8Unit;
        regs.q[i] = ld_stream16(unit + lane * 16);
        regs.d[i] = ld_stream4(unit + 512 + (lane >> 2) * 4);
    }
}

template <int NT>
__device__ __forceinline__ void q8_unit(const GemvParams &p, const uint4 &q, uint32_t dd, uint32_t blk,
                                        float (&acc)[NT][4]) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const float d0 = half_bits_to_float(dd & 0xffffu), d1 = half_bits_to_float(dd >> 16);
    const int8_t *dig = p.dig + ((uint64_t)blk * p.ncols + g) * 32 + t * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        uint2 b = make_uint2(0u, 0u);
        if (nt * 8 + g < p.ncols) b = __ldg(reinterpret_cast<const uint2 *>(dig + nt * 8 * 32));
        int d[4] = {0, 0, 0, 0};
        mma_s8s8(d, q.x, q.z, q.y, q.w, b.x, b.y);
        const uint32_t col = nt * 8 + 2 * t;
        const float c0 = col < p.ncols ? __ldg(p.cs + (uint64_t)blk * p.ncols + col) : 0.0f;
        const float c1 = col + 1 < p.ncols ? __ldg(p.cs + (uint64_t)blk * p.ncols + col + 1) : 0.0f;
        acc[nt][0] = fmaf((float)d[0], d0 * c0, acc[nt][0]);
        acc[nt][1] = fmaf((float)d[1], d0 * c1, acc[nt][1]);
        acc[nt][2] = fmaf((float)d[2], d1 * c0, acc[nt][2]);
        acc[nt][3] = fmaf((float)d[3], d1 * c1, acc[nt][3]);
    }
}

template <int NT>
__global__ void __launch_bounds__(256) gemv_q8_0_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ float patches[];
    const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const uint32_t warp = blockIdx.x * (blockDim.x >> 5) + wib;
    if (warp >= p.nwarps) return;
    float *patch = patches + wib * 16 * (NT * 8 + 1);
    const uint64_t u0 = (uint64_t)warp * p.q + min(warp, p.r);
    const uint64_t u1 = u0 + p.q + (warp < p.r ? 1u : 0u);
    uint32_t tile = (uint32_t)(u0 / p.upt), blk = (uint32_t)(u0 % p.upt), first_blk = blk;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    const uint64_t last = (uint64_t)((p.n + 15) / 16) * p.upt - 1;
    Q8Regs bufa, bufb;
    q8_load(bufa, p.w, u0, last, lane);
    for (uint64_t u = u0; u < u1; u += 2 * kQ8Group) {
        q8_load(bufb, p.w, u + kQ8Group, last, lane);
#pragma unroll
        for (int i = 0; i < kQ8Group; ++i) {
            if (u + i < u1) {
                q8_unit<NT>(p, bufa.q[i], bufa.d[i], blk, acc);
                if (++blk == p.upt || u + i + 1 == u1) {
                    flush_tile<NT>(p, acc, patch, warp, tile, first_blk, blk);
                    if (blk == p.upt) { blk = 0; ++tile; }
                    first_blk = blk;
                }
            }
        }
        q8_load(bufa, p.w, u + 2 * kQ8Group, last, lane);
#pragma unroll
        for (int i = 0; i < kQ8Group; ++i) {
            if (u + kQ8Group + i < u1) {
                q8_unit<NT>(p, bufb.q[i], bufb.d[i], blk, acc);
                if (++blk == p.upt || u + kQ8Group + i + 1 == u1) {
                    flush_tile<NT>(p, acc, patch, warp, tile, first_blk, blk);
                    if (blk == p.upt) { blk = 0; ++tile; }
                    first_blk = blk;
                }
            }
        }
    }
}

}  // namespace nc
