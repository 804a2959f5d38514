// Weight layouts: the verbatim GGUF order, the tiled order the MMA kernels stream,
// the seal kernel that turns the first into the second, and the bit-exact dequantiser.
//
// Tiled layout (NC_LAYOUT_TILED).  Rows are grouped in tiles of 32 (padded with zero
// rows); a tile's blocks follow each other along K, tile after tile, so the whole
// matrix is one contiguous stream of units of 32 rows x 1 block.  A unit is two halves
// of 16 rows (rows 0-15, then rows 16-31), each laid out for one m16n8k32 MMA tile:
//   Q4_K half = 16 rows x 1 super-block = 2304 B
//     [0, 256)    16 headers of 16 B (d, dmin, 12 scale bytes), row i at 16*i
//     [256, 2304) 4 nibble groups x 32 lanes x 16 B; lane (g = lane/4, t = lane%4) of
//                 group G holds bytes [16+32G+8t, +8) of row g, then the same of row g+8
//   Q8_0 half = 16 rows x 1 block = 544 B
//     [0, 512)    32 lanes x 16 B: quants [8t, +8) of row g, then of row g+8
//     [512, 544)  8 pairs of fp16 scales: (row g, row g+8) at 512 + 4g
// A unit is one contiguous run of bytes (a bulk copy moves it), and once it sits in
// shared memory every lane reads exactly the A-fragment bytes of mma.m16n8k32 (rows g
// and g+8, eight K values) with conflict-free 16-byte loads.
#pragma once
#include "common.cuh"
#include "qlinear_rows.cuh"

namespace nc {

struct WeightView {
    const uint8_t *data;
    uint32_t element, layout, n, k;
};

// Byte `o` of block `blk` of row `row`.
__device__ __forceinline__ uint32_t weight_byte(const WeightView &w, uint32_t row, uint32_t blk, uint32_t o) {
    if (w.element == NC_ELEMENT_Q4K) {
        const uint32_t nsb = w.k / kSuperBlock;
        if (w.layout == NC_LAYOUT_GGUF) return w.data[((uint64_t)row * nsb + blk) * kQ4kBytes + o];
        const uint32_t tile = row / 32, half = (row % 32) / 16, rr = row % 16, g = rr % 8, hi = rr / 8;
        const uint64_t unit = (((uint64_t)tile * nsb + blk) * 2 + half) * kQ4kUnit;
        if (o < 16) return w.data[unit + rr * 16 + o];
        const uint32_t qo = o - 16, G = qo / 32, r32 = qo % 32, t = r32 / 8, i = r32 % 8;
        return w.data[unit + 256 + G * 512 + (g * 4 + t) * 16 + hi * 8 + i];
    }
    const uint32_t nblk = w.k / kQ8Block;
    if (w.layout == NC_LAYOUT_GGUF) return w.data[((uint64_t)row * nblk + blk) * kQ8Bytes + o];
    const uint32_t tile = row / 32, half = (row % 32) / 16, rr = row % 16, g = rr % 8, hi = rr / 8;
    const uint64_t unit = (((uint64_t)tile * nblk + blk) * 2 + half) * kQ8Unit;
    if (o < 2) return w.data[unit + 512 + g * 4 + hi * 2 + o];
    const uint32_t qo = o - 2, t = qo / 8, i = qo % 8;
    return w.data[unit + (g * 4 + t) * 16 + hi * 8 + i];
}

// One element of unpack: q8_0_values / q4_k_values (crates/neura-precision/src/ggml.rs:211-216,
// :336-350).  Each product is rounded to f32 on its own (no fma), which is what makes it bit-exact.
__device__ __forceinline__ float dequant_at(const WeightView &w, uint32_t row, uint32_t at) {
    // the formats kept in GGUF order only
    if (w.element == NC_ELEMENT_Q6K) return gguf_value<NC_ELEMENT_Q6K>(w.data + (uint64_t)row * (w.k / kSuperBlock) * kQ6kBytes, at);
    if (w.element == NC_ELEMENT_Q5K) return gguf_value<NC_ELEMENT_Q5K>(w.data + (uint64_t)row * (w.k / kSuperBlock) * kQ5kBytes, at);
    if (w.element == NC_ELEMENT_Q3K) return gguf_value<NC_ELEMENT_Q3K>(w.data + (uint64_t)row * (w.k / kSuperBlock) * kQ3kBytes, at);
    if (w.element == NC_ELEMENT_HALF) return gguf_value<NC_ELEMENT_HALF>(w.data + (uint64_t)row * w.k * 2, at);
    if (w.element == NC_ELEMENT_BFLOAT16) return gguf_value<NC_ELEMENT_BFLOAT16>(w.data + (uint64_t)row * w.k * 2, at);
    if (w.element == NC_ELEMENT_Q8_0) {
        const uint32_t blk = at / kQ8Block, lane = at % kQ8Block;
        const float quantum = half_bits_to_float(weight_byte(w, row, blk, 0) | (weight_byte(w, row, blk, 1) << 8));
        return __fmul_rn((float)(int8_t)weight_byte(w, row, blk, 2 + lane), quantum);
    }
    const uint32_t blk = at / kSuperBlock, within = at % kSuperBlock;
    const uint32_t group = within / 64, seat = (within % 64) / 32, lane = within % 32;
    const uint32_t sub = group * 2 + seat;
    const float scale = half_bits_to_float(weight_byte(w, row, blk, 0) | (weight_byte(w, row, blk, 1) << 8));
    const float min = half_bits_to_float(weight_byte(w, row, blk, 2) | (weight_byte(w, row, blk, 3) << 8));
    uint32_t code, offset;  // scale_min_k4, ggml.rs:127-136
    if (sub < 4) {
        code = weight_byte(w, row, blk, 4 + sub) & 63u;
        offset = weight_byte(w, row, blk, 4 + sub + 4) & 63u;
    } else {
        code = (weight_byte(w, row, blk, 4 + sub + 4) & 0x0fu) | ((weight_byte(w, row, blk, 4 + sub - 4) >> 6) << 4);
        offset = (weight_byte(w, row, blk, 4 + sub + 4) >> 4) | ((weight_byte(w, row, blk, 4 + sub) >> 6) << 4);
    }
    const uint32_t packed = weight_byte(w, row, blk, 16 + group * 32 + lane);
    const uint32_t quant = seat ? packed >> 4 : packed & 0x0fu;
    const float quantum = __fmul_rn(scale, (float)code);
    const float low = __fmul_rn(min, (float)offset);
    return __fsub_rn(__fmul_rn(quantum, (float)quant), low);
}

__global__ void dequant_kernel(WeightView w, float *out) {
    const uint64_t total = (uint64_t)w.n * w.k;
    for (uint64_t e = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; e < total;
         e += (uint64_t)gridDim.x * blockDim.x)
        out[e] = dequant_at(w, (uint32_t)(e / w.k), (uint32_t)(e % w.k));
}

// GGUF -> tiled, Q4_K, one 8-byte granule per thread step.
// With `second` not null the output pairs two matrices: half 0 of tile T holds rows [16T, 16T+16) of
// `gguf`, half 1 the same rows of `second` (n counts the rows of each).
__global__ void seal_q4k_kernel(const uint8_t *gguf, const uint8_t *second, uint8_t *dst, uint32_t n, uint32_t nsb,
                                uint64_t granules) {
    for (uint64_t d = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; d < granules;
         d += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t unit = d / 576;
        const uint32_t half = (uint32_t)(d % 576) / 288, within = (uint32_t)(d % 288);
        const uint32_t tile = (uint32_t)(unit / nsb), sb = (uint32_t)(unit % nsb);
        uint32_t rr, o;
        if (within < 32) {
            rr = within / 2;
            o = (within % 2) * 8;
        } else {
            const uint32_t q = within - 32, G = q / 64, lane = (q % 64) / 2, hi = q % 2;
            rr = lane / 4 + 8 * hi;
            o = 16 + 32 * G + 8 * (lane % 4);
        }
        const uint32_t row = second ? tile * 16 + rr : tile * 32 + half * 16 + rr;
        const uint8_t *from = second && half ? second : gguf;
        uint2 v = make_uint2(0u, 0u);
        if (row < n) v = *reinterpret_cast<const uint2 *>(from + ((uint64_t)row * nsb + sb) * kQ4kBytes + o);
        *reinterpret_cast<uint2 *>(dst + d * 8) = v;
    }
}

// GGUF -> tiled, Q8_0, one 2-byte granule per thread step (34-byte blocks are only 2-byte aligned).
__global__ void seal_q8_0_kernel(const uint8_t *gguf, const uint8_t *second, uint8_t *dst, uint32_t n, uint32_t nblk,
                                 uint64_t granules) {
    for (uint64_t d = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; d < granules;
         d += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t unit = d / 544;
        const uint32_t half = (uint32_t)(d % 544) / 272, within = (uint32_t)(d % 272);
        const uint32_t tile = (uint32_t)(unit / nblk), blk = (uint32_t)(unit % nblk);
        uint32_t rr, o;
        if (within < 256) {
            const uint32_t b = within * 2, lane = b / 16, rem = b % 16;
            rr = lane / 4 + 8 * (rem / 8);
            o = 2 + 8 * (lane % 4) + rem % 8;
        } else {
            const uint32_t s = within - 256;
            rr = s / 2 + 8 * (s % 2);
            o = 0;
        }
        const uint32_t row = second ? tile * 16 + rr : tile * 32 + half * 16 + rr;
        const uint8_t *from = second && half ? second : gguf;
        unsigned short v = 0;
        if (row < n)
            v = *reinterpret_cast<const unsigned short *>(from + ((uint64_t)row * nblk + blk) * kQ8Bytes + o);
        *reinterpret_cast<unsigned short *>(dst + d * 2) = v;
    }
}

}  // namespace nc
