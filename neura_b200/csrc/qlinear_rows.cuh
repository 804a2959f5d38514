// Row-at-a-time products for the weight formats that are multiplied where the GGUF left them (Q6_K, Q5_K, Q3_K, half
// and bfloat16 numbers): out[r][c] = chain(sum_k W[c][k] x[r][k]) for up to eight activation rows a pass, one warp per
// weight row, f32 activations and f32 accumulation throughout.
//
// Q6_K (crates/neura-precision/src/ggml.rs:352-407; the reference's dot is crates/neura-kernel/src/dot.rs:663-797) is
// the format common GGUF mixes keep their heads and embeddings in: 256 numbers in 210 bytes, sixteen runs of 16 with
// an int8 scale each, six-bit codes biased by 32 (four low bits in [0, 128), two high bits in [128, 192), scales in
// [192, 208), d as a half float at 208):  w = d * scale * (code - 32).
// The blocks are read where the GGUF left them (210 is no multiple of 4, so byte loads; a warp's loads of a field are
// consecutive bytes).  Lane l of the warp takes the eight numbers l, 32 + l, ..., 224 + l of a super-block: its four
// code bytes, two high-bit bytes and eight scales.  This is the plain scalar path; the Q8_0 and Q4_K weights of the
// projections go through the streaming kernels.
#pragma once
#include "common.cuh"

namespace nc {

constexpr uint32_t kQ6kBytes = 210;    // crates/neura-abi/src/element.rs:167-170
constexpr uint32_t kQ5kBytes = 176;    // element.rs:163-166: d, dmin, 12 bytes of scales and mins, 32 of fifth bits, 128 of nibbles
constexpr uint32_t kQ3kBytes = 110;    // element.rs:171-174: 32 bytes of third bits, 64 of bit pairs, 12 of scales, d
constexpr uint32_t kRowsKernelMost = 8;   // activation rows one launch carries

struct RowsParams {
    const uint8_t *w;      // GGUF order: row after row of k / 256 blocks
    const float *x;        // [rows][x_stride]
    float *out;            // [rows][out_stride]
    uint64_t x_stride, out_stride;
    uint32_t n, k, rows;
    Chain chain;
};

// One element of q6_k_values, each product rounded on its own: (d * scale) * (code - 32), as the reference's host and
// device decoders compute it (ggml.rs:404, crates/neura-kernel/src/fetch.rs:300).
__device__ __forceinline__ float q6k_value(const uint8_t *block, uint32_t within) {
    const uint32_t half = within / 128, seat = within % 128, group = seat / 32, lane = seat % 32;
    const uint32_t packed = block[half * 64 + (group % 2) * 32 + lane];
    const uint32_t low = group >= 2 ? packed >> 4 : packed & 0x0fu;
    const uint32_t high = (block[128 + half * 32 + lane] >> (2 * group)) & 3u;
    const float scale = (float)(int8_t)block[192 + half * 8 + group * 2 + lane / 16];
    const float d = half_bits_to_float((uint32_t)block[208] | ((uint32_t)block[209] << 8));
    return __fmul_rn(__fmul_rn(d, scale), (float)(low | (high << 4)) - 32.0f);
}

__device__ __forceinline__ float half_at_bytes(const uint8_t *at) {
    return half_bits_to_float((uint32_t)__ldg(at) | ((uint32_t)__ldg(at + 1) << 8));
}

// The six-bit scale and min of sub-block `sub` out of the twelve bytes at `scales` (scale_min_k4, ggml.rs:127-136).
__device__ __forceinline__ void k4_scale_min(const uint8_t *scales, uint32_t sub, uint32_t &scale, uint32_t &min) {
    if (sub < 4) {
        scale = __ldg(scales + sub) & 63u;
        min = __ldg(scales + sub + 4) & 63u;
    } else {
        const uint32_t both = __ldg(scales + sub + 4);
        scale = (both & 0x0fu) | ((uint32_t)(__ldg(scales + sub - 4) >> 6) << 4);
        min = (both >> 4) | ((uint32_t)(__ldg(scales + sub) >> 6) << 4);
    }
}

// One element of q5_k_values (ggml.rs:318-334, crates/neura-kernel/src/fetch.rs:269-282): Q4_K's walk with a fifth bit
// a code; (d * scale) * code - dmin * min, each product rounded on its own.
__device__ __forceinline__ float q5k_value(const uint8_t *block, uint32_t within) {
    const uint32_t group = within / 64, seat = (within % 64) / 32, lane = within % 32, sub = group * 2 + seat;
    uint32_t scale, min;
    k4_scale_min(block + 4, sub, scale, min);
    const uint32_t packed = __ldg(block + 48 + group * 32 + lane);
    const uint32_t code = (seat ? packed >> 4 : packed & 0x0fu) | ((((uint32_t)__ldg(block + 16 + lane) >> sub) & 1u) << 4);
    return __fsub_rn(__fmul_rn(__fmul_rn(half_at_bytes(block), (float)scale), (float)code), __fmul_rn(half_at_bytes(block + 2), (float)min));
}

// One element of q3_k_values (ggml.rs:292-308, fetch.rs:226-254): sixteen runs of 16 with a six-bit scale biased by 32;
// a code is two bits of byte 32 + ... and a third bit that, when clear, takes four off: (d * (scale - 32)) * code.
__device__ __forceinline__ float q3k_value(const uint8_t *block, uint32_t within) {
    const uint32_t half = within / 128, local = within % 128, j = local / 32, seat = local % 32;
    const uint32_t index = half * 8 + j * 2 + seat / 16;
    const uint32_t low_byte = __ldg(block + 96 + index % 8);
    const uint32_t scale = (index >= 8 ? low_byte >> 4 : low_byte & 0x0fu) | ((((uint32_t)__ldg(block + 104 + index % 4) >> (2 * (index / 4))) & 3u) << 4);
    const uint32_t low = ((uint32_t)__ldg(block + 32 + half * 32 + seat) >> (2 * j)) & 3u;
    const bool high = ((uint32_t)__ldg(block + seat) >> (half * 4 + j)) & 1u;
    return __fmul_rn(__fmul_rn(half_at_bytes(block + 108), (float)scale - 32.0f), (float)low - (high ? 0.0f : 4.0f));
}

// Number `at` of a weight row in GGUF order.
template <uint32_t ELEMENT>
__device__ __forceinline__ float gguf_value(const uint8_t *row, uint32_t at) {
    if constexpr (ELEMENT == NC_ELEMENT_Q6K) return q6k_value(row + (uint64_t)(at / kSuperBlock) * kQ6kBytes, at % kSuperBlock);
    else if constexpr (ELEMENT == NC_ELEMENT_Q5K) return q5k_value(row + (uint64_t)(at / kSuperBlock) * kQ5kBytes, at % kSuperBlock);
    else if constexpr (ELEMENT == NC_ELEMENT_Q3K) return q3k_value(row + (uint64_t)(at / kSuperBlock) * kQ3kBytes, at % kSuperBlock);
    else if constexpr (ELEMENT == NC_ELEMENT_HALF) return half_at_bytes(row + 2 * (uint64_t)at);          // fetch.rs:95-98
    else return __uint_as_float(((uint32_t)__ldg(row + 2 * (uint64_t)at) | ((uint32_t)__ldg(row + 2 * (uint64_t)at + 1) << 8)) << 16);   // bfloat16, fetch.rs:100-107
}

// The plain walk for any of these formats: lane l of a weight row's warp takes numbers l, 32 + l, ...
template <uint32_t ELEMENT, int ROWS>
__global__ void __launch_bounds__(256) qlinear_rows_kernel(const __grid_constant__ RowsParams p, uint64_t row_bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; c < p.n; c += warps) {
        const uint8_t *row = p.w + (uint64_t)c * row_bytes;
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.0f;
        for (uint32_t at = lane; at < p.k; at += 32) {
            const float weight = gguf_value<ELEMENT>(row, at);
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (r < (int)p.rows) acc[r] = fmaf(weight, __ldg(p.x + (uint64_t)r * p.x_stride + at), acc[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float total = acc[r];
            for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0 && r < (int)p.rows) p.out[(uint64_t)r * p.out_stride + c] = chained(p.chain, r, c, total);
        }
    }
}

template <int ROWS>
__global__ void __launch_bounds__(256) qlinear_rows_q6k_kernel(const __grid_constant__ RowsParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5, nsb = p.k / kSuperBlock;
    const uint32_t upper = lane >> 4;   // which of the two scales of a 32-number group this lane reads
    for (uint32_t c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; c < p.n; c += warps) {
        const uint8_t *row = p.w + (uint64_t)c * nsb * kQ6kBytes;
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.0f;
        for (uint32_t sb = 0; sb < nsb; ++sb) {
            const uint8_t *block = row + (uint64_t)sb * kQ6kBytes;
            const float d = half_bits_to_float((uint32_t)__ldg(block + 208) | ((uint32_t)__ldg(block + 209) << 8));
            uint32_t codes[2][2], high[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                codes[half][0] = __ldg(block + half * 64 + lane);
                codes[half][1] = __ldg(block + half * 64 + 32 + lane);
                high[half] = __ldg(block + 128 + half * 32 + lane);
            }
            const float *x = p.x + (uint64_t)sb * kSuperBlock + lane;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int group = 0; group < 4; ++group) {
                    const uint32_t packed = codes[half][group & 1];
                    const uint32_t low = group >= 2 ? packed >> 4 : packed & 0x0fu;
                    const uint32_t code = low | (((high[half] >> (2 * group)) & 3u) << 4);
                    const float scale = (float)(int8_t)__ldg(block + 192 + half * 8 + group * 2 + upper);
                    const float weight = (d * scale) * ((float)code - 32.0f);
#pragma unroll
                    for (int r = 0; r < ROWS; ++r)
                        if (r < (int)p.rows) acc[r] = fmaf(weight, __ldg(x + (uint64_t)r * p.x_stride + half * 128 + group * 32), acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float total = acc[r];
            for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0 && r < (int)p.rows) p.out[(uint64_t)r * p.out_stride + c] = chained(p.chain, r, c, total);
        }
    }
}

}  // namespace nc
