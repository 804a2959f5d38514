// Device packer: f32 -> GGUF blocks, bit-exact with the reference's host packer
// (crates/neura-precision/src/ggml.rs).  Every f32 operation is an explicit
// round-to-nearest intrinsic so that nvcc cannot contract a*b+c into an fma.
#pragma once
#include "common.cuh"

namespace nc {

__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
    for (int o = 16; o; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// f32::round (half away from zero), exact: x - trunc(x) is representable.
__device__ __forceinline__ float round_away(float x) {
    const float whole = truncf(x);
    return fabsf(__fsub_rn(x, whole)) >= 0.5f ? __fadd_rn(whole, copysignf(1.0f, x)) : whole;
}
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

// span() (ggml.rs:110-114) folds `least`/`greatest` from 0.0 in element order, and those
// return their second argument on a tie, so the sign of a zero extreme is the sign of
// the last zero element walked.  These two reproduce that fold across a warp whose lane
// l holds element l: the extreme itself when it is not zero, else that signed zero.
__device__ __forceinline__ float zero_of_last(float v) {
    const uint32_t zeros = __ballot_sync(0xffffffffu, v == 0.0f);
    const uint32_t negative = __ballot_sync(0xffffffffu, signbit(v));
    if (zeros == 0u) return 0.0f;
    return (negative >> (31 - __clz(zeros))) & 1u ? -0.0f : 0.0f;
}
__device__ __forceinline__ float span_low(float v) {
    const float low = warp_min(v);
    const float zero = zero_of_last(v);
    return low < 0.0f ? low : zero;
}
__device__ __forceinline__ float span_high(float v) {
    const float high = warp_max(v);
    const float zero = zero_of_last(v);
    return high > 0.0f ? high : zero;
}

// put_half (ggml.rs:78-80).  The two bytes go out as one 16-bit store (blocks are 2-byte
// aligned): splitting the result of the f32->f16 conversion into two byte stores was
// seen to lose the low byte with nvcc 12.9 at -O3.
__device__ __forceinline__ void store_half(uint8_t *at, float value) {
    *reinterpret_cast<unsigned short *>(at) = __half_as_ushort(__float2half_rn(value));
}

// q8_0 (ggml.rs:201-209): one warp per 32-element block, one lane per element.
__global__ void quantize_q8_0_kernel(const float *src, uint8_t *dst, uint64_t blocks) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t b = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        const float v = src[b * kQ8Block + lane];
        const float size = warp_max(fabsf(v));
        const float quantum = __fdiv_rn(size, 127.0f);
        const float inverse = quantum == 0.0f ? 0.0f : __fdiv_rn(1.0f, quantum);
        const float code = clampf(round_away(__fmul_rn(v, inverse)), -127.0f, 127.0f);
        uint8_t *field = dst + b * kQ8Bytes;
        if (lane == 0) store_half(field, quantum);
        field[2 + lane] = (uint8_t)(int8_t)(int)code;
    }
}

// affine_block with steps = 15, sub = 32 (ggml.rs:149-199, :314-316): one warp per
// super-block; lane l holds element l of each of the eight sub-blocks.
__global__ void quantize_q4k_kernel(const float *src, uint8_t *dst, uint64_t blocks) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t b = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        float v[8], lows[8], quantums[8];
        float widest = 0.0f, deepest = 0.0f;
#pragma unroll
        for (int at = 0; at < 8; ++at) {
            v[at] = src[b * kSuperBlock + at * 32 + lane];
            const float low = span_low(v[at]);
            const float high = span_high(v[at]);
            lows[at] = 0.0f < low ? 0.0f : low;  // least(0.0, low)
            quantums[at] = __fdiv_rn(__fsub_rn(high, lows[at]), 15.0f);
            widest = widest > quantums[at] ? widest : quantums[at];  // greatest() keeps the newcomer on a tie
            deepest = deepest > -lows[at] ? deepest : -lows[at];
        }
        const float scale = __fdiv_rn(widest, 63.0f);
        const float min = __fdiv_rn(deepest, 63.0f);
        uint32_t codes[8], mins[8];
#pragma unroll
        for (int at = 0; at < 8; ++at) {
            const float c = scale == 0.0f ? 0.0f : __fdiv_rn(quantums[at], scale);
            const float m = min == 0.0f ? 0.0f : __fdiv_rn(-lows[at], min);
            codes[at] = (uint32_t)clampf(round_away(c), 0.0f, 63.0f);
            mins[at] = (uint32_t)clampf(round_away(m), 0.0f, 63.0f);
        }
        uint8_t *field = dst + b * kQ4kBytes;
        if (lane < 12) {  // put_scale_min_k4 (ggml.rs:138-147), byte `lane` of the twelve
            uint32_t byte;
            if (lane < 4) byte = codes[lane] | ((codes[lane + 4] >> 4) << 6);
            else if (lane < 8) byte = mins[lane - 4] | ((mins[lane] >> 4) << 6);
            else byte = (codes[lane - 4] & 0x0f) | ((mins[lane - 4] & 0x0f) << 4);
            field[4 + lane] = (uint8_t)byte;
        } else if (lane == 12) {
            store_half(field, scale);
        } else if (lane == 13) {
            store_half(field + 2, min);
        }
#pragma unroll
        for (int group = 0; group < 4; ++group) {
            uint32_t byte = 0;
#pragma unroll
            for (int seat = 0; seat < 2; ++seat) {
                const int at = group * 2 + seat;
                // the nibble is taken with the unrounded f32 scale and min (ggml.rs:184-187)
                const float quantum = __fmul_rn(scale, (float)codes[at]);
                const float low = __fmul_rn(min, (float)mins[at]);
                uint32_t code = 0;
                if (quantum != 0.0f)
                    code = (uint32_t)clampf(round_away(__fdiv_rn(__fadd_rn(v[at], low), quantum)), 0.0f, 15.0f);
                byte |= (code & 0x0f) << (seat ? 4 : 0);
            }
            field[16 + group * 32 + lane] = (uint8_t)byte;
        }
    }
}

}  // namespace nc
