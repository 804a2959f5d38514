// Row-at-a-time product for Q6_K weights in GGUF order: out[r][c] = chain(sum_k W[c][k] x[r][k]) for up to eight
// activation rows a pass, one warp per weight row, f32 activations and f32 accumulation throughout.
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
