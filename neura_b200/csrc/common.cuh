// Shared device helpers: block geometry, fp16 access, the fused pointwise chain.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/neura_cuda.h"

namespace nc {

constexpr uint32_t kQ8Block = 32;       // crates/neura-abi/src/element.rs:35
constexpr uint32_t kQ8Bytes = 34;       // element.rs:155-158
constexpr uint32_t kSuperBlock = 256;   // element.rs:36
constexpr uint32_t kQ4kBytes = 144;     // element.rs:159-162
constexpr uint32_t kTileRows = 32;      // rows of one tile of the sealed layout: two m16n8k32 MMA tiles
constexpr uint32_t kQ4kUnit = 16 * kQ4kBytes;  // 2304 B: 16 rows x one super-block (half a unit)
constexpr uint32_t kQ8Unit = 16 * kQ8Bytes;    // 544 B: 16 rows x one block (half a unit)

// Fused epilogue, passed by value to kernels.
struct Chain {
    uint32_t n;
    nc_step step[NC_MAX_STEPS];
};

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// The transcendental ops of the table, kept out of line: their slow paths need a
// stack frame that the streaming loops should not carry.
__device__ __noinline__ float op_apply_rare(uint32_t op, float a, float b) {
    switch (op) {
    case NC_OP_EXP: return expf(a);
    case NC_OP_LOG: return logf(a);
    case NC_OP_TANH: return tanhf(a);
    case NC_OP_SIN: return sinf(a);
    case NC_OP_COS: return cosf(a);
    case NC_OP_POW: return powf(a, b);
    case NC_OP_GELU: {
        float inner = 0.7978845608f * (a + 0.044715f * a * a * a);
        return 0.5f * a * (1.0f + tanhf(inner));
    }
    default: return a;
    }
}

// op_apply of the reference's pointwise table (crates/neura-pointwise/src/op.rs:141-170).
__device__ __forceinline__ float op_apply(uint32_t op, float a, float b) {
    switch (op) {
    case NC_OP_ADD: return a + b;
    case NC_OP_MUL: return a * b;
    case NC_OP_SUB: return a - b;
    case NC_OP_DIV: return a / b;
    case NC_OP_MAXIMUM: return fmaxf(a, b);
    case NC_OP_MINIMUM: return fminf(a, b);
    case NC_OP_RELU: return fmaxf(a, 0.0f);
    case NC_OP_SQRT: return sqrtf(a);
    case NC_OP_RECIP: return 1.0f / a;
    case NC_OP_SIGMOID: return sigmoid_f(a);
    case NC_OP_NEG: return -a;
    case NC_OP_ABS: return fabsf(a);
    case NC_OP_IDENTITY: return a;
    case NC_OP_FLOOR: return floorf(a);
    case NC_OP_SILU: return a * sigmoid_f(a);
    default: return op_apply_rare(op, a, b);
    }
}

// `chained` (crates/neura-kernel/src/pointwise.rs:90-104) at output coordinate (row, col).
__device__ __forceinline__ float chained(const Chain &chain, uint64_t row, uint64_t col, float carried) {
    float result = carried;
    for (uint32_t s = 0; s < chain.n; ++s) {
        const nc_step &step = chain.step[s];
        // read through L2: in a persistent kernel the operand may have been rewritten by another SM
        float operand = step.operand_dev
            ? __ldcg(step.operand_dev + ((int64_t)row * step.row_stride + (int64_t)col * step.col_stride))
            : 0.0f;
        result = step.swapped ? op_apply(step.op, operand, result) : op_apply(step.op, result, operand);
    }
    return result;
}

// An arrival on a counter of finished pieces: one atomic that releases the arriving thread's earlier writes (and,
// through the barrier before it, its warp's or CTA's) and acquires those of the arrivals before it.  Two fences
// around a relaxed atomic say the same and cost two more trips to L2.
__device__ __forceinline__ unsigned int arrive_on(unsigned int *counter) {
    unsigned int before;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(before) : "l"(counter) : "memory");
    return before;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)bits16));
}

// Streaming 16-byte load that does not displace the activation digits kept in L1.
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream4(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Q4_K 6-bit scale/min unpack (crates/neura-precision/src/ggml.rs:127-136) on the
// three 32-bit words of the 12 scale bytes: returns sc[0..3], sc[4..7], m[0..3], m[4..7]
// as one byte per sub-block.
__device__ __forceinline__ void q4k_scales(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t (&sc)[2],
                                           uint32_t (&mn)[2]) {
    sc[0] = u0 & 0x3f3f3f3fu;
    mn[0] = u1 & 0x3f3f3f3fu;
    sc[1] = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
    mn[1] = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
}

}  // namespace nc
