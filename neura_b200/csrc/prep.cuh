// Activation staging for the integer-MMA product.
//
// The decode product keeps f32 activations (the reference never quantises them,
// crates/neura-kernel/src/dot.rs:583-619), but a scalar f32 FMA per weight cannot keep
// up with HBM3e on B200 (about three issue slots per Q4_K weight at 6.5 TB/s).  So the
// activations are rewritten once per call as block fixed point: inside each exponent
// granule (256 elements for Q4_K, 32 for Q8_0) x = v * 2^-s with |v| < 2^22, and the
// integer v is split into three balanced base-256 digits v = d0 + 256 d1 + 65536 d2,
// each an int8.  Digit planes are columns of the s8 MMA operand; the integer dot
// products are exact, so the result differs from a sequential f32 sum only by the
// 2^-23 (relative to the granule's peak) rounding of v and by f32 accumulation order.
//
//   granule 32  (Q8_0): dig[kb][col][32]        int8, kb = 32-element block of K, col = 3*row + digit
//   granule 256 (Q4_K): dig[sb][col][t][sub][8] int8, sb = super-block of K, sub = its 32-block,
//                       t = which eight elements of that block (so an MMA lane's 64 bytes are contiguous)
//   cs[gi][col]         f32 2^-s * 256^digit, gi = exponent granule of K
//   granule 256 only:   sums[sb][col][t][4] u32: the B fragments of the two MMAs that take the Q4_K min
//                       term.  S = sum of a sub-block's 32 digits (|S| <= 4096) = S0 + 256 S1 in int8
//                       bytes; word 0 holds S0 of sub-block t in its low byte, word 1 S0 of sub-block
//                       4 + t, words 2 and 3 the same for S1; the other bytes are zero.
#pragma once
#include "common.cuh"
#include "exchange.cuh"

namespace nc {

struct PrepParams {
    const float *x;     // [rows][x_stride]
    uint64_t x_stride;
    int8_t *dig;
    float *cs;
    uint32_t *sums;     // granule 256 only: [sb][col][t] x {low b0, low b1, high b0, high b1}, see below
    uint32_t rows, k, ncols;
    uint32_t granule;   // 256 or 32
    uint32_t vector;    // 1: rows start 16-byte aligned, so a lane may fetch float4
    uint32_t lo, hi;    // the activations are elements [lo, hi) of K (multiples of 32); the rest of K reads as zero
};

// Digitises one 256-element chunk of row `row` held by a warp: lane l owns v[0..8) =
// elements [8l, 8l+8) of the chunk; `live` says whether those elements exist (k is a
// multiple of 32, so a lane is live or dead as a whole).  All 32 lanes must call.
__device__ __forceinline__ void stage_chunk(const PrepParams &p, uint32_t row, uint32_t chunk, const float (&v)[8],
                                            bool live) {
    const uint32_t lane = threadIdx.x & 31;
    float peak = 0.0f;
    bool odd = false;  // an inf or a nan among this lane's numbers
    if (live) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            peak = fmaxf(peak, fabsf(v[i]));
            odd |= !(fabsf(v[i]) <= 3.0e38f);
        }
    }
    // granule peak: 4 lanes share a 32-block, the warp shares the 256-chunk
    peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 1));
    peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 2));
    if (p.granule == 256) {
        peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 4));
        peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 8));
        peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 16));
    }
    // peak < 2^e  ->  |x * 2^(22-e)| < 2^22
    int s = 0;
    float unscale = 1.0f;
    const uint32_t vote = __ballot_sync(0xffffffffu, odd);
    const bool finite = p.granule == 256 ? vote == 0u : ((vote >> (lane & ~3u)) & 0xfu) == 0u;
    if (peak > 0.0f && finite) {
        int e;
        frexpf(peak, &e);
        s = min(max(22 - e, -100), 120);
        unscale = ldexpf(1.0f, -s);
    }
    if (!finite) unscale = __int_as_float(0x7fc00000);  // the product of this granule reads as nan
    const float up = ldexpf(1.0f, s);
    uint32_t d[3][2] = {{0, 0}, {0, 0}, {0, 0}};
    int total[3] = {0, 0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = (finite && live) ? __float2int_rn(v[i] * up) : 0;
        const int d0 = (int)(int8_t)(q & 255);
        q = (q - d0) >> 8;
        const int d1 = (int)(int8_t)(q & 255);
        const int d2 = (q - d1) >> 8;
        total[0] += d0;
        total[1] += d1;
        total[2] += d2;
        d[0][i >> 2] |= (uint32_t)(d0 & 255) << (8 * (i & 3));
        d[1][i >> 2] |= (uint32_t)(d1 & 255) << (8 * (i & 3));
        d[2][i >> 2] |= (uint32_t)(d2 & 255) << (8 * (i & 3));
    }
    const uint32_t kb = chunk * 8 + (lane >> 2);
    if (p.granule == 256) {
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            int sum = total[j];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) {
                const uint32_t sub = lane >> 2, col = row * 3 + j;
                const int s0 = (int)(int8_t)(sum & 255), s1 = (sum - s0) >> 8;
                uint32_t *entry = p.sums + (((uint64_t)chunk * p.ncols + col) * 4 + (sub & 3)) * 4 + (sub >> 2);
                entry[0] = (uint32_t)(s0 & 255);
                entry[2] = (uint32_t)(s1 & 255);
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const uint32_t col = row * 3 + j;
        const uint64_t at = p.granule == 256
            ? ((((uint64_t)chunk * p.ncols + col) * 4 + (lane & 3)) * 8 + (lane >> 2)) * 8
            : ((uint64_t)kb * p.ncols + col) * 32 + (lane & 3) * 8;
        *reinterpret_cast<uint2 *>(p.dig + at) = make_uint2(d[j][0], d[j][1]);
    }
    const bool writes = p.granule == 256 ? lane == 0 : (lane & 3) == 0;
    if (writes) {
        const uint32_t gi = p.granule == 256 ? chunk : kb;
        float c = unscale;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            p.cs[(uint64_t)gi * p.ncols + row * 3 + j] = c;
            c *= 256.0f;
        }
    }
}

// Fetches a lane's eight numbers of a chunk.
__device__ __forceinline__ void load_chunk(const PrepParams &p, uint32_t row, uint32_t at, bool live, float (&v)[8]) {
    if (live && at >= p.lo && at < p.hi) {
        const float *from = p.x + (uint64_t)row * p.x_stride + (at - p.lo);
        // (through L2: a persistent kernel stages activations another SM wrote moments ago)
        if (p.vector) {
            const float4 a = __ldcg(reinterpret_cast<const float4 *>(from));
            const float4 b = __ldcg(reinterpret_cast<const float4 *>(from + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __ldcg(from + i);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
}

// Staging by the producer.  In a persistent kernel the rows a product (or the attention merge) writes are the
// activations of the next product.  Instead of a staging pass of its own, the warp that completes the last
// tile of a 256-column chunk digitises that chunk at once (every chunk has a counter of finished tiles), so
// the next product finds its operand ready after one barrier.  With `gain` the chunk is multiplied by the
// coming rms_norm's weight first and the chunk's sum of squares is left in `sumsq`: the norm's scalar
// 1 / sqrt(mean(x^2) + floor) is applied by the consumer to its outputs (a product is linear in a row scale).
//
// On a rank of a tensor-parallel group two more things ride here.  The produced rows may be a window [lo, hi) of the
// consumer's K axis (a row-parallel weight keeps the whole blocks that cover its share of K): chunks, counters and
// the staged form are in the consumer's coordinates, the rows themselves start at lo.  And the produced rows may be
// partial sums over a share of K (`exchange`): the warp that completes a chunk first adds the ranks' chunks up
// (exchange_chunk), writes the sums back to the rows, and stages those.
struct StageAfter {
    PrepParams prep;         // x = the rows being produced, k = the consumer's K, [lo, hi) = where the rows sit in it
    const float *gain;       // [hi - lo] or null
    float *sumsq;            // [rows][chunks] or null
    unsigned int *counters;  // [rows][chunks] finished pieces, zero between launches
    uint32_t piece;          // columns one arrival covers (a tile's 32, a pair tile's 16)
    const ExchangeView *exchange;   // not null: the rows are this rank's partial sums of a [rows x (hi - lo)] all-reduce
    unsigned long long wait_nanos;  // how long a chunk waits for the peers, and the word raised when that runs out
    unsigned int *status;
};

// Digitises chunk `chunk` of row `row` from the produced values (the whole warp calls).
__device__ __forceinline__ void stage_after_chunk(const StageAfter &a, uint32_t row, uint32_t chunk) {
    const uint32_t lane = threadIdx.x & 31, from = chunk * 256 + lane * 8;
    const bool live = from < a.prep.k;
    float v[8];
    load_chunk(a.prep, row, from, live, v);
    if (a.exchange) {   // the row holds this rank's partial sums: add the ranks' up, keep the sums (lo = 0, whole chunks)
        const uint32_t chunks = a.prep.k / 256;
        if (!exchange_chunk(*a.exchange, row * a.prep.k + from - lane * 8, row * chunks + chunk, a.prep.rows * chunks, v, a.wait_nanos, a.status)) return;
        float *to = const_cast<float *>(a.prep.x) + (uint64_t)row * a.prep.x_stride + from;
        __stcg(reinterpret_cast<float4 *>(to), make_float4(v[0], v[1], v[2], v[3]));
        __stcg(reinterpret_cast<float4 *>(to + 4), make_float4(v[4], v[5], v[6], v[7]));
    }
    if (a.sumsq) {
        float square = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) square = fmaf(v[j], v[j], square);
        for (int o = 16; o; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
        if (lane == 0) __stcg(a.sumsq + row * ((a.prep.k + 255) / 256) + chunk, square);
    }
    if (a.gain && live && from >= a.prep.lo && from < a.prep.hi) {
        const float4 g0 = __ldg(reinterpret_cast<const float4 *>(a.gain + (from - a.prep.lo)));
        const float4 g1 = __ldg(reinterpret_cast<const float4 *>(a.gain + (from - a.prep.lo) + 4));
        v[0] *= g0.x; v[1] *= g0.y; v[2] *= g0.z; v[3] *= g0.w;
        v[4] *= g1.x; v[5] *= g1.y; v[6] *= g1.z; v[7] *= g1.w;
    }
    stage_chunk(a.prep, row, chunk, v, live);
}

// Columns [first, first + a.piece) of every row are final (the whole warp calls, after a __syncwarp that
// follows its stores).  Counts the arrival; the warp that completes a chunk digitises it for all rows.
__device__ __forceinline__ void stage_after_piece(const StageAfter &a, uint32_t first) {
    const uint32_t lane = threadIdx.x & 31;
    first += a.prep.lo;                      // where the piece sits on the consumer's K axis
    if (first >= a.prep.hi) return;
    const uint32_t chunk = first / 256;
    const uint32_t width = min(a.prep.hi, (chunk + 1) * 256) - max(a.prep.lo, chunk * 256);
    const uint32_t expected = (width + a.piece - 1) / a.piece;
    unsigned int seen = 0;
    if (lane == 0) {
        seen = arrive_on(a.counters + chunk);
    }
    seen = __shfl_sync(0xffffffffu, seen, 0);
    if (seen != expected - 1) return;
    for (uint32_t row = 0; row < a.prep.rows; ++row) stage_after_chunk(a, row, chunk);
    if (lane == 0) a.counters[chunk] = 0u;
}

// One warp per (row, 256-element chunk): lane l owns elements [8l, 8l+8) of the chunk.
__global__ void prep_kernel(const __grid_constant__ PrepParams p) {
    // Programmatic dependent launch: the product that follows may start fetching its
    // weights now; the activations this kernel reads must be complete first.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t chunks = (p.k + 255) / 256;
    const uint64_t total = (uint64_t)p.rows * chunks;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t w = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
        const uint32_t row = (uint32_t)(w / chunks), chunk = (uint32_t)(w % chunks);
        const uint32_t at = chunk * 256 + lane * 8;
        const bool live = at < p.k;
        float v[8];
        load_chunk(p, row, at, live, v);
        stage_chunk(p, row, chunk, v, live);
    }
}

// rms_norm (crates/neura-kernel/src/task/norm.rs:55-131, op = NORM_RMS) fused with the staging
// of its result: one CTA per row computes scale = 1 / sqrt(mean(x^2) + floor), then its warps
// digitise x * scale * weight chunk by chunk.  `normed`, when not null, also receives the f32 row.
struct NormStageParams {
    PrepParams prep;
    const float *weight;  // [k] or null
    float *normed;        // [rows][normed_stride] or null
    uint64_t normed_stride;
    float floor;
};

constexpr uint32_t kNormChunksPerWarp = 4;   // 8 warps x 4 chunks x 256 = rows of up to 8192 stay in registers

// One row by one CTA (of at most 32 warps); `partial` holds a float a warp, `scale_shared` one float.
__device__ __forceinline__ void rms_norm_stage_row(const NormStageParams &p, uint32_t row, float *partial, float *scale_shared) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const uint32_t chunks = (p.prep.k + 255) / 256;
    const bool held = chunks <= warps * kNormChunksPerWarp;
    // every load of the row is issued before the first use, so the row costs one memory round trip
    float v[kNormChunksPerWarp][8];
    float square = 0.0f;
    if (held) {
#pragma unroll
        for (uint32_t i = 0; i < kNormChunksPerWarp; ++i) {
            const uint32_t chunk = warp + i * warps, at = chunk * 256 + lane * 8;
            load_chunk(p.prep, row, at, chunk < chunks && at < p.prep.k, v[i]);
        }
#pragma unroll
        for (uint32_t i = 0; i < kNormChunksPerWarp; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) square = fmaf(v[i][j], v[i][j], square);
    } else {
        const float *x = p.prep.x + (uint64_t)row * p.prep.x_stride;
        for (uint32_t c = threadIdx.x; c < p.prep.k; c += blockDim.x) square = fmaf(x[c], x[c], square);
    }
    for (int o = 16; o; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
    if (lane == 0) partial[warp] = square;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (uint32_t w = 0; w < warps; ++w) total += partial[w];
        *scale_shared = 1.0f / sqrtf(total / (float)p.prep.k + p.floor);
    }
    __syncthreads();
    const float scale = *scale_shared;
#pragma unroll
    for (uint32_t i = 0; i < kNormChunksPerWarp; ++i) {
        for (uint32_t chunk = warp + i * warps; chunk < chunks; chunk += held ? chunks : warps * kNormChunksPerWarp) {
            const uint32_t at = chunk * 256 + lane * 8;
            const bool live = at < p.prep.k;
            float w[8];
            if (held) {
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = v[i][j];
            } else {
                load_chunk(p.prep, row, at, live, w);
            }
            if (live) {
                float gain[8];
                if (p.weight) {
                    const float4 a = *reinterpret_cast<const float4 *>(p.weight + at);
                    const float4 c = *reinterpret_cast<const float4 *>(p.weight + at + 4);
                    gain[0] = a.x; gain[1] = a.y; gain[2] = a.z; gain[3] = a.w;
                    gain[4] = c.x; gain[5] = c.y; gain[6] = c.z; gain[7] = c.w;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    w[j] = w[j] * scale;
                    if (p.weight) w[j] = w[j] * gain[j];
                    if (p.normed) p.normed[(uint64_t)row * p.normed_stride + at + j] = w[j];
                }
            }
            stage_chunk(p.prep, row, chunk, w, live);
        }
    }
}

__global__ void __launch_bounds__(1024) rms_norm_stage_kernel(const __grid_constant__ NormStageParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float partial[32];
    __shared__ float scale_shared;
    rms_norm_stage_row(p, blockIdx.x, partial, &scale_shared);
}

}  // namespace nc
