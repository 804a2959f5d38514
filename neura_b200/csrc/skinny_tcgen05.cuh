// Skinny product on the 5th-generation tensor cores: out[r][c] = chain(sum_k W[c][k] x[r][k]) for 9 to 32
// activation rows against a sealed Q4_K weight, the weight streamed ONCE from HBM for all the rows.
//
// This stands in for the reference's staged-run tiles (template_run_matmul_codes and its codes panel,
// crates/neura-kernel/src/task/matmul.rs:1083-1221, crates/neura-kernel/src/dot.rs:275-350): weights decoded once
// per tile into shared memory and reused by every activation row.  The reference keeps f32 activations; so does
// this kernel to within 2^-22 of each 256-element stretch's peak (below), which leaves f32 accumulation order as the
// only difference that shows at the 1e-3 bar.
//
// Arithmetic.  A Q4_K weight is (d * sc) * q - dmin * m (crates/neura-precision/src/ggml.rs:341-346) with q a
// nibble, sc and m six-bit integers per 32-element sub-block and d, dmin half floats per 256-element super-block.
// So   sum_k w_k x_k = sum_sb d_sb * sum_{k in sb} (sc q)_k x_k  -  sum_sb sum_sub (dmin_sb m_sub) * (sum of x over the sub-block).
//   * First sum, A operand: sc * q as a half float (an integer below 1024: exact), 128 weight rows x 128 k per
//     stage, written by the producers straight into tensor memory (tcgen05.st: lane = weight row, a column = two
//     consecutive half floats of K) and read from there by the MMA, so the operand never crosses shared memory.
//     B operand: the activations as half floats.  Each 256-element stretch of a row is scaled by a power of
//     two so that its peak lies in [2^13, 2^14) and split x = hi + lo * 2^-11, hi = fp16(x), lo = fp16((x - hi) * 2^11):
//     22 bits of the peak.  hi rows and lo rows are stacked along the MMA's N dimension (N = 2 x rows, padded to 16),
//     so one MMA serves both.  tcgen05.mma kind::f16 accumulates in f32 in tensor memory; products of integers below
//     2^11 with 11-bit half floats are exact.  After every super-block the accumulator (two, used in turn) is read
//     back and acc += 2^-e * d * D1 in f32 registers: d and the stretch's scale never meet a half float.
//   * Second sum, after the last super-block of an item: a few more stages whose A rows hold dmin * m of eight
//     super-blocks a stage, each as two half floats h1 + h2 (dmin has 11 significant bits, m six: the split is
//     exact), and whose B rows hold the sub-block sums of the row, scaled by one power of two per row and split hi + lo
//     like the activations.  They accumulate into a third accumulator that is read once per item.
//
// Roles of a CTA (one per SM, persistent over (128-row tile, K slice) items):
//   warps 0-15  producers, a thread per (weight row, 128-k stage of every other super-block): wait for a super-block of
//               raw units in the raw ring, turn the row's 64 quant bytes into 128 values sc * q (two weights per
//               instruction: the nibble is or-ed into the mantissa of 1024, one HFMA2 multiplies by sc and takes the
//               1024 sc away; the half-float constants of a scale come from a 64-entry table in shared memory) and
//               store them into the 64 columns of a tensor-memory stage;
//   warps 16-19 epilogue: read the accumulator of a finished super-block (tcgen05.ld), scale, add up; at the end of
//               an item take the second sum away, apply the fused chain and store, or leave a partial for the last
//               slice to arrive;
//   warp 20     one thread issues the MMAs;  warp 21: one thread asks the tensor memory accelerator for the activation
//               tiles (a ring of their own: a load's latency is several stages long);  warp 22: one thread issues the
//               bulk copies of the raw weight units into a ring of four super-blocks (asking later ones into L2 as well made
//               the kernel slower).
// Tensor memory: four A stages of 64 columns, then two accumulators of the first sum and one of the second (N columns
// each).  A stage is 128 k because the cost of a stage is mostly fixed: the waits, the fences, the arrival and, for the
// one thread that issues MMAs, its own instruction stream.
// Every wait is bounded; a wait that runs out raises the status word, and the CTA still frees its tensor memory.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm_tcgen05.cuh"
#include "gemv_mma.cuh"

namespace nc {

constexpr uint32_t kSkTileRows = 128;                   // weight rows of one item: the M of the MMA
constexpr uint32_t kSkMaxRows = 32;                     // activation rows one launch carries
constexpr uint32_t kSkStageCols = 64;                   // a stage of the A operand in tensor memory: 128 k as half floats, two to a column
constexpr uint32_t kSkStages = 4;
constexpr uint32_t kSkAccAt = kSkStages * kSkStageCols; // the accumulators follow the A stages
constexpr uint32_t kSkTmemCols = 512;                   // 256 columns of A stages + three accumulators of at most 64
constexpr uint32_t kSkRawStage = 4 * kQ4kStage;         // 18 KiB: the four 32-row units of one super-block
constexpr uint32_t kSkRawStages = 4;
constexpr uint32_t kSkXRing = 60 * 1024;                // activation tiles: a ring of their own
constexpr uint32_t kSkXStagesMost = 8;
constexpr uint32_t kSkProducerWarps = 16, kSkEpilogueWarp0 = 16, kSkMmaWarp = 20, kSkTmaWarp = 21, kSkRawWarp = 22;
constexpr uint32_t kSkThreads = 23 * 32;
constexpr uint32_t kSkBarriers = 2 * kSkStages + 2 * kSkXStagesMost + 2 * kSkRawStages + 6;

__host__ __device__ constexpr uint32_t skinny_x_stages(uint32_t bpad) {
    return kSkXRing / (2u * bpad * 256u) < kSkXStagesMost ? kSkXRing / (2u * bpad * 256u) : kSkXStagesMost;
}
__host__ __device__ inline uint32_t skinny_smem_bytes(uint32_t bpad) {
    return 1024u + skinny_x_stages(bpad) * 2u * bpad * 256u + kSkRawStages * kSkRawStage + kSkBarriers * 8u + 64u;
}
// Columns of the table of sub-block sums: 16 a super-block, padded so that every 128-column stage lies inside.
__host__ __device__ inline uint32_t skinny_sx_cols(uint32_t nsb) { return (nsb * 16u + 127u) / 128u * 128u; }

struct SkinnyParams {
    CUtensorMap x_map;        // half floats [2 bpad][k]: hi rows, then lo rows; boxes of 64 columns x 2 bpad rows
    CUtensorMap sx_map;       // half floats [2 bpad][sx_cols]: per super-block its 8 sub-block sums, each twice
    const uint8_t *w;         // sealed Q4_K weight (tiled, or a tiled pair)
    const float *xs;          // [nsb][bpad]: 2^-e of every 256-element stretch of every row
    const float *rs;          // [bpad]: 2^-e of every row's sub-block sums
    float *out;
    uint64_t out_stride;
    float *partial;           // [items][bpad][128]: sums of a K slice, when the K axis is split
    unsigned int *counters;   // [tiles of 128 rows][4]: slices arrived, zero between launches
    unsigned int *status;
    uint32_t n;               // output features (of each tensor of a pair)
    uint32_t rows, bpad;      // activation rows, and rows padded to a multiple of 8
    uint32_t nsb;             // super-blocks along K
    uint32_t tiles32;         // 32-row tiles the weight holds
    uint32_t ntile128, splits;
    uint32_t pair;            // 1: 16 gate rows over 16 up rows per 32-row tile, output = silu(gate) * up
    Chain chain;
#ifdef NC_SKINNY_TRACE
    unsigned long long *trace;   // [role][event] timestamps of CTA 0 (a development build only)
#endif
};

#ifdef NC_SKINNY_TRACE
#define SK_TRACE(role, index) do { if (blockIdx.x == 0 && (index) < 256) p.trace[(role) * 256 + (index)] = global_nanos(); } while (0)
#else
#define SK_TRACE(role, index) do { } while (0)
#endif

// ---- activation staging --------------------------------------------------------------------------------
struct SkinnyPrepParams {
    const float *x;           // [rows][x_stride]: elements [lo, hi) of the K axis
    uint64_t x_stride;
    __half *xh;               // [2 bpad][k]
    __half *sx;               // [2 bpad][sx_cols]
    float *xs;                // [nsb][bpad]
    float *rs;                // [bpad]
    uint32_t rows, bpad, k, sx_cols;
    uint32_t lo, hi;          // the rows hold elements [lo, hi) of K; the rest of K reads as zero
    uint32_t vector;          // 1: rows start 16-byte aligned
    const float *gain;        // rms_norm first: y = x / sqrt(mean(x^2) + floor) * gain (gain may be null with norm set)
    uint32_t norm;
    float floor;
    float *normed;            // when not null also receives y as f32
    uint64_t normed_stride;
};

// Position p of every eight numbers along K, in the A operand and in the B tiles alike, holds element kSkChunkOrder[p]
// of the eight (skinny_scaled says why).
__device__ constexpr int kSkChunkOrder[8] = {0, 2, 1, 3, 4, 6, 5, 7};
constexpr uint32_t kSkPrepSums = 2048;   // sub-block sums of a row kept in shared memory: rows of up to 65536 numbers

__device__ __forceinline__ void split_half(float value, __half &hi, __half &lo) {
    hi = __float2half_rn(value);
    lo = __float2half_rn((value - __half2float(hi)) * 2048.0f);
}

// One CTA per activation row; a warp per 256-element stretch (in turn, where the row has more stretches than the CTA
// has warps: the launch takes up to 32 warps, so rows of up to 8192 numbers go through in one round).
__global__ void __launch_bounds__(1024) skinny_prep_kernel(const __grid_constant__ SkinnyPrepParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float partial[32];
    __shared__ float shared_scalar;
    __shared__ float sums[kSkPrepSums];
    const uint32_t row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float *x = p.x + (uint64_t)row * p.x_stride;
    float scale = 1.0f;
    if (p.norm) {   // rms_norm (crates/neura-kernel/src/task/norm.rs:55-131) of the row before it is staged
        float square = 0.0f;
        for (uint32_t c = threadIdx.x; c < p.hi - p.lo; c += blockDim.x) {
            const float v = __ldcg(x + c);
            square = fmaf(v, v, square);
        }
        for (int o = 16; o; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
        if (lane == 0) partial[warp] = square;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.0f;
            for (uint32_t w = 0; w < warps; ++w) total += partial[w];
            shared_scalar = 1.0f / sqrtf(total / (float)(p.hi - p.lo) + p.floor);
        }
        __syncthreads();
        scale = shared_scalar;
        __syncthreads();
    }
    const uint32_t nsb = p.k / kSuperBlock;
    float largest = 0.0f;   // of this thread's sub-block sums
    bool wild = false;      // an inf or a nan anywhere in the row
    for (uint32_t sb = warp; sb < nsb; sb += warps) {
        const uint32_t at = sb * kSuperBlock + lane * 8;
        float v[8];
        if (at >= p.lo && at < p.hi) {
            const float *from = x + (at - p.lo);
            if (p.vector) {
                const float4 a = __ldcg(reinterpret_cast<const float4 *>(from));
                const float4 b = __ldcg(reinterpret_cast<const float4 *>(from + 4));
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __ldcg(from + i);
            }
            if (p.norm) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] *= scale;
                    if (p.gain) v[i] *= __ldg(p.gain + (at - p.lo) + i);
                    if (p.normed) p.normed[(uint64_t)row * p.normed_stride + (at - p.lo) + i] = v[i];
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        float peak = 0.0f, sum = 0.0f;
        bool odd = false;   // an inf or a nan
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            peak = fmaxf(peak, fabsf(v[i]));
            odd |= !(fabsf(v[i]) <= 3.0e38f);
            sum += v[i];
        }
        for (int o = 16; o; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
        const bool finite = __ballot_sync(0xffffffffu, odd) == 0u;
        wild |= !finite;
        int e = 0;
        if (peak > 0.0f && finite) {
            int ex;
            frexpf(peak, &ex);            // peak = f * 2^ex, f in [0.5, 1)
            e = min(max(14 - ex, -100), 120);
        }
        const float up = ldexpf(1.0f, e);
        float down = ldexpf(1.0f, -e);
        if (!finite) down = __int_as_float(0x7fc00000);   // the products of this stretch read as nan
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {   // (the order within a chunk of eight is the weight side's: kSkChunkOrder)
            __half ha, la, hb, lb;
            split_half(finite ? v[kSkChunkOrder[i]] * up : 0.0f, ha, la);
            split_half(finite ? v[kSkChunkOrder[i + 1]] * up : 0.0f, hb, lb);
            hi[i / 2] = (uint32_t)__half_as_ushort(ha) | ((uint32_t)__half_as_ushort(hb) << 16);
            lo[i / 2] = (uint32_t)__half_as_ushort(la) | ((uint32_t)__half_as_ushort(lb) << 16);
        }
        *reinterpret_cast<uint4 *>(p.xh + (uint64_t)row * p.k + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4 *>(p.xh + (uint64_t)(p.bpad + row) * p.k + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        // sums of the eight sub-blocks (four lanes each)
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) {
            sums[sb * 8 + (lane >> 2)] = finite ? sum : 0.0f;
            largest = fmaxf(largest, fabsf(sum));
        }
        if (lane == 0) p.xs[sb * p.bpad + row] = down;
    }
    // one power of two for the row's sub-block sums, then each sum as hi + lo, twice in a row (the weight side holds
    // dmin * m as two half floats)
    for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
    const uint32_t any_wild = __ballot_sync(0xffffffffu, wild);
    if (lane == 0) partial[warp] = any_wild ? __int_as_float(0x7f800000) : largest;
    __syncthreads();
    if (threadIdx.x == 0) {
        float top = 0.0f;
        for (uint32_t w = 0; w < warps; ++w) top = fmaxf(top, partial[w]);
        int e = 0;
        if (top > 0.0f && top <= 3.0e38f) {
            int ex;
            frexpf(top, &ex);
            e = min(max(14 - ex, -100), 120);
        }
        shared_scalar = ldexpf(1.0f, e);
        p.rs[row] = top <= 3.0e38f ? ldexpf(1.0f, -e) : __int_as_float(0x7fc00000);
    }
    __syncthreads();
    const float up = shared_scalar;
    __half *hi_row = p.sx + (uint64_t)row * p.sx_cols, *lo_row = p.sx + (uint64_t)(p.bpad + row) * p.sx_cols;
    for (uint32_t j = threadIdx.x; j < p.sx_cols / 2; j += blockDim.x) {
        __half h = __ushort_as_half(0), l = __ushort_as_half(0);
        if (j < nsb * 8) split_half(sums[j] * up, h, l);
        const uint32_t hh = (uint32_t)__half_as_ushort(h), ll = (uint32_t)__half_as_ushort(l);
        reinterpret_cast<uint32_t *>(hi_row)[j] = hh | (hh << 16);
        reinterpret_cast<uint32_t *>(lo_row)[j] = ll | (ll << 16);
    }
}

// ---- tensor-memory reads of eight columns -----------------------------------------------------------------
__device__ __forceinline__ void tmem_load_8(uint32_t address, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(address)
                 : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Instruction descriptor: half x half -> f32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t skinny_instruction(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint2 lds8(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Thirty-two nibbles of one kind (`mask` 0x000f000f: the low ones, 0x00f000f0: the high ones, in place) out of a weight
// row's 32 quant bytes, times their sub-block's scale, as sixteen pairs of half floats.  `mul` and `bias` are the scale's
// constants from the scale table:
//   low nibbles:            (1024 + q) * sc - 1024 sc          (halves (sc, sc), (-1024 sc, -1024 sc))
//   high nibbles, in place: (1024 + 16 q) * (sc / 16) - 64 sc  (halves (sc / 16) x 2, (-64 sc) x 2)
// A mask and an or turn the nibbles of bytes 0 and 2 of a word into two half floats at once (bytes 1 and 3 after a
// shift), so every eight elements come out in the order 0 2 1 3 4 6 5 7; the activation staging stores its numbers in
// the same order (kSkChunkOrder), and a dot product does not mind.
__device__ __forceinline__ void skinny_scaled(const uint2 (&q)[4], uint32_t mask, uint32_t mul, uint32_t bias, uint32_t (&out)[16]) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint32_t w0 = q[t].x, w1 = q[t].y, s0 = w0 >> 8, s1 = w1 >> 8;
        out[4 * t + 0] = hfma2_bits((w0 & mask) | 0x64006400u, mul, bias);
        out[4 * t + 1] = hfma2_bits((s0 & mask) | 0x64006400u, mul, bias);
        out[4 * t + 2] = hfma2_bits((w1 & mask) | 0x64006400u, mul, bias);
        out[4 * t + 3] = hfma2_bits((s1 & mask) | 0x64006400u, mul, bias);
    }
}

// Sixteen 32-bit columns of this thread's tensor-memory lane (the warp's 32 lanes start at the address's lane).
__device__ __forceinline__ void tmem_store_16(uint32_t address, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                 "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D (+)= A B with the A operand in tensor memory (lane = row of A, a column = two consecutive half floats of K) and B
// through a shared-memory descriptor.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The byte of sub-block `sub` out of the two words q4k_scales returns.
__device__ __forceinline__ uint32_t k4_byte(const uint32_t (&words)[2], uint32_t sub) {
    return (words[sub >> 2] >> (8 * (sub & 3))) & 0xffu;
}

// dmin * m of four sub-blocks (the bytes of `mins`) as pairs (h1, h2) of half floats with h1 + h2 = dmin * m exactly.
__device__ __forceinline__ uint4 skinny_min_chunk(float dmin, uint32_t mins) {
    uint32_t v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float product = dmin * (float)((mins >> (8 * i)) & 0xffu);
        const __half h1 = __float2half_rn(product), h2 = __float2half_rn(product - __half2float(h1));
        v[i] = (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(h2) << 16);
    }
    return make_uint4(v[0], v[1], v[2], v[3]);
}

// The roles that issue MMAs and copies run as whole warps with the issue itself under elect_one_lane(): their loop
// state is then the same in every lane, which lets the compiler keep descriptors and addresses in uniform registers
// (inside an `if (lane == 0)` branch every MMA paid for moving them there: 65 ns an MMA, whatever its shape).
__device__ __forceinline__ bool elect_one() { return elect_one_lane(); }

// A position in a ring of `n` stages and the phase of its barriers.
struct SkRing {
    uint32_t s = 0, phase = 0;
    __device__ __forceinline__ void next(uint32_t n) {
        if (++s == n) { s = 0; phase ^= 1u; }
    }
};

// The K slice of an item.
__device__ __forceinline__ void skinny_slice(const SkinnyParams &p, uint32_t item, uint32_t &tile, uint32_t &sb0, uint32_t &sb1) {
    tile = item / p.splits;
    const uint32_t slice = item - tile * p.splits;
    sb0 = (uint32_t)((uint64_t)slice * p.nsb / p.splits);
    sb1 = (uint32_t)((uint64_t)(slice + 1) * p.nsb / p.splits);
}

// NB = bpad / 8: the activation rows in groups of eight (tensor-memory reads of eight columns).
template <int NB>
__global__ void __launch_bounds__(kSkThreads, 1) skinny_q4k_tcgen05_kernel(const __grid_constant__ SkinnyParams p) {
    extern __shared__ uint8_t skinny_raw[];
    constexpr uint32_t BPAD = NB * 8, N = 2 * BPAD;
    constexpr uint32_t kXTile = N * 128, kXStage = 2 * kXTile, kXStages = skinny_x_stages(BPAD);
    const uint32_t base = (smem_addr(skinny_raw) + 1023u) & ~1023u;
    const uint32_t xring = base, raw = xring + kXStages * kXStage;
    const uint32_t bars = raw + kSkRawStages * kSkRawStage;
    const uint32_t a_full = bars, a_empty = a_full + 8 * kSkStages, x_full = a_empty + 8 * kSkStages;
    const uint32_t x_empty = x_full + 8 * kSkXStagesMost, raw_full = x_empty + 8 * kSkXStagesMost;
    const uint32_t raw_empty = raw_full + 8 * kSkRawStages, d_full = raw_empty + 8 * kSkRawStages, d_empty = d_full + 16;
    const uint32_t m_full = d_empty + 16, m_empty = m_full + 8, slot = m_empty + 8;
    __shared__ uint32_t failed;
    __shared__ __align__(16) uint4 scale_table[64];   // per six-bit scale sc: (sc, sc), (-1024 sc) x 2, (sc / 16) x 2, (-64 sc) x 2
    const uint32_t tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const uint32_t nitems = p.ntile128 * p.splits;

    if (tid >= 64 && tid < 128) {
        const uint32_t sc = tid - 64;
        const uint32_t h = (uint32_t)__half_as_ushort(__ushort2half_rn((unsigned short)sc)), mul_lo = h | (h << 16);
        const uint32_t mul_hi = hmul2_bits(mul_lo, 0x2c002c00u);   // 1 / 16
        scale_table[sc] = make_uint4(mul_lo, hmul2_bits(mul_lo, 0xe400e400u), mul_hi, hmul2_bits(mul_hi, 0xe400e400u));   // x -1024
    }
    if (tid == 0) {
        failed = 0;
        for (uint32_t s = 0; s < kSkStages; ++s) {
            mbar_init(a_full + 8 * s, 4);                  // the four producer warps of the slot
            mbar_init(a_empty + 8 * s, 1);                 // one tcgen05.commit
        }
        for (uint32_t s = 0; s < kXStages; ++s) {
            mbar_init(x_full + 8 * s, 1);                  // the thread that asks for the tiles (with their bytes)
            mbar_init(x_empty + 8 * s, 1);
        }
        for (uint32_t s = 0; s < kSkRawStages; ++s) {
            mbar_init(raw_full + 8 * s, 1);
            mbar_init(raw_empty + 8 * s, kSkProducerWarps / 2);   // the eight warps that write the two stages of the super-block
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(d_full + 8 * b, 1);
            mbar_init(d_empty + 8 * b, 4);
        }
        mbar_init(m_full, 1);
        mbar_init(m_empty, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kSkMmaWarp) tmem_alloc(slot, kSkTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds4(slot);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp < kSkProducerWarps) {
        // ---------------- producers: raw units -> sc * q in tensor memory ----------------
        // A warp reaches the 32 tensor-memory lanes of its rank in its group of four, so warp w writes weight rows
        // 32 (w % 4) + lane: lane l is row l of 32-row unit w % 4.  The stages of the launch are numbered in the order
        // the MMAs take them (for every item two per super-block, then the stages of its second sum), stage P lives
        // in ring slot P % 4, and the four warps w / 4 == s write exactly the stages of slot s, whatever they hold.
        // (A slot's writers must be the same warps every time: the wait for a slot to be free tells phases apart by
        // one parity bit, which only holds for a warp that wrote the slot's previous stage itself.  With the stages
        // dealt by super-block instead, a warp running ahead over an item's end took a slot two stages early, now and
        // then, and two items of a CTA came out wrong.)  A stage of the first sum is 128 k of a super-block: nibble
        // groups 2 h and 2 h + 1, each 32 quant bytes of the row whose low nibbles are one sub-block and whose high
        // nibbles the next; a thread pays for its row's header, its waits and its arrivals once per 128 k.
        const uint32_t quarter = warp & 3u, slot_a = warp >> 2;
        const uint32_t hu = lane >> 4, r16 = lane & 15, g = r16 & 7, upper = r16 >> 3;
        const uint32_t table = smem_addr(scale_table);
        const uint32_t my_unit = quarter * kQ4kStage + hu * kQ4kUnit;        // this row's half-unit inside a raw stage
        const uint32_t my_quants = my_unit + 256 + g * 64 + upper * 8;       // + 1024 h + 512 j + 16 t: quant bytes 8 t ... of group 2 h + j
        const uint32_t columns = tmem + ((quarter * 32u) << 16) + slot_a * kSkStageCols;
        uint32_t base = 0;       // number of the running item's first stage
        uint32_t seq_base = 0;   // super-blocks of this CTA before the running item (the raw ring follows them)
        bool alive = true;
        uint32_t events = 0;
        for (uint32_t item = blockIdx.x; item < nitems && alive; item += gridDim.x) {
            uint32_t tile, sb0, sb1;
            skinny_slice(p, item, tile, sb0, sb1);
            const uint32_t count = sb1 - sb0, main_end = base + 2 * count, end = main_end + (count + 7) / 8;
            const uint32_t held = min(tile * 4 + quarter, p.tiles32 - 1);
            const uint8_t *headers = p.w + ((uint64_t)held * p.nsb * 2 + hu) * kQ4kUnit + r16 * 16;
            for (uint32_t at = base + ((slot_a - base) & 3u); at < end && alive; at += 4) {
                const uint32_t a_phase = (at >> 2) & 1u;
                if (at < main_end) {
                    // ---- a stage of the first sum ----
                    const uint32_t step = (at - base) >> 1, h = (at - base) & 1u, seq = seq_base + step;
                    const uint32_t raw_slot = seq % kSkRawStages, raw_phase = (seq / kSkRawStages) & 1u;
                    if (!mbar_wait(raw_full + 8 * raw_slot, raw_phase)) { alive = false; break; }
                    if (tid == 0) { SK_TRACE(0, events); }
                    const uint32_t stage = raw + raw_slot * kSkRawStage;
                    const uint4 header = lds16(stage + my_unit + r16 * 16);
                    uint2 q[2][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int t = 0; t < 4; ++t) q[j][t] = lds8(stage + my_quants + 1024 * h + 512 * j + 16 * t);
                    // the six-bit scales of sub-blocks 4 h ... 4 h + 3, a byte each (q4k_scales' first or second word)
                    const uint32_t scales = h ? ((header.w & 0x0f0f0f0fu) | (((header.y >> 6) & 0x03030303u) << 4)) : (header.y & 0x3f3f3f3fu);
                    const uint2 low0 = lds8(table + (scales & 0xffu) * 16), high0 = lds8(table + ((scales >> 8) & 0xffu) * 16 + 8);
                    const uint2 low1 = lds8(table + ((scales >> 16) & 0xffu) * 16), high1 = lds8(table + (scales >> 24) * 16 + 8);
                    if (!mbar_wait(a_empty + 8 * slot_a, a_phase ^ 1u)) { alive = false; break; }
                    if (tid == 0) { SK_TRACE(1, events); }
                    tc_fence_after();
                    uint32_t out[16];
                    skinny_scaled(q[0], 0x000f000fu, low0.x, low0.y, out);
                    tmem_store_16(columns, out);
                    skinny_scaled(q[0], 0x00f000f0u, high0.x, high0.y, out);
                    tmem_store_16(columns + 16, out);
                    skinny_scaled(q[1], 0x000f000fu, low1.x, low1.y, out);
                    tmem_store_16(columns + 32, out);
                    skinny_scaled(q[1], 0x00f000f0u, high1.x, high1.y, out);
                    // every lane's loads of the raw stage have delivered (their values are in `out` and in the stores):
                    // the stage may be refilled.  (An arrival right behind the loads let the refill overtake loads
                    // still in flight.)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(raw_empty + 8 * raw_slot);
                    tmem_store_16(columns + 48, out);
                    if (tid == 0) { SK_TRACE(8, events); }
                } else {
                    // ---- a stage of the second sum: dmin * m of eight super-blocks, 16 half floats = 8 columns each ----
                    const uint32_t first = sb0 + 8 * (at - main_end);
                    bool waited = false;
#pragma unroll
                    for (uint32_t round = 0; round < 2; ++round) {
                        uint4 hd[4];
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint32_t sb = first + 4 * round + j;
                            hd[j] = sb < sb1 ? ld_stream16(headers + (uint64_t)sb * 2 * kQ4kUnit) : make_uint4(0u, 0u, 0u, 0u);
                        }
                        if (!waited) {
                            if (!mbar_wait(a_empty + 8 * slot_a, a_phase ^ 1u)) { alive = false; break; }
                            tc_fence_after();
                            waited = true;
                        }
#pragma unroll
                        for (uint32_t pair = 0; pair < 2; ++pair) {
                            uint32_t out[16];
#pragma unroll
                            for (uint32_t j = 0; j < 2; ++j) {
                                const uint4 &one = hd[2 * pair + j];
                                uint32_t sc[2], mn[2];
                                q4k_scales(one.y, one.z, one.w, sc, mn);
                                const float dmin = half_bits_to_float(one.x >> 16);   // (a super-block past the slice reads as zeros)
                                const uint4 c0 = skinny_min_chunk(dmin, mn[0]), c1 = skinny_min_chunk(dmin, mn[1]);
                                out[8 * j + 0] = c0.x; out[8 * j + 1] = c0.y; out[8 * j + 2] = c0.z; out[8 * j + 3] = c0.w;
                                out[8 * j + 4] = c1.x; out[8 * j + 5] = c1.y; out[8 * j + 6] = c1.z; out[8 * j + 7] = c1.w;
                            }
                            tmem_store_16(columns + 32 * round + 16 * pair, out);
                        }
                    }
                    if (!alive) break;
                }
                tmem_store_wait();
                tc_fence_before();
                if (tid == 0) { SK_TRACE(9, events); }
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full + 8 * slot_a);
                if (tid == 0) { SK_TRACE(2, events); }
                ++events;
            }
            base = end;
            seq_base += count;
        }
        if (!alive) failed = 1;
    } else if (warp < kSkMmaWarp) {
        // ---------------- epilogue: accumulators -> scaled sums -> outputs ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the staged activations and the output belong to the kernels before
        const uint32_t quarter = warp - kSkEpilogueWarp0;     // the 32 tensor-memory lanes this warp may read
        const uint32_t lanes = (quarter * 32u) << 16;
        uint32_t seq = 0, items_done = 0;
        bool alive = true;
        for (uint32_t item = blockIdx.x; item < nitems && alive; item += gridDim.x, ++items_done) {
            uint32_t tile, sb0, sb1;
            skinny_slice(p, item, tile, sb0, sb1);
            const uint32_t t32 = tile * 4 + quarter, held = min(t32, p.tiles32 - 1);
            // this lane's weight row: the header (d, dmin, scales) of super-block sb lies 2 half-units further per sb
            const uint8_t *header = p.w + ((uint64_t)held * p.nsb * 2 + (lane >> 4)) * kQ4kUnit + (lane & 15) * 16;
            float acc[BPAD];
#pragma unroll
            for (uint32_t r = 0; r < BPAD; ++r) acc[r] = 0.0f;
            uint32_t coming = ld_stream4(header + (uint64_t)sb0 * 2 * kQ4kUnit);
            for (uint32_t sb = sb0; sb < sb1; ++sb, ++seq) {
                const float d = half_bits_to_float(coming & 0xffffu);
                if (sb + 1 < sb1) coming = ld_stream4(header + (uint64_t)(sb + 1) * 2 * kQ4kUnit);
                const uint32_t b = seq & 1u;
                if (!mbar_wait(d_full + 8 * b, (seq >> 1) & 1u)) { alive = false; break; }
                if (quarter == 0 && lane == 0) { SK_TRACE(6, seq); }
                tc_fence_after();
                const uint32_t d1 = tmem + lanes + kSkAccAt + b * N;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    uint32_t hi[8], lo[8];
                    tmem_load_8(d1 + nb * 8, hi);
                    tmem_load_8(d1 + BPAD + nb * 8, lo);
                    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(p.xs + (uint64_t)sb * BPAD + nb * 8));
                    const float4 s1 = __ldg(reinterpret_cast<const float4 *>(p.xs + (uint64_t)sb * BPAD + nb * 8 + 4));
                    const float scale[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        acc[nb * 8 + i] = fmaf(scale[i] * d, fmaf(__uint_as_float(lo[i]), 0.00048828125f, __uint_as_float(hi[i])), acc[nb * 8 + i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_empty + 8 * b);
                if (quarter == 0 && lane == 0) { SK_TRACE(7, seq); }
            }
            if (!alive) break;
            // ---- the second sum of the item ----
            if (!mbar_wait(m_full, items_done & 1u)) { alive = false; break; }
            tc_fence_after();
            {
                const uint32_t d2 = tmem + lanes + kSkAccAt + 2 * N;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    uint32_t hi[8], lo[8];
                    tmem_load_8(d2 + nb * 8, hi);
                    tmem_load_8(d2 + BPAD + nb * 8, lo);
                    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(p.rs + nb * 8));
                    const float4 s1 = __ldg(reinterpret_cast<const float4 *>(p.rs + nb * 8 + 4));
                    const float scale[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        acc[nb * 8 + i] = fmaf(-scale[i], fmaf(__uint_as_float(lo[i]), 0.00048828125f, __uint_as_float(hi[i])), acc[nb * 8 + i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(m_empty);
            // ---- the item's sums are complete for this K slice ----
            bool final = true;
            if (p.splits > 1) {
                float *mine = p.partial + ((uint64_t)item * BPAD) * kSkTileRows + quarter * 32 + lane;
#pragma unroll
                for (uint32_t r = 0; r < BPAD; ++r) __stcg(mine + r * kSkTileRows, acc[r]);
                __syncwarp();
                unsigned int seen = 0;
                if (lane == 0) seen = arrive_on(p.counters + tile * 4 + quarter);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                final = seen == p.splits - 1;
                if (final) {   // the last slice to arrive adds them all, in slice order
                    const float *all = p.partial + ((uint64_t)tile * p.splits * BPAD) * kSkTileRows + quarter * 32 + lane;
#pragma unroll
                    for (uint32_t r = 0; r < BPAD; ++r) acc[r] = 0.0f;
                    for (uint32_t s = 0; s < p.splits; ++s)
#pragma unroll
                        for (uint32_t r = 0; r < BPAD; ++r) acc[r] += __ldcg(all + ((uint64_t)s * BPAD + r) * kSkTileRows);
                    if (lane == 0) p.counters[tile * 4 + quarter] = 0u;
                }
            }
            if (final && t32 < p.tiles32) {
                if (p.pair) {
                    const uint32_t col = t32 * 16 + (lane & 15);
#pragma unroll
                    for (uint32_t r = 0; r < BPAD; ++r) {
                        const float other = __shfl_down_sync(0xffffffffu, acc[r], 16);
                        if (r < p.rows && lane < 16 && col < p.n)
                            p.out[(uint64_t)r * p.out_stride + col] = chained(p.chain, r, col, acc[r] * sigmoid_f(acc[r]) * other);
                    }
                } else {
                    const uint32_t col = t32 * 32 + lane;
#pragma unroll
                    for (uint32_t r = 0; r < BPAD; ++r)
                        if (r < p.rows && col < p.n) p.out[(uint64_t)r * p.out_stride + col] = chained(p.chain, r, col, acc[r]);
                }
            }
        }
        if (!alive) failed = 1;
    } else if (warp == kSkMmaWarp) {
        // ---------------- MMA issue (the whole warp walks the loop; one lane issues) ----------------
        const uint32_t idesc = skinny_instruction(kSkTileRows, N);
        const uint64_t x_desc0 = smem_descriptor(xring);
        SkRing at_a, at_x;
        uint32_t seq = 0, items_done = 0, events = 0;
        bool alive = true;
        // one stage: 128 k as two tiles of four 16-k MMAs; `fresh`: the first MMA starts the accumulator anew
        auto stage_mmas = [&](uint32_t accumulator, bool fresh) -> bool {
            if (!mbar_wait(a_full + 8 * at_a.s, at_a.phase)) return false;
            if (!mbar_wait(x_full + 8 * at_x.s, at_x.phase)) return false;
            if (lane == 0) { SK_TRACE(3, events); }
            tc_fence_after();
            const uint32_t a_columns = tmem + at_a.s * kSkStageCols;
            const uint64_t desc_b = x_desc0 + (uint64_t)((at_x.s * kXStage) >> 4);
            if (elect_one()) {
#pragma unroll
                for (uint32_t j = 0; j < 2; ++j)
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk)   // 16 half floats: 8 columns of A, 32 bytes further along K inside B's swizzle atom
                        tc_mma_f16_ts(accumulator, a_columns + j * 32 + kk * 8, desc_b + j * (kXTile >> 4) + kk * 2, idesc,
                                      (fresh && j == 0 && kk == 0) ? 0u : 1u);
                tc_commit(a_empty + 8 * at_a.s);   // frees the stages when these MMAs have read them
                tc_commit(x_empty + 8 * at_x.s);
            }
            __syncwarp();
            if (lane == 0) { SK_TRACE(4, events); }
            ++events;
            at_a.next(kSkStages);
            at_x.next(kXStages);
            return true;
        };
        for (uint32_t item = blockIdx.x; item < nitems && alive; item += gridDim.x, ++items_done) {
            uint32_t tile, sb0, sb1;
            skinny_slice(p, item, tile, sb0, sb1);
            for (uint32_t sb = sb0; sb < sb1 && alive; ++sb, ++seq) {
                const uint32_t b = seq & 1u;
                if (!mbar_wait(d_empty + 8 * b, ((seq >> 1) & 1u) ^ 1u)) { alive = false; break; }
                tc_fence_after();
                if (!stage_mmas(tmem + kSkAccAt + b * N, true) || !stage_mmas(tmem + kSkAccAt + b * N, false)) { alive = false; break; }
                if (elect_one()) tc_commit(d_full + 8 * b);
                __syncwarp();
            }
            if (!alive) break;
            if (!mbar_wait(m_empty, (items_done & 1u) ^ 1u)) { alive = false; break; }
            tc_fence_after();
            for (uint32_t first = sb0; first < sb1; first += 8)
                if (!stage_mmas(tmem + kSkAccAt + 2 * N, first == sb0)) { alive = false; break; }
            if (alive && elect_one()) tc_commit(m_full);
            __syncwarp();
        }
        if (!alive) failed = 1;
    } else if (warp == kSkTmaWarp) {
        // ---------------- activation tiles by the tensor memory accelerator ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the staging kernel wrote them
        SkRing at_x;
        bool alive = true;
        // (x, the column, is a multiple of 16 half floats = 32 bytes: the 16-byte rule of the copy holds)
        auto load_stage = [&](const CUtensorMap *map, uint32_t column) -> bool {
            if (!mbar_wait(x_empty + 8 * at_x.s, at_x.phase ^ 1u)) return false;
            const uint32_t tiles = xring + at_x.s * kXStage;
            if (elect_one()) {
                mbar_expect(x_full + 8 * at_x.s, kXStage);
                tma_load_2d(tiles, map, column, 0, x_full + 8 * at_x.s);
                tma_load_2d(tiles + kXTile, map, column + 64, 0, x_full + 8 * at_x.s);
            }
            __syncwarp();
            at_x.next(kXStages);
            return true;
        };
        for (uint32_t item = blockIdx.x; item < nitems && alive; item += gridDim.x) {
            uint32_t tile, sb0, sb1;
            skinny_slice(p, item, tile, sb0, sb1);
            for (uint32_t sb = sb0; sb < sb1 && alive; ++sb)
                alive = load_stage(&p.x_map, sb * 256) && load_stage(&p.x_map, sb * 256 + 128);
            for (uint32_t first = sb0; first < sb1 && alive; first += 8) alive = load_stage(&p.sx_map, first * 16);
        }
        if (!alive) failed = 1;
    } else if (warp == kSkRawWarp) {
        // ---------------- raw weight units by bulk copies ----------------
        SkRing at_raw;
        bool alive = true;
        for (uint32_t item = blockIdx.x; item < nitems && alive; item += gridDim.x) {
            uint32_t tile, sb0, sb1;
            skinny_slice(p, item, tile, sb0, sb1);
            // rows past the weight's end re-read its last tile; nothing stores them
            const uint8_t *unit[4];
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) unit[u] = p.w + (uint64_t)min(tile * 4 + u, p.tiles32 - 1) * p.nsb * kQ4kStage;
            for (uint32_t sb = sb0; sb < sb1; ++sb) {
                if (!mbar_wait(raw_empty + 8 * at_raw.s, at_raw.phase ^ 1u)) { alive = false; break; }
                if (elect_one()) {
                    mbar_expect(raw_full + 8 * at_raw.s, kSkRawStage);
#pragma unroll
                    for (uint32_t u = 0; u < 4; ++u)
                        bulk_load(raw + at_raw.s * kSkRawStage + u * kQ4kStage, unit[u] + (uint64_t)sb * kQ4kStage, kQ4kStage, raw_full + 8 * at_raw.s);
                }
                __syncwarp();
                at_raw.next(kSkRawStages);
            }
        }
        if (!alive) failed = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (failed && tid == 0) atomicOr(p.status, 8u);
    if (warp == kSkMmaWarp) tmem_free(tmem, kSkTmemCols);
}

}  // namespace nc
