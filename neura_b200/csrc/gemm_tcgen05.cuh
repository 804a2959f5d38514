// Prefill product on the 5th-generation tensor cores: out[M][N] = chain(X[M][K] . W[N][K]^T) with
// Q4_K weights dequantised to bf16 tiles in shared memory, bf16 activations, f32 accumulation in
// tensor memory (tcgen05.mma, kind::f16).
//
// This stands in for the reference's tensor path, template_run_matmul_cooperative
// (crates/neura-kernel/src/task/matmul.rs:1344-1565), which converts both operands to 16-bit
// floats in shared memory and multiplies them with cooperative-matrix MMAs into f32.
//
// One CTA computes a 256 (rows of X) x 256 (rows of W) tile of the output as two 128 x 256
// accumulators, so a dequantised weight tile feeds two MMAs.  K advances in steps of 64 (one
// 128-byte swizzle atom of bf16).  For every step one thread asks the tensor memory accelerator
// for the X tile (cp.async.bulk.tensor, 128-byte swizzle, rows past M zero-filled) and warps 0-15
// dequantise a quarter super-block of 256 weight rows into the W tile (the raw blocks of the next
// step are fetched while this one is dequantised); warp 16 issues the MMAs; the tiles cycle through a ring of stages
// guarded by mbarriers (full: producers -> MMA, empty: tcgen05.commit -> producers).  When K is
// exhausted the producer warps read the accumulator out of tensor memory (tcgen05.ld), apply
// the fused chain and store f32.  Every wait is bounded; a wait that runs out raises the status
// word, and the CTA still frees its tensor memory before it leaves.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "gemv_mma.cuh"

namespace nc {

constexpr uint32_t kGemmBM = 256, kGemmBN = 256, kGemmBK = 64, kGemmStages = 3;
constexpr uint32_t kGemmABytes = kGemmBM * kGemmBK * 2;   // 32 KiB: two 128-row MMA operands
constexpr uint32_t kGemmBBytes = kGemmBN * kGemmBK * 2;   // 32 KiB
constexpr uint32_t kGemmStageBytes = kGemmABytes + kGemmBBytes;
constexpr uint32_t kGemmTmemCols = 512;                   // two accumulators of 128 lanes x 256 f32 columns
constexpr uint32_t kGemmProducers = 512;                  // 16 producer/epilogue warps
constexpr uint32_t kGemmThreads = kGemmProducers + 32;    // ... + the MMA warp
constexpr uint32_t kGemmSmem = kGemmStages * kGemmStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

struct GemmParams {
    CUtensorMap x_map;           // the bf16 activations as a 2-D tensor [m][k], boxes of 256 rows x 64 columns
    const uint8_t *w;            // tiled Q4_K weights
    const __nv_bfloat16 *x;      // [m][k] bf16 activations
    float *out;                  // [m][out_stride]
    uint64_t out_stride;
    uint32_t m, n, k;
    uint32_t units32;            // 32-row units along N the sealed weight holds
    unsigned int *status;
    Chain chain;
    // gridDim.z CTAs share a tile, each taking a run of whole super-blocks of K; CTA z then writes its sums to
    // out + z * split_stride (scratch: the launcher sums the runs in order afterwards and applies the chain there)
    uint64_t split_stride;
    // pair = 1: the weight is a sealed gate|up pair (every 32-row unit holds 16 gate rows, then the 16 up rows of the
    // same columns) and the epilogue writes out[r][16 u + i] = chain(silu(gate) * up) for unit u: n_out columns in all
    uint32_t pair, n_out;
    // tma_out = 1: `out_map` describes the output ([m][n] f32, boxes of 32 x 32, 128-byte swizzled) and the epilogue
    // hands each 32 x 32 block to a bulk tensor store instead of storing it row by row
    uint32_t tma_out;
    CUtensorMap out_map;
};

// f32 -> bf16 with round-to-nearest-even (crates/neura-precision/src/lib.rs:325-329).
__global__ void to_bf16_kernel(const float *x, uint64_t x_stride, uint32_t rows, uint32_t k, __nv_bfloat16 *out) {
    const uint64_t total = (uint64_t)rows * k;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(x[(i / k) * x_stride + i % k]);
}

// ---- tcgen05 plumbing -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One lane of a converged warp.
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t chosen;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(chosen));
    return chosen != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The barrier is told when this thread's asynchronous copies issued so far have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, swizzled in
// 128-byte atoms: groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
    uint64_t desc = 0;
    desc |= (uint64_t)((address & 0x3ffffu) >> 4);   // start address
    desc |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzled K-major tiles)
    desc |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows x 128 bytes
    desc |= (uint64_t)1 << 46;                        // descriptor version of this architecture
    desc |= (uint64_t)2 << 61;                        // 128-byte swizzle
    return desc;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t instruction_descriptor(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// 32 lanes x 32 columns of f32 out of tensor memory: thread i of the warp gets lane i's 32 columns.
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- dequantising a quarter super-block of one weight row into two 16-byte chunks of bf16 -------
// `w0`, `w1`: the eight quant bytes [8t, 8t+8) of nibble group G of the row; low nibbles are
// elements 8t.. of sub-block 2G, high nibbles the same elements of sub-block 2G+1.
// value = (d*sc)*q - dmin*m rounded to f32 as q4_k_values does (crates/neura-precision/src/ggml.rs:341-346):
// d*sc, dmin*m and (d*sc)*q are exact in f32 (11 x 6 x 4 significant bits), so one fused
// multiply-subtract rounds exactly where the reference's separate operations round; then bf16 RNE.
__device__ __forceinline__ uint32_t bf16_pair(float quantum, float low, uint32_t bytes, uint32_t lane_a, uint32_t lane_b) {
    const float a = __uint_as_float(__byte_perm(bytes, 0x4b000000u, 0x7650u | lane_a)) - 8388608.0f;
    const float b = __uint_as_float(__byte_perm(bytes, 0x4b000000u, 0x7650u | lane_b)) - 8388608.0f;
    const __nv_bfloat162 pair = __floats2bfloat162_rn(fmaf(quantum, a, -low), fmaf(quantum, b, -low));
    return *reinterpret_cast<const uint32_t *>(&pair);
}

// The 6-bit scale and min of sub-blocks 2G and 2G+1 out of the twelve scale bytes (y = bytes 0-3,
// z = 4-7, w = 8-11; scale_min_k4, crates/neura-precision/src/ggml.rs:127-136).
__device__ __forceinline__ void quarter_scales(const uint4 &header, uint32_t G, float (&quantum)[2], float (&low)[2]) {
    const float d = half_bits_to_float(header.x & 0xffffu), dmin = half_bits_to_float(header.x >> 16);
    const uint32_t shift = 16 * (G & 1);   // sub-blocks 2G, 2G+1 sit in bytes 2(G&1), 2(G&1)+1 of their words
    uint32_t sc, mn;                       // two bytes each: the pair of this quarter
    if (G < 2) {
        sc = (header.y >> shift) & 0x3f3fu;
        mn = (header.z >> shift) & 0x3f3fu;
    } else {
        sc = ((header.w >> shift) & 0x0f0fu) | ((((header.y >> shift) >> 6) & 0x0303u) << 4);
        mn = (((header.w >> shift) >> 4) & 0x0f0fu) | ((((header.z >> shift) >> 6) & 0x0303u) << 4);
    }
    quantum[0] = d * (float)(sc & 0xffu);
    quantum[1] = d * (float)(sc >> 8);
    low[0] = dmin * (float)(mn & 0xffu);
    low[1] = dmin * (float)(mn >> 8);
}

__device__ __forceinline__ void dequant_row_quarter(uint32_t tile, uint32_t row, uint32_t t, uint32_t G, uint32_t w0,
                                                    uint32_t w1, const uint4 &header) {
    float quantum[2], low[2];
    quarter_scales(header, G, quantum, low);
    const uint32_t lo0 = w0 & 0x0f0f0f0fu, lo1 = w1 & 0x0f0f0f0fu;
    const uint32_t hi0 = (w0 >> 4) & 0x0f0f0f0fu, hi1 = (w1 >> 4) & 0x0f0f0f0fu;
    const uint32_t at = tile + row * 128;
    // Eight lanes store together: two rows (g, g + 1) x four chunks t.  Both rows' low chunks swizzle into the same
    // four 16-byte columns and would collide two by two, so odd rows store their high chunk first: every group of
    // eight then covers all eight columns of the 128-byte line.
    const bool odd = row & 1u;
    const float qa = odd ? quantum[1] : quantum[0], la = odd ? low[1] : low[0];
    const float qb = odd ? quantum[0] : quantum[1], lb = odd ? low[0] : low[1];
    const uint32_t a0 = odd ? hi0 : lo0, a1 = odd ? hi1 : lo1, b0 = odd ? lo0 : hi0, b1 = odd ? lo1 : hi1;
    const uint32_t ca = odd ? 4 + t : t, cb = odd ? t : 4 + t;
    sts16(at + ((ca ^ (row & 7)) << 4), bf16_pair(qa, la, a0, 0, 1), bf16_pair(qa, la, a0, 2, 3), bf16_pair(qa, la, a1, 0, 1),
          bf16_pair(qa, la, a1, 2, 3));
    sts16(at + ((cb ^ (row & 7)) << 4), bf16_pair(qb, lb, b0, 0, 1), bf16_pair(qb, lb, b0, 2, 3), bf16_pair(qb, lb, b1, 0, 1),
          bf16_pair(qb, lb, b1, 2, 3));
}

// Warp w of the 16 producers owns half (w & 1) of 32-row unit (w >> 1) of the 256-row W tile.  What one of its
// threads fetches: per k-step the 16 bytes of quants of its lane, per super-block (four k-steps) the headers of
// its two rows.
__device__ __forceinline__ const uint8_t *half_unit_of(const GemmParams &p, uint32_t n0, uint32_t sb, uint32_t warp) {
    const uint32_t nsb = p.k / kSuperBlock, unit = min(n0 / 32 + (warp >> 1), p.units32 - 1);
    return p.w + (((uint64_t)unit * nsb + sb) * 2 + (warp & 1)) * kQ4kUnit;
}
__device__ __forceinline__ uint4 fetch_quants(const GemmParams &p, uint32_t n0, uint32_t it, uint32_t warp, uint32_t lane) {
    return ld_stream16(half_unit_of(p, n0, it >> 2, warp) + 256 + (it & 3) * 512 + lane * 16);
}
__device__ __forceinline__ void fetch_headers(uint4 (&h)[2], const GemmParams &p, uint32_t n0, uint32_t sb, uint32_t warp,
                                              uint32_t lane) {
    const uint8_t *from = half_unit_of(p, n0, sb, warp);
    h[0] = ld_stream16(from + (lane >> 2) * 16);
    h[1] = ld_stream16(from + ((lane >> 2) + 8) * 16);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t src_smem) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src_smem)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_q4k_tcgen05_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t gemm_raw[];
    const uint32_t base = (smem_addr(gemm_raw) + 1023u) & ~1023u;   // swizzle atoms want 1024-byte alignment
    const uint32_t bars = base + kGemmStages * kGemmStageBytes;
    const uint32_t full = bars, empty = bars + 8 * kGemmStages, accum = bars + 16 * kGemmStages;
    const uint32_t slot = accum + 8;
    __shared__ uint32_t failed;
    const uint32_t tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const uint32_t m0 = blockIdx.y * kGemmBM, n0 = blockIdx.x * kGemmBN;
    const uint32_t every_sb = p.k / kSuperBlock;
    const uint32_t sb_first = (uint32_t)((uint64_t)every_sb * blockIdx.z / gridDim.z);
    const uint32_t sb_last = (uint32_t)((uint64_t)every_sb * (blockIdx.z + 1) / gridDim.z);
    const uint32_t step_first = sb_first * (kSuperBlock / kGemmBK), ksteps = sb_last * (kSuperBlock / kGemmBK);   // this CTA's k-steps: [step_first, ksteps)
    float *const out = p.out + blockIdx.z * p.split_stride;
    constexpr uint32_t kMmaWarp = kGemmProducers / 32;

    if (tid == 0) {
        failed = 0;
        for (uint32_t s = 0; s < kGemmStages; ++s) {
            mbar_init(full + 8 * s, kGemmProducers / 32 + 1);   // every producer warp arrives, and the thread that asks for the X tile
            mbar_init(empty + 8 * s, 1);                   // one tcgen05.commit
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(slot, kGemmTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds4(slot);
    // the bf16 activations are written by the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp < kMmaWarp) {
        // ---------------- producers ----------------
        const uint32_t g = lane >> 2, t = lane & 3, half = warp & 1;
        bool alive = true;
        // the quants travel three steps ahead of their use, the headers one super-block ahead, and the super-block
        // after the next is asked into L2 (a miss to HBM takes longer than a step); rows past the weight's end
        // re-read its last unit, and the epilogue does not store them
        const uint32_t nsb = sb_last;
        uint4 quants[4], headers[2], coming[2];
#pragma unroll
        for (uint32_t j = 0; j < 3; ++j)
            if (step_first + j < ksteps) quants[j] = fetch_quants(p, n0, step_first + j, warp, lane);
        fetch_headers(headers, p, n0, sb_first, warp, lane);
        for (uint32_t it0 = step_first; it0 < ksteps && alive; it0 += 4) {
            const uint32_t sb = it0 >> 2;
            if (sb + 1 < nsb) fetch_headers(coming, p, n0, sb + 1, warp, lane);
            if (lane == 0 && sb + 2 < nsb)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(half_unit_of(p, n0, sb + 2, warp)), "r"(kQ4kUnit) : "memory");
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                const uint32_t it = it0 + j;
                if (it >= ksteps || !alive) break;
                const uint32_t s = (it - step_first) % kGemmStages, parity = ((it - step_first) / kGemmStages) & 1u;
                if (it + 3 < ksteps) quants[(j + 3) & 3] = fetch_quants(p, n0, it + 3, warp, lane);
                if (!mbar_wait(empty + 8 * s, parity ^ 1u)) { alive = false; break; }
                const uint32_t a_tile = base + s * kGemmStageBytes, b_tile = a_tile + kGemmABytes;
                if (tid == 0) {   // x (columns) is a multiple of 64 bf16 = 128 bytes: the 16-byte rule of the copy holds
                    mbar_expect(full + 8 * s, kGemmABytes);
                    tma_load_2d(a_tile, &p.x_map, it * kGemmBK, m0, full + 8 * s);
                }
                const uint32_t row = (warp >> 1) * 32 + half * 16 + g;
                dequant_row_quarter(b_tile, row, t, j, quants[j].x, quants[j].y, headers[0]);
                dequant_row_quarter(b_tile, row + 8, t, j, quants[j].z, quants[j].w, headers[1]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full + 8 * s);   // one arrival per warp: 512 arrivals on one barrier word would queue up
            }
            headers[0] = coming[0];
            headers[1] = coming[1];
        }
        if (!alive) failed = 1;
        // ---------------- epilogue: warp w reads lanes 32 (w % 4).. of accumulator (w / 4) % 2, column half w / 8 ----------------
        if (alive && mbar_wait(accum, 0)) {
            tc_fence_after();
            const uint32_t which = (warp >> 2) & 1, lanes = (warp & 3) * 32, columns = (warp >> 3) * (kGemmBN / 2);
            const uint32_t row = m0 + which * 128 + lanes + lane;
            float *turn = reinterpret_cast<float *>(gemm_raw + (base - smem_addr(gemm_raw))) + warp * 32 * 33;
            const uint32_t stage = base + warp * 8192;   // (the bulk stores' form of `turn`: two blocks of 32 rows x 128 bytes a warp)
            uint32_t handed = 0;
            for (uint32_t c0 = columns; c0 < columns + kGemmBN / 2; c0 += 32) {
                uint32_t r[32];
                tmem_load_32(tmem + (lanes << 16) + which * kGemmBN + c0, r);
                if (p.tma_out) {
                    // The block goes to shared memory as the tensor map expects it (row = lane, 16-byte chunk c of row r at
                    // chunk c ^ (r & 7) of its 128 bytes) and one bulk store writes what of it lies inside the output;
                    // the warp fills its other buffer meanwhile.
                    const uint32_t first_row = m0 + which * 128 + lanes;
                    if (first_row >= p.m || n0 + c0 >= p.n) continue;   // (the same for the whole warp)
                    if (handed >= 2) {
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        __syncwarp();
                    }
                    const uint32_t at = stage + (handed & 1u) * 4096 + lane * 128;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        float v[4];
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i)
                            v[i] = (row < p.m && n0 + c0 + 4 * j + i < p.n) ? chained(p.chain, row, n0 + c0 + 4 * j + i, __uint_as_float(r[4 * j + i])) : 0.0f;
                        sts16(at + ((j ^ (lane & 7)) << 4), __float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tma_store_2d(&p.out_map, n0 + c0, first_row, stage + (handed & 1u) * 4096);
                    ++handed;
                    continue;
                }
                // A lane holds 32 consecutive outputs of ONE row; stored as they are, one instruction touches 32
                // rows (32 sectors), and those stores held the whole kernel back (without them it runs twice as
                // fast).  So the warp turns its 32 x 32 block through shared memory (the ring is idle by now) and
                // every store instruction writes 128 contiguous bytes of one row.
                if (p.pair) {
                    // a lane holds one unit of one row: its gate sums in r[0..15], its up sums in r[16..31]
                    const uint32_t first_col = (n0 + c0) / 2;
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const float gate = __uint_as_float(r[i]), other = __uint_as_float(r[16 + i]);
                        turn[lane * 33 + i] = (row < p.m && first_col + i < p.n_out) ? chained(p.chain, row, first_col + i, gate * sigmoid_f(gate) * other) : 0.0f;
                    }
                    __syncwarp();
                    const uint32_t col = first_col + (lane & 15);
                    if (col < p.n_out) {   // the two halves of the warp take the even and the odd rows: 64 contiguous bytes each
                        const uint32_t first_row = m0 + which * 128 + lanes;
                        float *to = out + (uint64_t)first_row * p.out_stride + col;
#pragma unroll 8
                        for (uint32_t rr = lane >> 4; rr < 32; rr += 2)
                            if (first_row + rr < p.m) __stcs(to + (uint64_t)rr * p.out_stride, turn[rr * 33 + (lane & 15)]);
                    }
                    __syncwarp();
                    continue;
                }
#pragma unroll
                for (uint32_t i = 0; i < 32; ++i)
                    turn[lane * 33 + i] = (row < p.m && n0 + c0 + i < p.n) ? chained(p.chain, row, n0 + c0 + i, __uint_as_float(r[i])) : 0.0f;
                __syncwarp();
                const uint32_t col = n0 + c0 + lane;
                if (col < p.n) {
                    const uint32_t first_row = m0 + which * 128 + lanes;
                    float *to = out + (uint64_t)first_row * p.out_stride + col;
#pragma unroll 8
                    for (uint32_t rr = 0; rr < 32; ++rr)
                        if (first_row + rr < p.m) __stcs(to + (uint64_t)rr * p.out_stride, turn[rr * 33 + lane]);
                }
                __syncwarp();
            }
            if (p.tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the shared memory outlives its readers
        } else {
            failed = 1;
        }
    } else {
        // ---------------- MMA issue ----------------
        // The whole warp walks the loop and one elected lane issues: the loop state is then the same in every lane
        // and the compiler keeps the descriptors in uniform registers.  (Inside an `if (lane == 0)` branch every
        // MMA paid about 65 ns for moving them there, as much as the MMA itself takes.)
        const uint32_t idesc = instruction_descriptor(128, kGemmBN);
        bool alive = true;
        for (uint32_t it = 0; it < ksteps - step_first; ++it) {
            const uint32_t s = it % kGemmStages, parity = (it / kGemmStages) & 1u;
            if (!mbar_wait(full + 8 * s, parity)) { alive = false; break; }
            tc_fence_after();
            const uint32_t a_tile = base + s * kGemmStageBytes;
            const uint64_t desc_a0 = smem_descriptor(a_tile), desc_a1 = smem_descriptor(a_tile + kGemmABytes / 2);
            const uint64_t desc_b = smem_descriptor(a_tile + kGemmABytes);
            if (elect_one_lane()) {
#pragma unroll
                for (uint32_t kk = 0; kk < kGemmBK / 16; ++kk) {   // 16 bf16 = 32 bytes further along K inside the swizzle atom
                    tc_mma_bf16(tmem, desc_a0 + kk * 2, desc_b + kk * 2, idesc, (it | kk) != 0 ? 1u : 0u);
                    tc_mma_bf16(tmem + kGemmBN, desc_a1 + kk * 2, desc_b + kk * 2, idesc, (it | kk) != 0 ? 1u : 0u);
                }
                tc_commit(empty + 8 * s);   // frees the stage when these MMAs have read it
            }
            __syncwarp();
        }
        if (alive) {
            if (elect_one_lane()) tc_commit(accum);
            __syncwarp();
        } else {
            failed = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (failed && tid == 0) atomicOr(p.status, 2u);
    if (warp == kMmaWarp) tmem_free(tmem, kGemmTmemCols);
}

}  // namespace nc
