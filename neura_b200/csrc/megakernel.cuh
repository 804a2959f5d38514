// One persistent kernel for a whole decode step.
//
// The reference runs a step as one device "megakernel" that walks a list of task records
// (crates/neura-kernel/src/substrate.rs, crates/neura-runtime/src/runtime.rs:833-880).  This is the
// same idea for the decoder path on B200: one CTA per SM, launched cooperatively so that all of them
// are resident, walks a table of phases (embedding, products, attention, staging, argmax) and meets at
// a grid-wide barrier between phases.  What it buys over one launch per phase:
//   * no launch, fill and drain per phase: a phase boundary costs one barrier (about a microsecond);
//   * the weight stream never stops: before a warp arrives at a barrier it has already issued the
//     first copies of its next product, whose weights depend on nothing;
//   * rms_norm and the activation staging fold into the producers: the warp that completes a 256-column
//     chunk of a product's output (or of the attention's) digitises it at once for the next product
//     (prep.cuh, StageAfter), and the norm's scalar is applied by that product to its outputs.
// The products are the streaming product of gemv_mma.cuh (same units, same split, same ring).
//
// Every wait is bounded (the ring's copies and the grid barrier, by %globaltimer); a CTA whose wait
// runs out raises the status word, stops taking work and leaves, and so do the others at their next
// barrier.
#pragma once
#include "common.cuh"
#include "decoder_ops.cuh"
#include "gemv_mma.cuh"
#include "layout.cuh"
#include "prep.cuh"

namespace nc {

constexpr int kMkWarps = 16;
constexpr int kMkThreads = kMkWarps * 32;
constexpr uint32_t kMkRing = kMkWarps * 2 * kQ4kStage;        // two stages a warp (a Q8_0 stage is shorter)
constexpr uint32_t kMkBars = kMkWarps * 2 * 8;
constexpr uint32_t kMkPatch = kMkWarps * 32 * 9 * sizeof(float);
constexpr uint32_t kMkSmem = kMkRing + kMkBars + kMkPatch;
constexpr uint32_t kMkTile = 64;                              // cached positions one attention item takes
constexpr uint32_t kMkNone = 0xffffffffu;

enum : uint32_t { MK_EMBED = 1, MK_GEMV = 2, MK_ATTEND = 3, MK_STAGE = 4, MK_ARGMAX = 5, MK_CHOOSE = 6 };

struct MkPhase {
    uint32_t kind;
    uint32_t flags;          // MK_ARGMAX: 1 = leave the rows' winners for an MK_CHOOSE phase instead of writing the tokens
    uint32_t prefetch;       // the product whose first copies are issued when this phase ends, or kMkNone
    uint32_t k;              // columns of the input rows
    GemvParams g;            // MK_GEMV (dig, cs, sums: the staged input rows)
    StageAfter after;        // MK_GEMV, MK_ATTEND, MK_STAGE: how the rows this phase writes are staged for the next product
    uint32_t has_after, pad;
    const float *x;          // f32 input rows (MK_STAGE, MK_ARGMAX)
    uint64_t x_stride;
    float *keys, *values;    // MK_ATTEND: this layer's cache
    WeightView table;        // MK_EMBED
    float *out;              // MK_EMBED: rows of `out_stride`
    uint64_t out_stride;
    uint32_t lo, hi;         // MK_STAGE: the input is elements [lo, hi) of K, zero elsewhere
};

struct MkParams {
    const MkPhase *phases;
    uint32_t nphases;
    unsigned int *barrier;       // zero at launch
    unsigned int *status;
    uint32_t *tokens, *position; // [rows]
    uint32_t rows, granule;      // sequences; 256 (Q4_K) or 32 (Q8_0)
    // attention
    const float *qkv;            // [rows][qkv_stride]: q | k | v of this step
    uint64_t qkv_stride;
    float *attended;             // [rows][attended_stride]
    uint64_t attended_stride;
    float *attend_partial;       // [rows][heads][max_splits][width + 2]
    unsigned int *attend_counters;  // [rows][key_heads], zero between launches
    uint32_t heads, key_heads, width, capacity, max_splits;
    float scale, rope_base, floor;
    float2 *rope_table;          // [rows][width / 2]: the step's angles, written by the embedding phase
    // argmax
    float *slice_value;          // [rows][gridDim.x]
    uint32_t *slice_index;
    unsigned int *argmax_counters;  // [rows], zero between launches
    float *best_value;           // [rows]: this rank's winners, for the phase that picks among the ranks'
    uint32_t *best_index;
    unsigned long long *trace;   // [nphases + 1]: %globaltimer as CTA 0 enters each phase, and as it leaves the last
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid-wide barrier number `epoch` (1, 2, ...) of this launch.  The kernel is launched cooperatively,
// so every CTA is resident and will arrive; the wait is bounded all the same.  Returns false once this
// CTA has given up (now or earlier): the caller stops taking work.
__device__ __forceinline__ bool mk_barrier(const MkParams &p, uint32_t epoch, volatile uint32_t *aborted) {
    __syncthreads();
    if (threadIdx.x == 0 && !*aborted) {
        // arrivals count on one line, the release is a flag on another: the CTAs that wait read the flag's
        // line only and do not stand in the way of the arrivals still on their way
        unsigned int *flag = p.barrier + 32;
        __threadfence();
        const unsigned int before = atomicAdd(p.barrier, 1u);
        if (before + 1u == epoch * gridDim.x) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
        } else if (ld_acquire_gpu(flag) < epoch) {
            const unsigned long long start = global_nanos();
            for (;;) {
                bool met = false;
#pragma unroll 1
                for (int tries = 0; tries < 32 && !met; ++tries) met = ld_acquire_gpu(flag) >= epoch;
                if (met) break;
                if (global_nanos() - start > kWaitNanos) {
                    *aborted = 1u;
                    atomicOr(p.status, 2u);
                    break;
                }
            }
        }
        __threadfence();
        // a phase that gave up (a copy that never landed, a peer that never answered) has raised the status word:
        // what follows would compute on rows that are not there
        if (__ldcg(p.status)) *aborted = 1u;
    }
    __syncthreads();
    return *aborted == 0u;
}

// ---- activation fragments -----------------------------------------------------------------------------------
// load_frags of gemv_mma.cuh for one 8-column MMA tile.  Ordinary loads, so that the SM's L1 serves the warps
// that share a block of K: the fragments were written in an earlier phase, and the fence of the barrier
// between (mk_barrier) makes this SM's L1 drop what it held before.  (Not ld.global.nc: that path is for
// data no one writes during the kernel.)
template <bool Q4K>
__device__ __forceinline__ void mk_load_frags(StageFrags<Q4K, 1> &f, const GemvParams &s, uint32_t blk, uint32_t have) {
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int j = 0; j < StageFrags<Q4K, 1>::kUnits; ++j) {
        const uint32_t col = 2 * t;
        f.c[j][0][0] = col < s.ncols ? s.cs[blk * s.col_stride + s.col0 + col] : 0.0f;
        f.c[j][0][1] = col + 1 < s.ncols ? s.cs[blk * s.col_stride + s.col0 + col + 1] : 0.0f;
        const bool live = g < s.ncols;
        if constexpr (Q4K) {
            const uint32_t entry = (blk * s.col_stride + s.col0 + g) * 4 + t;
            const uint4 *from = reinterpret_cast<const uint4 *>(s.dig) + entry * 4u;
#pragma unroll
            for (int i = 0; i < 4; ++i) f.wide[0][i] = live ? from[i] : make_uint4(0u, 0u, 0u, 0u);
            f.sums[0] = live ? reinterpret_cast<const uint4 *>(s.sums)[entry] : make_uint4(0u, 0u, 0u, 0u);
        } else {
            f.narrow[j][0] = live ? *reinterpret_cast<const uint2 *>(s.dig + (blk * s.col_stride + s.col0 + g) * 32u + t * 8u)
                                  : make_uint2(0u, 0u);
        }
        if ((uint32_t)(j + 1) < have && ++blk == s.upt) blk = 0;
    }
}

// ---- products ----------------------------------------------------------------------------------------
// A warp's ring as it lives across the phases of one launch.
struct MkRing {
    uint32_t ring, bars;     // shared-memory addresses of this warp's two stages and their barriers
    uint32_t fills;          // stages filled and consumed so far (their number fixes stage and parity)
    uint32_t ahead_phase;    // the product whose first `ahead` stages are already on their way
    uint32_t ahead;
};

// The grid's warps are numbered across the CTAs (warp w of CTA c is w * gridDim.x + c): a product gives its
// first r warps one unit more than the rest, and this way every SM gets its share of them.
__device__ __forceinline__ uint32_t mk_warp() { return (threadIdx.x >> 5) * gridDim.x + blockIdx.x; }

// This warp's run of units in a product.
struct MkRun {
    const uint8_t *src;
    uint64_t bytes;
    uint32_t u0, units, steps;
};
template <bool Q4K>
__device__ __forceinline__ MkRun mk_run_of(const uint8_t *w, uint32_t nwarps, uint32_t q, uint32_t r, uint32_t warp) {
    constexpr uint32_t kUnit = Q4K ? kQ4kStage : 2 * kQ8Unit;
    constexpr uint32_t kGroup = Q4K ? 1 : kQ8Group;
    MkRun run;
    run.u0 = warp * q + min(warp, r);
    run.units = warp < nwarps ? q + (warp < r ? 1u : 0u) : 0u;
    run.steps = (run.units + kGroup - 1) / kGroup;
    run.src = w + (uint64_t)run.u0 * kUnit;
    run.bytes = (uint64_t)run.units * kUnit;
    return run;
}

// Issues fills [from, upto) of a run (lane 0 of the warp calls).
template <bool Q4K>
__device__ __forceinline__ void mk_issue(const MkRing &rg, const MkRun &run, uint32_t from, uint32_t upto) {
    constexpr uint32_t kStage = Q4K ? kQ4kStage : kQ8Stage;
    // the ring may have been written by ordinary stores (the attention phase borrows it)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (uint32_t i = from; i < upto; ++i) {
        const uint32_t stage = (rg.fills + i) & 1u;
        const uint64_t at = (uint64_t)i * kStage;
        const uint32_t len = (uint32_t)min((uint64_t)kStage, run.bytes - at);
        mbar_expect(rg.bars + stage * 8, len);
        bulk_load(rg.ring + stage * kStage, run.src + at, len, rg.bars + stage * 8);
    }
}

// Before a barrier: start the copies of the next product, whose weights depend on nothing.
template <bool Q4K>
__device__ __forceinline__ void mk_prefetch(const MkParams &p, uint32_t next, MkRing &rg) {
    if (next == kMkNone || rg.ahead_phase == next) return;   // (a phase before this one may have started them)
    const GemvParams &g = p.phases[next].g;
    const MkRun run = mk_run_of<Q4K>(g.w, g.nwarps, g.q, g.r, mk_warp());
    rg.ahead_phase = next;
    rg.ahead = min(run.steps, 2u);
    if ((threadIdx.x & 31) == 0) mk_issue<Q4K>(rg, run, 0, rg.ahead);
    __syncwarp();
}

template <bool Q4K>
__device__ __forceinline__ bool mk_stream(const GemvParams &g, MkRing &rg, const MkRun &run, float *patch, uint32_t warp,
                                          float scale0, float scale1) {
    constexpr uint32_t kGroup = Q4K ? 1 : kQ8Group;
    GemvWarp<Q4K, 1, 2, true> w{g};
    w.ring = rg.ring;
    w.bars = rg.bars;
    w.patch = patch;
    w.src = run.src;
    w.bytes = run.bytes;
    w.warp = warp;
    w.units = run.units;
    w.steps = run.steps;
    w.base = rg.fills;
    w.scale0 = scale0;
    w.scale1 = scale1;
    w.tile = run.u0 / g.upt;
    w.blk = run.u0 % g.upt;
    w.first_blk = w.blk;
    w.done = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) w.acc[h][0][0] = w.acc[h][0][1] = w.acc[h][0][2] = w.acc[h][0][3] = 0.0f;
    StageFrags<Q4K, 1> even, odd;
    mk_load_frags<Q4K>(even, g, w.blk, min(w.units, kGroup));
    uint32_t failed = kMkNone;
    for (uint32_t step = 0; step < w.steps; step += 2) {
        const bool second = step + 1 < w.steps;
        if (second) mk_load_frags<Q4K>(odd, g, w.block_after(w.blk), min(w.units - (step + 1) * kGroup, kGroup));
        if (!w.run(step, even)) { failed = step; break; }
        if (second) {
            if (step + 2 < w.steps) mk_load_frags<Q4K>(even, g, w.block_after(w.blk), min(w.units - (step + 2) * kGroup, kGroup));
            if (!w.run(step + 1, odd)) { failed = step + 1; break; }
        }
    }
    if (failed != kMkNone) {
        // a copy never landed: give the copies still in flight a bounded time before the memory is reused
        const uint32_t pending = min(2u, w.steps - failed);
        for (uint32_t s = 0; s < pending; ++s)
            mbar_wait(w.bars + ((w.base + failed + s) & 1u) * 8, ((w.base + failed + s) >> 1) & 1u);
        return false;
    }
    rg.fills += run.steps;
    return true;
}

// The rms_norm scalar of input row `row`: the chunks' sums of squares, added in chunk order.
__device__ __forceinline__ float mk_row_scale(const GemvParams &g, uint32_t row) {
    float total = 0.0f;
    for (uint32_t c = 0; c < g.sumsq_chunks; ++c) total += __ldcg(g.sumsq + row * g.sumsq_chunks + c);
    return 1.0f / sqrtf(total * g.inv_k + g.floor);
}

template <bool Q4K>
__device__ __noinline__ void mk_gemv(const MkParams &p, const MkPhase &ph, uint32_t index, MkRing &rg, float *patch,
                                        volatile uint32_t *aborted) {
    const uint32_t lane = threadIdx.x & 31, warp = mk_warp();
    const GemvParams &g = ph.g;
    const MkRun run = mk_run_of<Q4K>(g.w, g.nwarps, g.q, g.r, warp);
    const uint32_t ahead = rg.ahead_phase == index ? rg.ahead : 0u;
    if (lane == 0) mk_issue<Q4K>(rg, run, ahead, min(run.steps, 2u));
    rg.ahead_phase = kMkNone;
    __syncwarp();
    if (!run.units) return;
    float scale0 = 1.0f, scale1 = 1.0f;
    if (g.sumsq) {
        scale0 = mk_row_scale(g, 0);
        if (g.rows > 1) scale1 = mk_row_scale(g, 1);
    }
    if (!mk_stream<Q4K>(g, rg, run, patch, warp, scale0, scale1) && lane == 0) {
        atomicOr(p.status, 1u);
        *aborted = 1u;
    }
}

// ---- attention -----------------------------------------------------------------------------------------
// rope_cache_kernel and attend_kernel of decoder_ops.cuh as one phase.  An item is (sequence, key head,
// split of kMkTile cached positions); items are dealt round-robin to the CTAs.  Every item turns the
// query heads of its key head itself; the item whose split holds the new position turns the new key,
// puts it and the new value into its tile and into the cache.  Splits leave (largest logit, sum of
// exponentials, weighted values) per query head; the last split of a (sequence, key head) to arrive
// merges them in split order.  `shared` is the ring, idle during this phase.
template <uint32_t WIDTH>
__device__ __forceinline__ void mk_attend_item(const MkParams &p, const MkPhase &ph, float *shared, uint32_t *arrived,
                                               uint32_t b, uint32_t kh, uint32_t split, uint32_t splits, uint32_t position,
                                               uint32_t count) {
    constexpr uint32_t TILE = kMkTile, KROW = WIDTH + 4, HALF = WIDTH / 2;
    const uint32_t group = p.heads / p.key_heads;
    float *ks = shared;                                   // [TILE][KROW]
    float *vs = ks + TILE * KROW;                         // [TILE][WIDTH]
    float *qs = vs + TILE * WIDTH;                        // [group][WIDTH]
    float *logits = qs + kAttendMaxGroup * WIDTH;         // [group][kAttendMaxChunk]
    float *stats = logits + kAttendMaxGroup * kAttendMaxChunk;  // [group][2]
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const uint32_t first = split * TILE, last = min(first + TILE, count), held = last - first;
    const bool fresh = position < p.capacity && position >= first && position < last;   // the new row is ours
    const uint32_t fresh_row = position - first;
    const uint64_t slot0 = ((uint64_t)b * p.key_heads + kh) * p.capacity;
    const float *k = ph.keys + (slot0 + first) * WIDTH;
    const float *v = ph.values + (slot0 + first) * WIDTH;
    for (uint32_t i = threadIdx.x; i < held * (WIDTH / 4); i += blockDim.x) {
        const uint32_t row = i / (WIDTH / 4), quad = i % (WIDTH / 4);
        if (fresh && row == fresh_row) continue;
        copy16_async(ks + row * KROW + quad * 4, k + i * 4);
        copy16_async(vs + i * 4, v + i * 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float *row_qkv = p.qkv + (uint64_t)b * p.qkv_stride;
    for (uint32_t i = threadIdx.x; i < group * HALF; i += blockDim.x) {
        const uint32_t g = i / HALF, c = i % HALF;
        const float *q = row_qkv + (uint64_t)(kh * group + g) * WIDTH;
        const float2 turn = __ldcg(p.rope_table + b * HALF + c);
        const float2 turned = rope_turn(__ldcg(q + c), __ldcg(q + c + HALF), turn.x, turn.y);
        qs[g * WIDTH + c] = turned.x;
        qs[g * WIDTH + c + HALF] = turned.y;
    }
    if (fresh) {
        const float *nk = row_qkv + (uint64_t)(p.heads + kh) * WIDTH;
        const float *nv = row_qkv + (uint64_t)(p.heads + p.key_heads + kh) * WIDTH;
        float *cache_k = ph.keys + (slot0 + position) * WIDTH, *cache_v = ph.values + (slot0 + position) * WIDTH;
        // (the last threads of the CTA, so that they do not queue behind the query turns)
        for (uint32_t i = blockDim.x - 1 - threadIdx.x; i < HALF; i += blockDim.x) {
            const float2 turn = __ldcg(p.rope_table + b * HALF + i);
            const float2 turned = rope_turn(__ldcg(nk + i), __ldcg(nk + i + HALF), turn.x, turn.y);
            ks[fresh_row * KROW + i] = turned.x;
            ks[fresh_row * KROW + i + HALF] = turned.y;
            cache_k[i] = turned.x;
            cache_k[i + HALF] = turned.y;
        }
        for (uint32_t i = blockDim.x - 1 - threadIdx.x; i < WIDTH; i += blockDim.x) {
            const float value = __ldcg(nv + i);
            vs[fresh_row * WIDTH + i] = value;
            cache_v[i] = value;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    for (uint32_t item = threadIdx.x; item < group * held; item += blockDim.x) {
        const uint32_t g = item / held, pos = item % held;
        const float4 *kr = reinterpret_cast<const float4 *>(ks + pos * KROW);
        const float4 *qr = reinterpret_cast<const float4 *>(qs + g * WIDTH);
        float t0 = 0.0f, t1 = 0.0f, t2 = 0.0f, t3 = 0.0f;
#pragma unroll 8
        for (uint32_t c = 0; c < WIDTH / 4; ++c) {
            const float4 a = kr[c], q4 = qr[c];
            t0 = fmaf(a.x, q4.x, t0);
            t1 = fmaf(a.y, q4.y, t1);
            t2 = fmaf(a.z, q4.z, t2);
            t3 = fmaf(a.w, q4.w, t3);
        }
        logits[g * kAttendMaxChunk + pos] = ((t0 + t1) + (t2 + t3)) * p.scale;
    }
    __syncthreads();
    for (uint32_t g = warp; g < group; g += warps) {
        float largest = -INFINITY;
        for (uint32_t i = lane; i < held; i += 32) largest = fmaxf(largest, logits[g * kAttendMaxChunk + i]);
        for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
        float sum = 0.0f;
        for (uint32_t i = lane; i < held; i += 32) {
            const float e = expf(logits[g * kAttendMaxChunk + i] - largest);
            logits[g * kAttendMaxChunk + i] = e;
            sum += e;
        }
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) { stats[g * 2] = largest; stats[g * 2 + 1] = sum; }
    }
    __syncthreads();
    float *mine = p.attend_partial + ((uint64_t)b * p.heads + kh * group) * p.max_splits * (WIDTH + 2);
    // weighted values: one thread per (query head, channel)
    for (uint32_t item = threadIdx.x; item < group * WIDTH; item += blockDim.x) {
        const uint32_t g = item / WIDTH, d = item % WIDTH;
        float acc = 0.0f;
        for (uint32_t pos = 0; pos < held; ++pos) acc = fmaf(logits[g * kAttendMaxChunk + pos], vs[pos * WIDTH + d], acc);
        __stcg(mine + ((uint64_t)g * p.max_splits + split) * (WIDTH + 2) + d, acc);
    }
    if (threadIdx.x < group * 2) {
        const uint32_t g = threadIdx.x / 2, which = threadIdx.x % 2;
        __stcg(mine + ((uint64_t)g * p.max_splits + split) * (WIDTH + 2) + WIDTH + which, stats[g * 2 + which]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *arrived = arrive_on(p.attend_counters + b * p.key_heads + kh);
    }
    __syncthreads();
    if (*arrived == splits - 1) {
        float *factor = logits;   // [group][splits]
        float *sums = ks;         // [group][splits]
        float *totals = stats;    // [group]
        for (uint32_t i = threadIdx.x; i < group * splits; i += blockDim.x) {
            const float *from = mine + ((uint64_t)(i / splits) * p.max_splits + i % splits) * (WIDTH + 2) + WIDTH;
            factor[(i / splits) * kAttendMaxChunk + i % splits] = __ldcg(from);
            sums[(i / splits) * kAttendMaxChunk + i % splits] = __ldcg(from + 1);
        }
        __syncthreads();
        for (uint32_t g = warp; g < group; g += warps) {
            float largest = -INFINITY;
            for (uint32_t s = lane; s < splits; s += 32) largest = fmaxf(largest, factor[g * kAttendMaxChunk + s]);
            for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
            float total = 0.0f;
            for (uint32_t s = lane; s < splits; s += 32) {
                const float m = factor[g * kAttendMaxChunk + s];
                const float f = m == -INFINITY ? 0.0f : expf(m - largest);
                factor[g * kAttendMaxChunk + s] = f;
                total = fmaf(sums[g * kAttendMaxChunk + s], f, total);
            }
            for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0) totals[g] = total;
        }
        __syncthreads();
        for (uint32_t item = threadIdx.x; item < group * WIDTH; item += blockDim.x) {
            const uint32_t g = item / WIDTH, d = item % WIDTH;
            float acc = 0.0f;
            for (uint32_t s = 0; s < splits; ++s)
                acc = fmaf(__ldcg(mine + ((uint64_t)g * p.max_splits + s) * (WIDTH + 2) + d), factor[g * kAttendMaxChunk + s], acc);
            p.attended[(uint64_t)b * p.attended_stride + (uint64_t)(kh * group + g) * WIDTH + d] = acc / totals[g];
        }
        if (threadIdx.x == 0) p.attend_counters[b * p.key_heads + kh] = 0u;
        if (ph.has_after) {
            // the heads of this key head are columns [kh, kh + 1) * group * WIDTH of the row the output product
            // multiplies: count this arrival on the 256-column chunks they touch; whoever completes a chunk stages it
            __syncthreads();
            // (on a rank of a tensor-parallel group the row sits at [lo, hi) of the axis of K, see StageAfter)
            const StageAfter &a = ph.after;
            const uint32_t span = group * WIDTH, chunks = (a.prep.k + 255) / 256, lo = a.prep.lo;
            const uint32_t c0 = (lo + kh * span) / 256, c1 = (lo + (kh + 1) * span - 1) / 256;
            for (uint32_t c = c0 + warp; c <= c1; c += warps) {
                // the key heads whose columns reach into chunk c
                const uint32_t from = max(c * 256, lo) - lo, upto = min(a.prep.hi, (c + 1) * 256) - lo;
                const uint32_t expected = (upto - 1) / span - from / span + 1;
                unsigned int seen = 0;
                if (lane == 0) {
                    seen = arrive_on(a.counters + b * chunks + c);
                }
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen == expected - 1) {
                    stage_after_chunk(a, b, c);
                    if (lane == 0) a.counters[b * chunks + c] = 0u;
                }
            }
        }
    }
    __syncthreads();   // the tile is free for the CTA's next item
}

template <uint32_t WIDTH>
__device__ __forceinline__ void mk_attend(const MkParams &p, const MkPhase &ph, float *shared, uint32_t *arrived) {
    uint32_t dealt = 0;   // items of the sequences before this one
    for (uint32_t b = 0; b < p.rows; ++b) {
        const uint32_t position = __ldcg(p.position + b);
        const uint32_t count = min(position + 1, p.capacity);
        const uint32_t splits = (count + kMkTile - 1) / kMkTile;
        const uint32_t items = p.key_heads * splits;
        const uint32_t skip = (blockIdx.x + gridDim.x - dealt % gridDim.x) % gridDim.x;
        for (uint32_t i = skip; i < items; i += gridDim.x)
            mk_attend_item<WIDTH>(p, ph, shared, arrived, b, i / splits, i % splits, splits, position, count);
        dealt += items;
    }
}


// ---- the small phases -------------------------------------------------------------------------------------
// A staging pass of its own (after the embedding gather, whose rows no product wrote): one warp per
// (row, 256 columns) of ph.after.
__device__ __forceinline__ void mk_stage(const MkParams &p, const MkPhase &ph) {
    const uint32_t chunks = (ph.after.prep.k + 255) / 256, total = p.rows * chunks;
    for (uint32_t w = blockIdx.x * kMkWarps + (threadIdx.x >> 5); w < total; w += gridDim.x * kMkWarps)
        stage_after_chunk(ph.after, w / chunks, w % chunks);
}

// embed_kernel as a phase.
__device__ __forceinline__ void mk_embed(const MkParams &p, const MkPhase &ph) {
    const uint32_t total = p.rows * ph.table.k;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t r = idx / ph.table.k, at = idx % ph.table.k;
        const uint32_t row = min(__ldcg(p.tokens + r), ph.table.n - 1);
        ph.out[(uint64_t)r * ph.out_stride + at] = dequant_at(ph.table, row, at);
    }
    // the step's RoPE angles, the same in every layer (the last CTA has the least to gather)
    if (blockIdx.x == gridDim.x - 1) {
        const uint32_t half = p.width / 2;
        for (uint32_t i = threadIdx.x; i < p.rows * half; i += blockDim.x)
            p.rope_table[i] = rope_angle(__ldcg(p.position + i / half), i % half, p.width, p.rope_base);
    }
}

// argmax_kernel and advance_kernel as the last phase: every CTA takes a slice of every row, the last CTA
// to arrive at a row picks among the slices (lowest index on ties), writes the token and moves the cursor.
__device__ __forceinline__ void mk_argmax(const MkParams &p, const MkPhase &ph, float *best_value, uint32_t *best_index,
                                          uint32_t *arrived) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per = (ph.k + gridDim.x - 1) / gridDim.x;
    const uint32_t first = min(blockIdx.x * per, ph.k), last = min(first + per, ph.k);
    for (uint32_t row = 0; row < p.rows; ++row) {
        const float *x = ph.x + (uint64_t)row * ph.x_stride;
        float value = -INFINITY;
        uint32_t index = 0xffffffffu;
        for (uint32_t c = first + threadIdx.x; c < last; c += blockDim.x) argmax_take(value, index, __ldcg(x + c), c);
        for (int o = 16; o; o >>= 1)
            argmax_take(value, index, __shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
        __syncthreads();   // the row before has been read out of the tables
        if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) argmax_take(value, index, best_value[w], best_index[w]);
            __stcg(p.slice_value + row * gridDim.x + blockIdx.x, value);
            __stcg(p.slice_index + row * gridDim.x + blockIdx.x, index);
            *arrived = arrive_on(p.argmax_counters + row);
        }
        __syncthreads();
        if (*arrived == gridDim.x - 1 && warp == 0) {
            value = -INFINITY;
            index = 0xffffffffu;
            for (uint32_t s = lane; s < gridDim.x; s += 32)
                argmax_take(value, index, __ldcg(p.slice_value + row * gridDim.x + s), __ldcg(p.slice_index + row * gridDim.x + s));
            for (int o = 16; o; o >>= 1)
                argmax_take(value, index, __shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
            if (lane == 0) {
                if (ph.flags & 1u) {
                    __stcg(p.best_value + row, value);
                    __stcg(p.best_index + row, index);
                } else {
                    p.tokens[row] = index == 0xffffffffu ? 0u : index;
                    p.position[row] = __ldcg(p.position + row) + 1u;
                }
                p.argmax_counters[row] = 0u;
            }
        }
    }
}

// The last phase on a rank of a tensor-parallel group, whose head holds rows [rank, rank + 1) * ph.k of the
// vocabulary: warp 0 of CTA 0 gathers the ranks' winners of every row (an exchange of a vector that is zero except
// for this rank's (value, index) pair, so the sum over the ranks is the list of pairs), picks among them (lowest
// index on ties, as one device would), writes the token and moves the cursor.  Every rank computes the same.
__device__ __forceinline__ void mk_choose(const MkParams &p, const MkPhase &ph) {
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    const uint32_t lane = threadIdx.x;
    const ExchangeView &e = *ph.after.exchange;
    for (uint32_t row = 0; row < p.rows; ++row) {
        const float value = __ldcg(p.best_value + row);
        const uint32_t index = __ldcg(p.best_index + row);
        // pair r sits at numbers [2 r, 2 r + 2) of the vector: lane r / 4, numbers 2 (r % 4) of its eight
        float mine8[8];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const bool here = lane * 4 + i == e.rank;
            mine8[2 * i] = here ? value : 0.0f;
            mine8[2 * i + 1] = here ? (float)(index == 0xffffffffu ? 0u : index + e.rank * ph.k) : 0.0f;   // (exact below 2^24)
        }
        if (!exchange_chunk(e, 0, 0, 1, mine8, ph.after.wait_nanos, ph.after.status)) return;
        float best = -INFINITY;
        uint32_t chosen = 0xffffffffu;
#pragma unroll
        for (uint32_t r = 0; r < kMaxRanks; ++r) {
            const float v = __shfl_sync(0xffffffffu, mine8[2 * (r % 4)], r / 4);
            const float at = __shfl_sync(0xffffffffu, mine8[2 * (r % 4) + 1], r / 4);
            if (r < e.world) argmax_take(best, chosen, v, (uint32_t)at);
        }
        if (lane == 0) {
            p.tokens[row] = chosen == 0xffffffffu ? 0u : chosen;
            p.position[row] = __ldcg(p.position + row) + 1u;
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------------------------------
template <bool Q4K>
__global__ void __launch_bounds__(kMkThreads, 1) decode_megakernel(const __grid_constant__ MkParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) MkPhase phase;
    __shared__ float reduce[kMkWarps];
    __shared__ uint32_t best_index[kMkWarps];
    __shared__ uint32_t arrived;
    __shared__ volatile uint32_t aborted;
    const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    constexpr uint32_t kStage = Q4K ? kQ4kStage : kQ8Stage;
    MkRing rg;
    rg.ring = smem_addr(smem) + wib * 2 * kStage;
    rg.bars = smem_addr(smem) + kMkRing + wib * 16;
    rg.fills = 0;
    rg.ahead_phase = kMkNone;
    rg.ahead = 0;
    float *patch = reinterpret_cast<float *>(smem + kMkRing + kMkBars) + wib * 32 * 9;
    if (threadIdx.x == 0) aborted = 0u;
    if (lane == 0) {
        mbar_init(rg.bars, 1);
        mbar_init(rg.bars + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    for (uint32_t index = 0; index < p.nphases; ++index) {
        {
            const uint32_t *from = reinterpret_cast<const uint32_t *>(p.phases + index);
            uint32_t *to = reinterpret_cast<uint32_t *>(&phase);
            for (uint32_t i = threadIdx.x; i < sizeof(MkPhase) / 4; i += blockDim.x) to[i] = __ldg(from + i);
        }
        __syncthreads();
        if (aborted) break;
        if (blockIdx.x == 0 && threadIdx.x == 0) p.trace[index] = global_nanos();
        switch (phase.kind) {
        case MK_EMBED: mk_embed(p, phase); break;
        case MK_GEMV: mk_gemv<Q4K>(p, phase, index, rg, patch, &aborted); break;
        case MK_ATTEND:
            if (p.width == 128) mk_attend<128>(p, phase, reinterpret_cast<float *>(smem), &arrived);
            else mk_attend<64>(p, phase, reinterpret_cast<float *>(smem), &arrived);
            break;
        case MK_STAGE: mk_stage(p, phase); break;
        case MK_ARGMAX: mk_argmax(p, phase, reduce, best_index, &arrived); break;
        case MK_CHOOSE: mk_choose(p, phase); break;
        default: break;
        }
        if (index + 1 == p.nphases) break;   // nothing follows the last phase
        __syncthreads();                     // the CTA is done with the ring and with `phase`
        mk_prefetch<Q4K>(p, phase.prefetch, rg);
        if (!mk_barrier(p, index + 1, &aborted)) break;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) p.trace[p.nphases] = global_nanos();
    // copies issued ahead of a product that never ran: let them land before the memory is handed back
    if (rg.ahead_phase != kMkNone) {
        for (uint32_t s = 0; s < rg.ahead; ++s) mbar_wait(rg.bars + ((rg.fills + s) & 1u) * 8, ((rg.fills + s) >> 1) & 1u);
    }
}

}  // namespace nc
