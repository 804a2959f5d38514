// The steps either side of the products in a decoder layer: RoPE with the KV-cache write,
// grouped-query attention of one new row over the cache, argmax, and the gather of a
// quantised embedding row.  (rms_norm lives in prep.cuh, fused with the activation staging.)
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "layout.cuh"

namespace nc {

// rope (crates/neura-kernel/src/task/rope.rs:48-122, half rotation) on the query and key
// thirds of a fused q|k|v row, then Cache::write (crates/neura-decoder/src/cache.rs:267-310):
// the turned key and the value go to slot position[b] of their sequence's cache.
struct RopeCacheParams {
    float *qkv;               // [batch][row_stride]: q (heads*width) | k (key_heads*width) | v (key_heads*width)
    uint64_t row_stride;
    const uint32_t *position; // [batch]
    float *keys, *values;     // [batch][key_heads][capacity][width]
    float base;
    uint32_t batch, heads, key_heads, width, capacity;
    uint32_t shared;          // 1: every row belongs to ONE sequence, whose cache starts at keys / values (a prompt chunk)
};

// Half-rotation of one channel pair by (cosine, sine), every rounding pinned so that all callers agree bit for bit.
__device__ __forceinline__ float2 rope_turn(float low, float high, float cosine, float sine) {
    return make_float2(__fmaf_rn(low, cosine, -__fmul_rn(high, sine)), __fmaf_rn(high, cosine, __fmul_rn(low, sine)));
}

// (cosine, sine) of a position's angle in one channel.
__device__ __forceinline__ float2 rope_angle_inline(uint32_t position, uint32_t channel, uint32_t width, float base) {
    const float angle = (float)position * powf(base, -2.0f * (float)channel / (float)width);
    return make_float2(cosf(angle), sinf(angle));
}
// The same out of line, for callers whose loops should not carry the stack frame that the slow paths of powf,
// cosf and sinf want.
__device__ __noinline__ float2 rope_angle(uint32_t position, uint32_t channel, uint32_t width, float base) {
    return rope_angle_inline(position, channel, width, base);
}

__device__ __forceinline__ float2 rope_pair(float low, float high, uint32_t position, uint32_t channel, uint32_t width,
                                            float base) {
    const float2 turn = rope_angle_inline(position, channel, width, base);
    return rope_turn(low, high, turn.x, turn.y);
}

// The angles of one decode step: table[b][channel] = (cosine, sine) of position[b] in that channel.  They are the
// same in every layer, so a step computes them once (rope_attend reads them).
__global__ void rope_table_kernel(const uint32_t *position, float base, uint32_t batch, uint32_t width, float2 *table) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t half = width / 2;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < batch * half; i += gridDim.x * blockDim.x)
        table[i] = rope_angle(position[i / half], i % half, width, base);
}

__global__ void rope_cache_kernel(const __grid_constant__ RopeCacheParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t half = p.width / 2;
    const uint32_t turned = (p.heads + p.key_heads) * half;   // pairs to rotate per row
    const uint32_t copied = p.key_heads * p.width;            // values to store per row
    const uint32_t per_row = turned + copied;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < p.batch * per_row; idx += gridDim.x * blockDim.x) {
        const uint32_t b = idx / per_row, at = idx % per_row;
        float *row = p.qkv + (uint64_t)b * p.row_stride;
        const uint32_t position = p.position[b];
        if (at < turned) {
            const uint32_t head = at / half, channel = at % half;
            float *v = row + (uint64_t)head * p.width;   // key heads follow the query heads in the row
            const float2 turned = rope_pair(v[channel], v[channel + half], position, channel, p.width, p.base);
            const float new_low = turned.x, new_high = turned.y;
            v[channel] = new_low;
            v[channel + half] = new_high;
            if (head >= p.heads && position < p.capacity) {
                const uint32_t kh = head - p.heads;
                float *slot = p.keys + (((uint64_t)(p.shared ? 0 : b) * p.key_heads + kh) * p.capacity + position) * p.width;
                slot[channel] = new_low;
                slot[channel + half] = new_high;
            }
        } else if (position < p.capacity) {
            const uint32_t c = at - turned, kh = c / p.width, d = c % p.width;
            const float value = row[(uint64_t)(p.heads + p.key_heads) * p.width + c];
            p.values[(((uint64_t)(p.shared ? 0 : b) * p.key_heads + kh) * p.capacity + position) * p.width + d] = value;
        }
    }
}

// Cache::attend for one new row per sequence (crates/neura-decoder/src/cache.rs:311-406 over
// crates/neura-kernel/src/task/attention.rs:309-617): softmax(q.k * scale) v with query head h
// reading key head h / (heads / key_heads); positions 0..position[b] are live.
//
// One CTA per (sequence, key head, split of the positions): the query heads that share the key
// head are served together, so keys and values are read once.  Each CTA leaves, per query head,
// its partial (largest logit, sum of exponentials, weighted values); the last CTA of a
// (sequence, key head) to arrive merges the splits in order (the reference's key-split attention
// with its AttentionFold merge, crates/neura-abi/src/kind.rs:638-645).
constexpr uint32_t kAttendMaxGroup = 8;    // query heads per key head
constexpr uint32_t kAttendMaxChunk = 128;  // row length of the per-head logit and merge tables (>= tile, >= splits)
constexpr uint32_t kAttendMaxCluster = 8;  // splits that merge through distributed shared memory
#ifndef NC_ATTEND_THREADS
#define NC_ATTEND_THREADS 256
#endif
constexpr uint32_t kAttendThreads = NC_ATTEND_THREADS;

struct AttendParams {
    const float *q;           // [batch][q_stride], head h at h*width
    uint64_t q_stride;
    const float *keys, *values;   // [batch][key_heads][capacity][width]
    const uint32_t *position;
    float *out;               // [batch][out_stride]
    uint64_t out_stride;
    float *partial;           // [batch][heads][splits][width + 2]
    unsigned int *counters;   // [batch][key_heads], zero between launches
    float scale;
    uint32_t batch, heads, key_heads, width, capacity, splits;
    // rope_cache_kernel folded in: when `fresh` is not null, q points at the un-turned q | k | v rows of this
    // step; the queries are turned as they are loaded, and the split that holds the new position turns the new
    // key and puts it and the new value into its tile and into the cache (`fresh` = the cache, writable)
    float *fresh_keys, *fresh_values;
    const float2 *rope_table;   // [batch][width / 2] (cosine, sine) of each sequence's position (rope_table_kernel)
    uint32_t shared;            // 1: every row belongs to ONE sequence, whose cache starts at keys / values (a prompt chunk)
};

__device__ __forceinline__ void copy16_async(void *dst_shared, const void *src_global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)),
                 "l"(src_global)
                 : "memory");
}

// WIDTH is the head width (64 or 128).  The split's keys and values (contiguous in the cache)
// are copied to shared memory with asynchronous 16-byte copies, all in flight at once, so the
// cache costs one memory round trip per CTA.
// TILE is the number of positions one CTA takes (64 or 128).  With CLUSTER the splits of one
// (sequence, key head) form a thread-block cluster and merge their partials through distributed
// shared memory behind a cluster barrier; otherwise they merge through global memory, the last
// CTA to arrive doing the work.
template <uint32_t WIDTH, uint32_t TILE, bool CLUSTER, bool TURNING>
__global__ void __launch_bounds__(kAttendThreads) attend_kernel(const __grid_constant__ AttendParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ __align__(16) float shared[];
    const uint32_t group = p.heads / p.key_heads;
    constexpr uint32_t KROW = WIDTH + 4;                 // padded key row: float4 reads of 8 rows hit 32 banks
    float *ks = shared;                                  // [TILE][KROW]
    float *vs = ks + TILE * KROW;                 // [TILE][WIDTH]
    float *qs = vs + TILE * WIDTH;                // [group][WIDTH]
    float *logits = qs + kAttendMaxGroup * WIDTH;        // [group][kAttendMaxChunk]
    float *stats = logits + kAttendMaxGroup * kAttendMaxChunk;  // [group][2]: largest, sum
    __shared__ unsigned int arrived;
    const uint32_t split = blockIdx.x % p.splits;
    const uint32_t kh = (blockIdx.x / p.splits) % p.key_heads;
    const uint32_t b = blockIdx.x / (p.splits * p.key_heads);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const uint32_t count = min(p.position[b] + 1, p.capacity);
    const uint32_t chunk = min((count + p.splits - 1) / p.splits, TILE);
    // (the host sizes `splits` so that capacity / splits <= TILE)
    const uint32_t first = min(split * chunk, count), last = min(first + chunk, count), held = last - first;
    const uint32_t sequence = p.shared ? 0u : b;
    const float *k = p.keys + (((uint64_t)sequence * p.key_heads + kh) * p.capacity + first) * WIDTH;
    const float *v = p.values + (((uint64_t)sequence * p.key_heads + kh) * p.capacity + first) * WIDTH;
    const uint32_t position = p.position[b];
    constexpr bool turning = TURNING;   // (the plain instantiation carries none of the folded-in RoPE)
    const bool fresh = turning && position < p.capacity && position >= first && position < last;  // the new row is ours
    const uint32_t fresh_row = position - first;
    for (uint32_t i = threadIdx.x; i < held * (WIDTH / 4); i += blockDim.x) {
        const uint32_t row = i / (WIDTH / 4), quad = i % (WIDTH / 4);
        if (fresh && row == fresh_row) continue;
        copy16_async(ks + row * KROW + quad * 4, k + i * 4);
        copy16_async(vs + i * 4, v + i * 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if constexpr (TURNING) {
        constexpr uint32_t HALF = WIDTH / 2;
        const float *row_qkv = p.q + (uint64_t)b * p.q_stride;
        for (uint32_t i = threadIdx.x; i < group * HALF; i += blockDim.x) {
            const uint32_t g = i / HALF, c = i % HALF;
            const float *q = row_qkv + (uint64_t)(kh * group + g) * WIDTH;
            const float2 turn = p.rope_table[b * HALF + c];
            const float2 turned = rope_turn(q[c], q[c + HALF], turn.x, turn.y);
            qs[g * WIDTH + c] = turned.x;
            qs[g * WIDTH + c + HALF] = turned.y;
        }
        if (fresh) {
            const float *nk = row_qkv + (uint64_t)(p.heads + kh) * WIDTH;
            const float *nv = row_qkv + (uint64_t)(p.heads + p.key_heads + kh) * WIDTH;
            const uint64_t slot = (((uint64_t)sequence * p.key_heads + kh) * p.capacity + position) * WIDTH;
            for (uint32_t i = blockDim.x - 1 - threadIdx.x; i < HALF; i += blockDim.x) {   // (the threads the queries use least)
                const float2 turn = p.rope_table[b * HALF + i];
                const float2 turned = rope_turn(nk[i], nk[i + HALF], turn.x, turn.y);
                ks[fresh_row * KROW + i] = turned.x;
                ks[fresh_row * KROW + i + HALF] = turned.y;
                p.fresh_keys[slot + i] = turned.x;
                p.fresh_keys[slot + i + HALF] = turned.y;
            }
            for (uint32_t i = blockDim.x - 1 - threadIdx.x; i < WIDTH; i += blockDim.x) {
                const float value = nv[i];
                vs[fresh_row * WIDTH + i] = value;
                p.fresh_values[slot + i] = value;
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < group * WIDTH; i += blockDim.x)
            qs[i] = p.q[(uint64_t)b * p.q_stride + (uint64_t)(kh * group) * WIDTH + i];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // logits of this split: one thread per (query head, position), the whole dot product in registers
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
    // per query head: largest logit and sum of exponentials of the split (one warp per head)
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
    // weighted values: a thread per channel, every value row read once for all the group's heads.  With at least
    // 2 * WIDTH threads two threads share a channel, one taking the even positions and one the odd; the odd half
    // hands its sums over through the query rows (no longer needed) and the even half adds them.
    {
        const uint32_t parts = blockDim.x >= 2 * WIDTH ? 2u : 1u;
        const uint32_t part = threadIdx.x / WIDTH, d = threadIdx.x % WIDTH;
        float acc[kAttendMaxGroup];
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g) acc[g] = 0.0f;
        if (part < parts) {
            for (uint32_t pos = part; pos < held; pos += parts) {
                const float value = vs[pos * WIDTH + d];
#pragma unroll
                for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                    if (g < group) acc[g] = fmaf(logits[g * kAttendMaxChunk + pos], value, acc[g]);
            }
        }
        if (parts == 2) {
            if (part == 1) {
#pragma unroll
                for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                    if (g < group) qs[g * WIDTH + d] = acc[g];
            }
            __syncthreads();
            if (part == 0) {
#pragma unroll
                for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                    if (g < group) acc[g] += qs[g * WIDTH + d];
            }
        }
        if (part == 0) {
            if constexpr (CLUSTER) {
                // (every thread of the CTA is past the logits phase, which was the last reader of the key tile)
#pragma unroll
                for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                    if (g < group) ks[g * WIDTH + d] = acc[g];
            } else {
#pragma unroll
                for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                    if (g < group)
                        __stcg(p.partial + (((uint64_t)b * p.heads + kh * group + g) * p.splits + split) * (WIDTH + 2) + d, acc[g]);
            }
        }
    }
    if constexpr (CLUSTER) {
        // every split's partial sits in its CTA's shared memory; each CTA merges a slice of the channels
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const uint32_t per = (WIDTH + p.splits - 1) / p.splits;
        const uint32_t d0 = min(split * per, WIDTH), d1 = min(d0 + per, WIDTH);
        for (uint32_t item = threadIdx.x; item < group * (d1 - d0); item += blockDim.x) {
            const uint32_t g = item / (d1 - d0), d = d0 + item % (d1 - d0);
            float largest = -INFINITY;
            for (uint32_t s2 = 0; s2 < p.splits; ++s2) largest = fmaxf(largest, cluster.map_shared_rank(stats, s2)[g * 2]);
            float total = 0.0f, acc = 0.0f;
            for (uint32_t s2 = 0; s2 < p.splits; ++s2) {
                const float m = cluster.map_shared_rank(stats, s2)[g * 2];
                const float f = m == -INFINITY ? 0.0f : expf(m - largest);
                total = fmaf(cluster.map_shared_rank(stats, s2)[g * 2 + 1], f, total);
                acc = fmaf(cluster.map_shared_rank(ks, s2)[g * WIDTH + d], f, acc);
            }
            p.out[(uint64_t)b * p.out_stride + (uint64_t)(kh * group + g) * WIDTH + d] = acc / total;
        }
        cluster.sync();   // no CTA leaves while its shared memory may still be read
        return;
    }
    if (threadIdx.x < group * 2) {
        const uint32_t g = threadIdx.x / 2, which = threadIdx.x % 2;
        __stcg(p.partial + (((uint64_t)b * p.heads + kh * group + g) * p.splits + split) * (WIDTH + 2) + WIDTH + which,
               stats[g * 2 + which]);
    }
    // the last split of this (sequence, key head) to arrive merges them all, in split order
    __syncthreads();
    if (threadIdx.x == 0) {
        arrived = arrive_on(p.counters + b * p.key_heads + kh);
    }
    __syncthreads();
    if (arrived != p.splits - 1) return;
    // merge: every load of a phase is issued before its first use, so each phase costs one round trip
    float *factor = logits;                    // [group][splits] (splits <= kAttendMaxChunk)
    float *sums = ks;                          // [group][splits], the key tile is no longer needed
    float *totals = stats;                     // [group]
    const float *mine = p.partial + ((uint64_t)b * p.heads + kh * group) * p.splits * (p.width + 2);
    for (uint32_t i = threadIdx.x; i < group * p.splits; i += blockDim.x) {
        factor[(i / p.splits) * kAttendMaxChunk + i % p.splits] = __ldcg(mine + (uint64_t)i * (p.width + 2) + p.width);
        sums[(i / p.splits) * kAttendMaxChunk + i % p.splits] = __ldcg(mine + (uint64_t)i * (p.width + 2) + p.width + 1);
    }
    __syncthreads();
    for (uint32_t g = warp; g < group; g += warps) {
        float largest = -INFINITY;
        for (uint32_t s = lane; s < p.splits; s += 32) largest = fmaxf(largest, factor[g * kAttendMaxChunk + s]);
        for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
        float total = 0.0f;
        for (uint32_t s = lane; s < p.splits; s += 32) {
            const float m = factor[g * kAttendMaxChunk + s];
            const float f = m == -INFINITY ? 0.0f : expf(m - largest);
            factor[g * kAttendMaxChunk + s] = f;
            total = fmaf(sums[g * kAttendMaxChunk + s], f, total);
        }
        for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) totals[g] = total;
    }
    __syncthreads();
    // one thread per channel; the partial rows of eight splits of every head of the group travel together
    for (uint32_t d = threadIdx.x; d < p.width; d += blockDim.x) {
        float acc[kAttendMaxGroup];
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g) acc[g] = 0.0f;
        for (uint32_t s = 0; s < p.splits; s += 8) {
            float part[kAttendMaxGroup][8];
#pragma unroll
            for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    part[g][u] = (g < group && s + u < p.splits)
                        ? __ldcg(mine + ((uint64_t)g * p.splits + s + u) * (p.width + 2) + d) : 0.0f;
#pragma unroll
            for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (g < group && s + u < p.splits) acc[g] = fmaf(part[g][u], factor[g * kAttendMaxChunk + s + u], acc[g]);
        }
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
            if (g < group)
                p.out[(uint64_t)b * p.out_stride + (uint64_t)(kh * group + g) * p.width + d] = acc[g] / totals[g];
    }
    if (threadIdx.x == 0) p.counters[b * p.key_heads + kh] = 0u;
}

// argmax, the lowest index winning a tie (choice_precedes, crates/neura-kernel/src/task/choice.rs:46-52).
// A row is shared by `slices` CTAs; the last of them to arrive merges their candidates.
struct ArgmaxParams {
    const float *x;
    uint64_t stride;             // between rows
    uint64_t segment_stride;     // column c of a row lives at (c / segment) * segment_stride + c % segment
    uint32_t segment;            // (a row gathered from several ranks is split in segments; else segment = width)
    uint32_t width, slices;
    uint32_t *out;
    float *slice_value;          // [rows][slices]
    uint32_t *slice_index;       // [rows][slices]
    unsigned int *counters;      // [rows], zero between launches
};

__device__ __forceinline__ void argmax_take(float &value, uint32_t &index, float other, uint32_t other_index) {
    if (other > value || (other == value && other_index < index)) { value = other; index = other_index; }
}

__global__ void __launch_bounds__(256) argmax_kernel(const __grid_constant__ ArgmaxParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float best_value[8];
    __shared__ uint32_t best_index[8];
    __shared__ unsigned int arrived;
    const uint32_t row = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
    const float *x = p.x + (uint64_t)row * p.stride;
    const uint32_t per = (p.width + p.slices - 1) / p.slices;
    const uint32_t first = slice * per, last = min(first + per, p.width);
    float value = -INFINITY;
    uint32_t index = 0xffffffffu;
    for (uint32_t c = first + threadIdx.x; c < last; c += blockDim.x * 8) {   // eight loads in flight per thread
        float other[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t at = c + u * blockDim.x;
            other[u] = at < last ? x[(uint64_t)(at / p.segment) * p.segment_stride + at % p.segment] : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) argmax_take(value, index, other[u], c + u * blockDim.x);
    }
    for (int o = 16; o; o >>= 1)
        argmax_take(value, index, __shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) argmax_take(value, index, best_value[w], best_index[w]);
        __stcg(p.slice_value + row * p.slices + slice, value);
        __stcg(p.slice_index + row * p.slices + slice, index);
        arrived = arrive_on(p.counters + row);
    }
    __syncthreads();
    if (arrived != p.slices - 1 || warp != 0) return;
    value = -INFINITY;
    index = 0xffffffffu;
    for (uint32_t s = lane; s < p.slices; s += 32)
        argmax_take(value, index, __ldcg(p.slice_value + row * p.slices + s), __ldcg(p.slice_index + row * p.slices + s));
    for (int o = 16; o; o >>= 1)
        argmax_take(value, index, __shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
    if (lane == 0) {
        p.out[row] = index == 0xffffffffu ? 0u : index;
        p.counters[row] = 0u;
    }
}

// run_gather over a quantised table (crates/neura-kernel/src/task/select.rs:29-49 with fetch_q8_0 /
// fetch_q4_k, fetch.rs:236-267): out[r] = the dequantised row tokens[r], bit-exact, either layout.
__global__ void embed_kernel(WeightView table, const uint32_t *tokens, uint32_t rows, float *out, uint64_t out_stride) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < rows * table.k; idx += gridDim.x * blockDim.x) {
        const uint32_t r = idx / table.k, at = idx % table.k;
        const uint32_t row = min(tokens[r], table.n - 1);
        out[(uint64_t)r * out_stride + at] = dequant_at(table, row, at);
    }
}

// cursor += 1 between decode steps (Batch::advance, crates/neura-generate/src/batch.rs:1716-1725).
__global__ void advance_kernel(uint32_t *position, uint32_t rows, uint32_t by) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) position[i] += by;
}

// Attention for many rows of ONE sequence (a wide prompt chunk): a CTA takes 16 consecutive rows and one key head, so
// a tile of keys and values is read from the cache once for 16 x group queries instead of once for `group`.  The
// tiles are walked in order with the running largest logit and sum of each query (the same softmax, summed tile by
// tile); row r sees the positions up to its own cursor.  All f32, as the decode attention.
constexpr uint32_t kBlockRows = 16;      // query rows a CTA
constexpr uint32_t kBlockTile = 32;      // positions a tile: one a lane
constexpr uint32_t kBlockThreads = 512;   // 16 warps: an SM holds one CTA, so the warps that hide each other's loads are its own
constexpr uint32_t kAttendBlockFrom = 64;   // fewer rows than this keep the kernel of the decode step (a CTA a row)
constexpr uint32_t kBlockWarps = kBlockThreads / 32;
static_assert(kBlockRows == kBlockWarps, "warp w holds the queries w + 16 j, one a query head of the group");

struct AttendBlockParams {
    const float *q;               // [rows][q_stride], head h at h*width
    uint64_t q_stride;
    const float *keys, *values;   // [key_heads][capacity][width] of the sequence
    const uint32_t *position;     // [rows]
    float *out;                   // [rows][out_stride]
    uint64_t out_stride;
    float scale;
    uint32_t rows, heads, key_heads, capacity;
};

inline size_t attend_block_smem(uint32_t width, uint32_t group) {
    const size_t queries = (size_t)kBlockRows * group;
    return (queries * width + (size_t)kBlockTile * (width + 4) + (size_t)kBlockTile * width + queries * kBlockTile + queries * 3) * sizeof(float);
}

// GROUP (query heads a key head) is a template parameter: with a run-time bound the unrolled loops over a warp's queries were
// predicated, and a group of 5 issued the instructions of 8.
template <uint32_t WIDTH, uint32_t GROUP>
__global__ void __launch_bounds__(kBlockThreads, 1) attend_block_kernel(const __grid_constant__ AttendBlockParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ __align__(16) float shared[];
    constexpr uint32_t KROW = WIDTH + 4;      // padded key row: float4 reads of 8 rows hit 32 banks
    constexpr uint32_t PER = WIDTH / 32;      // output channels a lane
    constexpr uint32_t group = GROUP, queries = kBlockRows * GROUP;
    float *qs = shared;                                   // [queries][WIDTH], query r*group + g
    float *ks = qs + queries * WIDTH;                     // [32][KROW]
    float *vs = ks + kBlockTile * KROW;                   // [32][WIDTH]
    float *weights = vs + kBlockTile * WIDTH;             // [queries][32]: exp(logit - largest so far) of this tile
    float *largest = weights + queries * kBlockTile;      // [queries]
    float *sums = largest + queries;                      // [queries]
    float *shrink = sums + queries;                       // [queries]: exp(largest before - largest after) of this tile
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t blocks = (p.rows + kBlockRows - 1) / kBlockRows;
    // (the longest row blocks first: a block's work grows with its cursors)
    const uint32_t block = blocks - 1 - blockIdx.x / p.key_heads, kh = blockIdx.x % p.key_heads;
    const uint32_t row0 = block * kBlockRows;
    uint32_t most = 0;
    for (uint32_t r = 0; r < kBlockRows; ++r) most = max(most, min(p.position[min(row0 + r, p.rows - 1)] + 1, p.capacity));
    for (uint32_t i = threadIdx.x; i < queries * (WIDTH / 4); i += blockDim.x) {
        const uint32_t query = i / (WIDTH / 4), quad = i % (WIDTH / 4);
        const uint32_t row = min(row0 + query / group, p.rows - 1), g = query % group;   // (a row past the end repeats the last)
        reinterpret_cast<float4 *>(qs)[i] = *reinterpret_cast<const float4 *>(p.q + (uint64_t)row * p.q_stride + (uint64_t)(kh * group + g) * WIDTH + quad * 4);
    }
    for (uint32_t i = threadIdx.x; i < queries; i += blockDim.x) { largest[i] = -INFINITY; sums[i] = 0.0f; }
    float acc[GROUP][PER];
#pragma unroll
    for (uint32_t j = 0; j < GROUP; ++j)
#pragma unroll
        for (uint32_t c = 0; c < PER; ++c) acc[j][c] = 0.0f;
    const float *k = p.keys + (uint64_t)kh * p.capacity * WIDTH, *v = p.values + (uint64_t)kh * p.capacity * WIDTH;
    for (uint32_t t0 = 0; t0 < most; t0 += kBlockTile) {
        __syncthreads();   // the tile before is done with (and, the first time, the queries are in place)
        const uint32_t held = min(kBlockTile, most - t0);
        for (uint32_t i = threadIdx.x; i < kBlockTile * (WIDTH / 4); i += blockDim.x) {
            const uint32_t pos = i / (WIDTH / 4), quad = i % (WIDTH / 4);
            if (pos < held) {
                copy16_async(ks + pos * KROW + quad * 4, k + (uint64_t)(t0 + pos) * WIDTH + quad * 4);
                copy16_async(vs + pos * WIDTH + quad * 4, v + (uint64_t)(t0 + pos) * WIDTH + quad * 4);
            } else {   // past the last cursor of the block: nothing a weight of zero could turn into a NaN
                *reinterpret_cast<float4 *>(ks + pos * KROW + quad * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4 *>(vs + pos * WIDTH + quad * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // logits: a warp takes the queries warp, warp + 16, ... (one a query head of the group); a lane one position of
        // the tile; all the warp's queries share each read of the key row
        {
            const float4 *kr = reinterpret_cast<const float4 *>(ks + lane * KROW);
            float dot[GROUP][2];
#pragma unroll
            for (uint32_t j = 0; j < GROUP; ++j) dot[j][0] = dot[j][1] = 0.0f;
#pragma unroll 4
            for (uint32_t c = 0; c < WIDTH / 4; ++c) {
                const float4 a = kr[c];
#pragma unroll
                for (uint32_t j = 0; j < GROUP; ++j) {
                    const float4 b = reinterpret_cast<const float4 *>(qs + (warp + kBlockWarps * j) * WIDTH)[c];
                    dot[j][0] = fmaf(a.x, b.x, dot[j][0]);
                    dot[j][1] = fmaf(a.y, b.y, dot[j][1]);
                    dot[j][0] = fmaf(a.z, b.z, dot[j][0]);
                    dot[j][1] = fmaf(a.w, b.w, dot[j][1]);
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < GROUP; ++j) {
                const uint32_t query = warp + kBlockWarps * j;
                const uint32_t row = min(row0 + query / group, p.rows - 1);
                const uint32_t count = min(p.position[row] + 1, p.capacity);
                const float logit = t0 + lane < count ? (dot[j][0] + dot[j][1]) * p.scale : -INFINITY;
                float top = logit;
                for (int o = 16; o; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
                const float before = largest[query], after = fmaxf(before, top);
                // (tile 0 holds position 0, which every row sees: `after` is finite from the first tile on)
                const float weight = expf(logit - after);
                float sum = weight;
                for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                weights[query * kBlockTile + lane] = weight;
                if (lane == 0) {
                    const float factor = expf(before - after);
                    shrink[query] = factor;
                    sums[query] = fmaf(sums[query], factor, sum);
                    largest[query] = after;
                }
            }
        }
        __syncthreads();
        // weighted values: a lane holds PER channels of every query of its warp
#pragma unroll
        for (uint32_t j = 0; j < GROUP; ++j) {
            const float factor = shrink[warp + kBlockWarps * j];
#pragma unroll
            for (uint32_t c = 0; c < PER; ++c) acc[j][c] *= factor;
        }
        for (uint32_t pos = 0; pos < kBlockTile; pos += 4) {
            float value[4][PER];
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                if constexpr (PER == 4) {
                    const float4 a = *reinterpret_cast<const float4 *>(vs + (pos + i) * WIDTH + lane * 4);
                    value[i][0] = a.x; value[i][1] = a.y; value[i][2] = a.z; value[i][3] = a.w;
                } else {
                    const float2 a = *reinterpret_cast<const float2 *>(vs + (pos + i) * WIDTH + lane * 2);
                    value[i][0] = a.x; value[i][1] = a.y;
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < GROUP; ++j) {
                const float4 w4 = *reinterpret_cast<const float4 *>(weights + (warp + kBlockWarps * j) * kBlockTile + pos);
#pragma unroll
                for (uint32_t c = 0; c < PER; ++c) {
                    acc[j][c] = fmaf(w4.x, value[0][c], acc[j][c]);
                    acc[j][c] = fmaf(w4.y, value[1][c], acc[j][c]);
                    acc[j][c] = fmaf(w4.z, value[2][c], acc[j][c]);
                    acc[j][c] = fmaf(w4.w, value[3][c], acc[j][c]);
                }
            }
        }
    }
    __syncwarp();   // (a query's sum was last written by lane 0 of the warp that reads it here)
#pragma unroll
    for (uint32_t j = 0; j < GROUP; ++j) {
        const uint32_t query = warp + kBlockWarps * j;
        const uint32_t row = row0 + query / group, g = query % group;
        if (row >= p.rows) continue;
        const float total = sums[query];
        float *to = p.out + (uint64_t)row * p.out_stride + (uint64_t)(kh * group + g) * WIDTH + lane * PER;
#pragma unroll
        for (uint32_t c = 0; c < PER; ++c) to[c] = acc[j][c] / total;
    }
}

// rms_norm alone (crates/neura-decoder/src/op.rs:3-5 -> crates/neura-kernel/src/task/norm.rs:55-131, op = NORM_RMS)
// for any number of rows: one CTA a row, y = x / sqrt(mean(x^2) + floor) * weight as f32.  The rows of a wide prompt
// chunk take it on their way to the tensor-core product, which rounds them to bf16 itself.
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const float *x, uint64_t x_stride, uint32_t k, const float *weight,
                                                           float floor, float *out, uint64_t out_stride) {
    __shared__ float partial[8];
    __shared__ float scale_shared;
    const float *row = x + (uint64_t)blockIdx.x * x_stride;
    float square = 0.0f;
    for (uint32_t c = threadIdx.x; c < k; c += blockDim.x) square = fmaf(row[c], row[c], square);
    for (int o = 16; o; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = square;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (uint32_t w = 0; w < blockDim.x >> 5; ++w) total += partial[w];
        scale_shared = 1.0f / sqrtf(total / (float)k + floor);
    }
    __syncthreads();
    const float scale = scale_shared;
    float *to = out + (uint64_t)blockIdx.x * out_stride;
    for (uint32_t c = threadIdx.x; c < k; c += blockDim.x) {
        float y = row[c] * scale;
        if (weight) y = y * weight[c];
        to[c] = y;
    }
}

// What follows a tensor-core product that left its sums in scratch: `splits` runs of K (each [rows][both_stride], one
// after another at `split_stride`) are added in order, and
//   pair = 0: out[r][c] = chain(sum[r][c]);
//   pair = 1: the product ran over a sealed gate|up pair's 32-row tiles (16 gate rows, then the 16 up rows of the same
//             columns): out[r][c] = chain(silu(gate) * up).
__global__ void gemm_finish_kernel(const float *both, uint64_t both_stride, uint64_t split_stride, uint32_t splits, uint32_t rows,
                                   uint32_t n, uint32_t pair, float *out, uint64_t out_stride, const __grid_constant__ Chain chain) {
    const uint64_t total = (uint64_t)rows * n;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / n;
        const uint32_t c = (uint32_t)(i % n);
        const float *at = both + r * both_stride + (pair ? (uint64_t)(c / 16) * 32 + c % 16 : (uint64_t)c);
        float first = 0.0f, second = 0.0f;
        for (uint32_t z = 0; z < splits; ++z) {
            first += at[z * split_stride];
            if (pair) second += at[z * split_stride + 16];
        }
        out[r * out_stride + c] = chained(chain, r, c, pair ? first * sigmoid_f(first) * second : first);
    }
}

}  // namespace nc
