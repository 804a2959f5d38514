// The steps either side of the products in a decoder layer: RoPE with the KV-cache write,
// grouped-query attention of one new row over the cache, argmax, and the gather of a
// quantised embedding row.  (rms_norm lives in prep.cuh, fused with the activation staging.)
#pragma once
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
};

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
            const float angle = (float)position * powf(p.base, -2.0f * (float)channel / (float)p.width);
            const float cosine = cosf(angle), sine = sinf(angle);
            const float low = v[channel], high = v[channel + half];
            const float new_low = low * cosine - high * sine;
            const float new_high = high * cosine + low * sine;
            v[channel] = new_low;
            v[channel + half] = new_high;
            if (head >= p.heads && position < p.capacity) {
                const uint32_t kh = head - p.heads;
                float *slot = p.keys + (((uint64_t)b * p.key_heads + kh) * p.capacity + position) * p.width;
                slot[channel] = new_low;
                slot[channel + half] = new_high;
            }
        } else if (position < p.capacity) {
            const uint32_t c = at - turned, kh = c / p.width, d = c % p.width;
            const float value = row[(uint64_t)(p.heads + p.key_heads) * p.width + c];
            p.values[(((uint64_t)b * p.key_heads + kh) * p.capacity + position) * p.width + d] = value;
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
constexpr uint32_t kAttendMaxChunk = 128;  // positions one CTA takes

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
};

__global__ void __launch_bounds__(128) attend_kernel(const __grid_constant__ AttendParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ float shared[];
    const uint32_t group = p.heads / p.key_heads;
    float *qs = shared;                                  // [group][width]
    float *logits = qs + group * p.width;                // [group][kAttendMaxChunk]
    float *stats = logits + group * kAttendMaxChunk;     // [group][2]: largest, sum
    __shared__ unsigned int arrived;
    const uint32_t split = blockIdx.x % p.splits;
    const uint32_t kh = (blockIdx.x / p.splits) % p.key_heads;
    const uint32_t b = blockIdx.x / (p.splits * p.key_heads);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const uint32_t count = min(p.position[b] + 1, p.capacity);
    const uint32_t chunk = min((count + p.splits - 1) / p.splits, kAttendMaxChunk);
    // (the host sizes `splits` so that capacity / splits <= kAttendMaxChunk)
    const uint32_t first = min(split * chunk, count), last = min(first + chunk, count);
    const float *k = p.keys + ((uint64_t)b * p.key_heads + kh) * p.capacity * p.width;
    const float *v = p.values + ((uint64_t)b * p.key_heads + kh) * p.capacity * p.width;
    for (uint32_t i = threadIdx.x; i < group * p.width; i += blockDim.x)
        qs[i] = p.q[(uint64_t)b * p.q_stride + (uint64_t)(kh * group) * p.width + i];
    __syncthreads();
    // logits of this split: one warp per position, lanes across the head width
    for (uint32_t pos = first + warp; pos < last; pos += warps) {
        float acc[kAttendMaxGroup];
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g) acc[g] = 0.0f;
        for (uint32_t d = lane; d < p.width; d += 32) {
            const float kv = k[(uint64_t)pos * p.width + d];
#pragma unroll
            for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                if (g < group) acc[g] = fmaf(qs[g * p.width + d], kv, acc[g]);
        }
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g) {
            if (g < group) {
                float total = acc[g];
                for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                if (lane == 0) logits[g * kAttendMaxChunk + (pos - first)] = total * p.scale;
            }
        }
    }
    __syncthreads();
    // per query head: largest logit and sum of exponentials of the split (one warp per head)
    for (uint32_t g = warp; g < group; g += warps) {
        float largest = -INFINITY;
        for (uint32_t i = lane; i < last - first; i += 32) largest = fmaxf(largest, logits[g * kAttendMaxChunk + i]);
        for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
        float sum = 0.0f;
        for (uint32_t i = lane; i < last - first; i += 32) {
            const float e = expf(logits[g * kAttendMaxChunk + i] - largest);
            logits[g * kAttendMaxChunk + i] = e;
            sum += e;
        }
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) { stats[g * 2] = largest; stats[g * 2 + 1] = sum; }
    }
    __syncthreads();
    // weighted values: one thread per channel, every value row read once for all the group's heads
    for (uint32_t d = threadIdx.x; d < p.width; d += blockDim.x) {
        float acc[kAttendMaxGroup];
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g) acc[g] = 0.0f;
        for (uint32_t pos = first; pos < last; ++pos) {
            const float value = v[(uint64_t)pos * p.width + d];
#pragma unroll
            for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
                if (g < group) acc[g] = fmaf(logits[g * kAttendMaxChunk + (pos - first)], value, acc[g]);
        }
#pragma unroll
        for (uint32_t g = 0; g < kAttendMaxGroup; ++g)
            if (g < group)
                __stcg(p.partial + (((uint64_t)b * p.heads + kh * group + g) * p.splits + split) * (p.width + 2) + d, acc[g]);
    }
    if (threadIdx.x < group * 2) {
        const uint32_t g = threadIdx.x / 2, which = threadIdx.x % 2;
        __stcg(p.partial + (((uint64_t)b * p.heads + kh * group + g) * p.splits + split) * (p.width + 2) + p.width + which,
               stats[g * 2 + which]);
    }
    // the last split of this (sequence, key head) to arrive merges them all, in split order
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        arrived = atomicAdd(p.counters + b * p.key_heads + kh, 1u);
        __threadfence();
    }
    __syncthreads();
    if (arrived != p.splits - 1) return;
    for (uint32_t g = 0; g < group; ++g) {
        const float *mine = p.partial + ((uint64_t)b * p.heads + kh * group + g) * p.splits * (p.width + 2);
        float largest = -INFINITY;
        for (uint32_t s = 0; s < p.splits; ++s) largest = fmaxf(largest, __ldcg(mine + s * (p.width + 2) + p.width));
        float total = 0.0f;
        for (uint32_t s = 0; s < p.splits; ++s) {
            const float m = __ldcg(mine + s * (p.width + 2) + p.width);
            const float factor = m == -INFINITY ? 0.0f : expf(m - largest);
            total = fmaf(__ldcg(mine + s * (p.width + 2) + p.width + 1), factor, total);
        }
        for (uint32_t d = threadIdx.x; d < p.width; d += blockDim.x) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < p.splits; ++s) {
                const float m = __ldcg(mine + s * (p.width + 2) + p.width);
                const float factor = m == -INFINITY ? 0.0f : expf(m - largest);
                acc = fmaf(__ldcg(mine + s * (p.width + 2) + d), factor, acc);
            }
            p.out[(uint64_t)b * p.out_stride + (uint64_t)(kh * group + g) * p.width + d] = acc / total;
        }
    }
    if (threadIdx.x == 0) p.counters[b * p.key_heads + kh] = 0u;
}

// argmax, the lowest index winning a tie (choice_precedes, crates/neura-kernel/src/task/choice.rs:46-52).
// One CTA per row.
__global__ void __launch_bounds__(1024) argmax_kernel(const float *x, uint64_t stride, uint32_t width, uint32_t *out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float best_value[32];
    __shared__ uint32_t best_index[32];
    const float *row = x + (uint64_t)blockIdx.x * stride;
    float value = -INFINITY;
    uint32_t index = 0xffffffffu;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        const float other = row[c];
        if (other > value || (other == value && c < index)) { value = other; index = c; }
    }
    for (int o = 16; o; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, o);
        const uint32_t other_index = __shfl_xor_sync(0xffffffffu, index, o);
        if (other > value || (other == value && other_index < index)) { value = other; index = other_index; }
    }
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        value = lane < (blockDim.x >> 5) ? best_value[lane] : -INFINITY;
        index = lane < (blockDim.x >> 5) ? best_index[lane] : 0xffffffffu;
        for (int o = 16; o; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, value, o);
            const uint32_t other_index = __shfl_xor_sync(0xffffffffu, index, o);
            if (other > value || (other == value && other_index < index)) { value = other; index = other_index; }
        }
        if (lane == 0) out[blockIdx.x] = index == 0xffffffffu ? 0u : index;
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

}  // namespace nc
