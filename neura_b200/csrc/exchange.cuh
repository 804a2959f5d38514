// Peer-memory plumbing shared by the one-shot all-reduce (allreduce.cuh) and the exchange a row-parallel product
// does in its own epilogue (prep.cuh, stage_after_piece): system-scope flags, peer stores, and the layout of a
// rank's communication buffer.  No counterpart in the reference, which runs on one device.
//
// A rank's buffer:  [0]           call counter (calls completed)
//                   [4]           chunks of the running call completed (the fused exchange)
//                   [64 + 4 r]    whole-call flag of sender r (allreduce_kernel)
//                   [256 + 32 c + 4 r]  flag of sender r for 256-number chunk c of a call (the fused exchange)
//                   [header ...)  two slots of `world` seats of slot_bytes each: sender r's partial sums
// Sequence numbers only grow; a call uses slot (sequence & 1).
#pragma once
#include "common.cuh"

namespace nc {

constexpr uint32_t kMaxRanks = 8;
constexpr uint32_t kCommFlagsAt = 64, kCommChunkFlagsAt = 256;

__device__ __forceinline__ unsigned long long exchange_nanos() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned int load_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 load_peer16(const float *p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_peer16(float *p, float4 v) {
    asm volatile("st.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// What a kernel needs to take part in an exchange (lives in device memory, written when the communicator connects).
struct ExchangeView {
    unsigned char *mine;                 // this rank's communication buffer
    unsigned char *peer[kMaxRanks];      // every rank's buffer as mapped here (peer[rank] == mine)
    uint64_t slot_bytes;                 // bytes of one sender's seat; a slot is `world` seats
    uint32_t header_bytes;               // where the seats start
    uint32_t world, rank;
    uint32_t chunks_most;                // chunk flags the header holds
};

// The all-reduce of ONE 256-number chunk by ONE warp: lane l owns numbers [8l, 8l + 8) of the chunk, `mine8` on entry
// this rank's partial sums, on return (true) the sums over the ranks, added in rank order.  `at` is the chunk's offset
// in numbers inside the call's vector, `index` its number among the call's `total` chunks.  Every rank's warp pushes its
// eight numbers into its seat at every rank (plain peer stores), publishes the call's sequence number in the chunk's
// flag at every rank, waits (bounded) for all senders' flags in its own memory and adds the seats up.  The warp that
// completes the call's last chunk moves the call counter on.  Returns false when the wait ran out (`wait_nanos`), after
// raising bit 4 of `status`; the call then never completes, and the group has to make a new communicator.
__device__ __forceinline__ bool exchange_chunk(const ExchangeView &e, uint32_t at, uint32_t index, uint32_t total, float (&mine8)[8],
                                               unsigned long long wait_nanos, unsigned int *status) {
    const uint32_t lane = threadIdx.x & 31;
    unsigned int *counter = reinterpret_cast<unsigned int *>(e.mine);
    const unsigned int seq = __ldcg(counter) + 1u;   // (stays put until every chunk of this call is complete, this one included)
    const uint64_t slot = e.header_bytes + (uint64_t)(seq & 1u) * e.world * e.slot_bytes;
    const float4 a = make_float4(mine8[0], mine8[1], mine8[2], mine8[3]), b = make_float4(mine8[4], mine8[5], mine8[6], mine8[7]);
#pragma unroll
    for (uint32_t r = 0; r < kMaxRanks; ++r) {
        if (r < e.world) {
            float *seat = reinterpret_cast<float *>(e.peer[r] + slot + e.rank * e.slot_bytes) + at + lane * 8;
            store_peer16(seat, a);
            store_peer16(seat + 4, b);
        }
    }
    __syncwarp();   // orders every lane's stores before the fences below
    bool gave_up = false;
    if (lane < e.world) {
        __threadfence_system();
        store_release_sys(reinterpret_cast<unsigned int *>(e.peer[lane] + kCommChunkFlagsAt + 32 * index) + e.rank, seq);
        const unsigned int *flag = reinterpret_cast<const unsigned int *>(e.mine + kCommChunkFlagsAt + 32 * index) + lane;
        const unsigned long long start = exchange_nanos();
        // (flags only grow; a peer may already be one call ahead)
        while ((int)(load_acquire_sys(flag) - seq) < 0) {
            if (exchange_nanos() - start > wait_nanos) { gave_up = true; break; }
        }
    }
    if (__ballot_sync(0xffffffffu, gave_up)) {
        if (lane == 0) atomicOr(status, 4u);
        return false;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) mine8[i] = 0.0f;
#pragma unroll
    for (uint32_t r = 0; r < kMaxRanks; ++r) {
        if (r < e.world) {
            const float *seat = reinterpret_cast<const float *>(e.mine + slot + r * e.slot_bytes) + at + lane * 8;
            const float4 c = load_peer16(seat), d = load_peer16(seat + 4);
            mine8[0] += c.x; mine8[1] += c.y; mine8[2] += c.z; mine8[3] += c.w;
            mine8[4] += d.x; mine8[5] += d.y; mine8[6] += d.z; mine8[7] += d.w;
        }
    }
    __syncwarp();
    if (lane == 0) {   // the last chunk of the call to complete moves the call counter on
        unsigned int *done = counter + 1;
        if (atomicAdd(done, 1u) == total - 1u) {
            *done = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned int *>(counter) = seq;
        }
    }
    return true;
}

}  // namespace nc
