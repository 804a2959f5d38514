// One-shot all-reduce over NVLink peer memory for the row-parallel projections of a tensor-parallel
// decode step (no counterpart in the reference, which runs on one device).
//
// Every rank owns a communication buffer that its peers map (CUDA IPC): a call counter, one flag
// per sender and two slots of one partial per sender.  A call pushes the rank's partial sums into
// its seat of every rank's slot (posted stores over NVLink; nothing is read remotely), then
// publishes the call's sequence number in its flag at every rank (release, system scope), waits
// until all senders' flags in its own memory show that number (local acquire loads, bounded by a
// timer) and adds the seats in rank order, so every rank computes bit-identical sums.  Two slots
// suffice: a rank can only reach call s+2 after every peer has published s+1, i.e. has finished
// reading call s.  A wait that runs out (the context's wait limit) raises the status word and leaves
// the input untouched; the call counter stays, so the next call repeats the sequence number and
// completes once the missing peer has published it.
#pragma once
#include "common.cuh"
#include "exchange.cuh"
#include "gemv_mma.cuh"
#include "prep.cuh"

namespace nc {

struct AllreduceParams {
    unsigned char *mine;                 // this rank's communication buffer
    unsigned char *peer[kMaxRanks];      // every rank's buffer as mapped here (peer[rank] == mine)
    float *inout;                        // [count]
    uint64_t slot_bytes;                 // bytes of one sender's seat; a slot is world seats
    uint32_t header_bytes;               // where the seats start in a buffer
    uint32_t count, world, rank;
    unsigned int *status;
    unsigned long long wait_nanos;       // how long a rank waits for its peers' flags before it gives up
};

// One CTA; count is a multiple of 4.  Returns false when the wait for the peers ran out.
__device__ __forceinline__ bool allreduce_body(const AllreduceParams &p) {
    __shared__ unsigned int gave_up;
    unsigned int *counter = reinterpret_cast<unsigned int *>(p.mine);
    const unsigned int seq = *counter + 1u;
    const uint64_t slot = (uint64_t)(seq & 1u) * p.world * p.slot_bytes;
    if (threadIdx.x == 0) gave_up = 0u;
    // push this rank's partial into its seat at every rank
    for (uint32_t i = threadIdx.x * 4; i < p.count; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4 *>(p.inout + i);
#pragma unroll
        for (uint32_t r = 0; r < kMaxRanks; ++r)
            if (r < p.world)
                store_peer16(reinterpret_cast<float *>(p.peer[r] + p.header_bytes + slot + p.rank * p.slot_bytes) + i, v);
    }
    __syncthreads();   // orders every thread's stores before the fences below
    if (threadIdx.x < p.world) {
        __threadfence_system();
        store_release_sys(reinterpret_cast<unsigned int *>(p.peer[threadIdx.x] + kCommFlagsAt) + p.rank, seq);
        const unsigned int *flag = reinterpret_cast<const unsigned int *>(p.mine + kCommFlagsAt) + threadIdx.x;
        const unsigned long long start = global_nanos();
        // (flags only grow; a peer may already be one call ahead)
        while ((int)(load_acquire_sys(flag) - seq) < 0) {
            if (global_nanos() - start > p.wait_nanos) { gave_up = 1u; break; }
        }
    }
    __syncthreads();
    if (gave_up) {
        if (threadIdx.x == 0) atomicOr(p.status, 4u);
        return false;   // the counter stays: the next call repeats this sequence number
    }
    for (uint32_t i = threadIdx.x * 4; i < p.count; i += blockDim.x * 4) {
        float4 part[kMaxRanks];
#pragma unroll
        for (uint32_t r = 0; r < kMaxRanks; ++r)
            if (r < p.world)
                part[r] = load_peer16(reinterpret_cast<const float *>(p.mine + p.header_bytes + slot + r * p.slot_bytes) + i);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (uint32_t r = 0; r < kMaxRanks; ++r) {
            if (r < p.world) {
                sum.x += part[r].x; sum.y += part[r].y; sum.z += part[r].z; sum.w += part[r].w;
            }
        }
        *reinterpret_cast<float4 *>(p.inout + i) = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) *counter = seq;
    return true;
}

__global__ void __launch_bounds__(1024) allreduce_kernel(const __grid_constant__ AllreduceParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    allreduce_body(p);
}

// The all-reduce of a row-parallel projection's partial sums followed, in the same launch, by the rms_norm of the
// summed rows and their staging for the next product (prep.cuh): the CTA that added the rows up has them at hand.
__global__ void __launch_bounds__(1024) allreduce_norm_stage_kernel(const __grid_constant__ AllreduceParams p,
                                                                     const __grid_constant__ NormStageParams then) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float partial[32];
    __shared__ float scale_shared;
    if (!allreduce_body(p)) return;
    __syncthreads();
    for (uint32_t row = 0; row < then.prep.rows; ++row) {
        rms_norm_stage_row(then, row, partial, &scale_shared);
        __syncthreads();
    }
}

}  // namespace nc
