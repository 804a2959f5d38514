// libneura_cuda: the extern "C" surface declared in include/neura_cuda.h.
// Built for sm_100a only; there is no CPU path behind any entry point.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <new>
#include <string>
#include <vector>

#include "allreduce.cuh"
#include "common.cuh"
#include "decoder_ops.cuh"
#include "gemm_tcgen05.cuh"
#include "gemv_mma.cuh"
#include "layout.cuh"
#include "megakernel.cuh"
#include "prep.cuh"
#include "quantize.cuh"
#include "skinny_tcgen05.cuh"

using namespace nc;

#ifndef NC_GEMV_STAGES
#define NC_GEMV_STAGES 2
#endif

namespace {

thread_local std::string g_error;

int32_t refuse(int32_t code, const char *fmt, ...) {
    char text[512];
    va_list args;
    va_start(args, fmt);
    vsnprintf(text, sizeof text, fmt, args);
    va_end(args);
    g_error = text;
    return code;
}

int32_t cuda_refuse(cudaError_t e, const char *what) {
    char text[512];
    snprintf(text, sizeof text, "%s: %s", what, cudaGetErrorString(e));
    g_error = text;
    return (int32_t)e;
}

#define NC_CUDA(call)                                         \
    do {                                                      \
        cudaError_t e_ = (call);                              \
        if (e_ != cudaSuccess) return cuda_refuse(e_, #call); \
    } while (0)

constexpr int32_t kBadArgument = -1;
constexpr int32_t kBadState = -2;
constexpr int32_t kDeviceRefusal = -3;
constexpr uint32_t kMaxRowsPerPass = 16;  // activation rows one staging of digit planes holds
constexpr uint32_t kRowsPerLaunch = 8;    // activation rows one launch of the streaming product carries (three 8-column MMA tiles)
// From this many rows on a Q4_K product takes the tensor-core skinny kernel (skinny_tcgen05.cuh), which streams the
// weight once for up to kSkMaxRows rows: the reference's choice between folded and staged-run tiles by row count
// (Product::planned, crates/neura-plan/src/product.rs:103-195: folded up to 4 rows of a K-quant, staged runs above).
#ifndef NC_SKINNY_FROM
#define NC_SKINNY_FROM 9
#endif
constexpr uint32_t kSkinnyFrom = NC_SKINNY_FROM;

struct Region {
    void *ptr = nullptr;
    uint64_t bytes = 0;
};

}  // namespace

// One staged form of some activation rows (prep.cuh): what the products read.  A context holds kStagingSlots
// of them, so that a product can read one while its epilogue stages its own output into another.
struct Staging {
    Region dig, cs, sums, chunks;   // chunks: finished pieces of every 256-column chunk (StageAfter::counters)
    uint32_t rows = 0, k = 0, granule = 0;   // what was last staged here
    uint32_t halves = 0;            // 1: the rows were staged as half floats for the skinny product (the context's
                                    //    one set of skinny buffers), not as digit planes
};
constexpr uint32_t kStagingSlots = 3;

struct nc_context {
    int device = 0;
    int sms = 0;
    Staging slots[kStagingSlots];
    uint32_t cur = 0;            // the slot neura_cuda_stage writes and the products read (neura_cuda_staging_select)
    Region squares;              // [rows][chunks] sums of squares left by an epilogue that staged with a norm's gain
    Region partial, counters, status, stage_x, stage_out, attend_partial, attend_counters, argmax_scratch, x_bf16, pair_out;
    Region sk_xh, sk_sx, sk_xs, sk_rs, sk_partial, sk_counters;   // the skinny product's staged activations and split-K scratch
    uint32_t sk_bpad = 0, sk_sx_cols = 0;
    uint64_t launches = 0;
    unsigned long long wait_nanos = 2000000000ull;   // how long a kernel waits for another party (neura_cuda_set_wait_limit)
    bool capturing = false;
    cudaStream_t capture_stream = nullptr;
    uint64_t capture_mark = 0;
};

struct nc_comm {
    int device = 0;
    unsigned char *mine = nullptr;
    unsigned char *peer[kMaxRanks] = {nullptr};
    uint64_t slot_bytes = 0, max_count = 0;
    uint32_t header_bytes = 0, chunks_most = 0;
    ExchangeView *view_dev = nullptr;   // what a product that exchanges in its own epilogue reads (filled on connect)
    uint32_t world = 0, rank = 0;
    bool connected = false;
    bool local = false;   // the peers are communicators of this process (plain pointers, nothing to unmap)
};

struct nc_program {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;  // kernels one run replays
};

namespace {

// Grows a scratch region (never shrinks).  Growing frees the old block, which
// waits for the device: callers that cannot afford that call neura_cuda_reserve first.
int32_t ensure(nc_context *ctx, Region &region, uint64_t bytes, bool zero) {
    if (region.bytes >= bytes) return 0;
    if (ctx->capturing)
        return refuse(kBadState, "a recorded program may not grow the scratch: call neura_cuda_reserve for its largest product first");
    if (region.ptr) NC_CUDA(cudaFree(region.ptr));
    region.ptr = nullptr;
    region.bytes = 0;
    const uint64_t want = (bytes + 255) / 256 * 256;
    NC_CUDA(cudaMalloc(&region.ptr, want));
    if (zero) NC_CUDA(cudaMemset(region.ptr, 0, want));
    region.bytes = want;
    return 0;
}

// The formats that are multiplied where the GGUF left them (qlinear_rows.cuh); the streaming kernels take Q8_0 and Q4K.
bool gguf_only(uint32_t element) {
    return element == NC_ELEMENT_Q6K || element == NC_ELEMENT_Q5K || element == NC_ELEMENT_Q3K || element == NC_ELEMENT_HALF ||
           element == NC_ELEMENT_BFLOAT16;
}
uint32_t block_elements(uint32_t element) {
    switch (element) {
    case NC_ELEMENT_Q8_0: return kQ8Block;
    case NC_ELEMENT_Q4K: case NC_ELEMENT_Q5K: case NC_ELEMENT_Q6K: case NC_ELEMENT_Q3K: return kSuperBlock;
    case NC_ELEMENT_HALF: case NC_ELEMENT_BFLOAT16: return 1;
    default: return 0;
    }
}
uint32_t block_bytes(uint32_t element) {
    switch (element) {
    case NC_ELEMENT_Q8_0: return kQ8Bytes;
    case NC_ELEMENT_Q4K: return kQ4kBytes;
    case NC_ELEMENT_Q5K: return kQ5kBytes;
    case NC_ELEMENT_Q6K: return kQ6kBytes;
    case NC_ELEMENT_Q3K: return kQ3kBytes;
    case NC_ELEMENT_HALF: case NC_ELEMENT_BFLOAT16: return 2;
    default: return 0;
    }
}

struct GemvPlan {
    uint32_t ntiles, upt, nwarps, q, r, maxp, blocks;
};

// The (q, r) split of gemv_mma.cuh for a grid that fills the GPU once.
GemvPlan plan_gemv(const nc_context *ctx, uint32_t element, uint32_t n, uint32_t k, int resident_blocks_per_sm) {
    GemvPlan plan;
    plan.ntiles = (n + kTileRows - 1) / kTileRows;
    plan.upt = k / block_elements(element);
    const uint64_t units = (uint64_t)plan.ntiles * plan.upt;  // below 2^32: n and k are 32-bit, units = n*k/8192 at most
    // 32-row units a warp should at least stream: one Q4_K unit (the small projections want every warp), one
    // stage of four Q8_0 units
    const uint64_t least = element == NC_ELEMENT_Q4K ? 1 : 4;
    uint64_t warps = (uint64_t)ctx->sms * resident_blocks_per_sm * kGemvWarps;
    if (warps > units / least) warps = units / least;
    if (warps < 1) warps = 1;
    plan.nwarps = (uint32_t)warps;
    plan.q = (uint32_t)(units / warps);
    plan.r = (uint32_t)(units % warps);
    plan.maxp = (plan.upt + plan.q - 1) / plan.q + 1;
    plan.blocks = (plan.nwarps + kGemvWarps - 1) / kGemvWarps;
    return plan;
}

constexpr int kStages = NC_GEMV_STAGES;   // ring depth of the streaming product (stages a warp)

// Launches with the programmatic-stream-serialization attribute, so that a kernel's
// prologue (for the product: its first weight copies) overlaps the tail of the kernel
// before it; the kernels order themselves with griddepcontrol.wait.
template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args &&...args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <bool Q4K, int NT, bool HOOKS = false>
int32_t launch_gemv_as(nc_context *ctx, cudaStream_t stream, uint32_t element, GemvParams &p, uint32_t n, uint32_t k) {
    auto kernel = qlinear_stream_kernel<Q4K, NT, kStages, HOOKS>;
    constexpr size_t stage = Q4K ? kQ4kStage : kQ8Stage;
    constexpr size_t smem = kGemvWarps * kStages * (stage + 8) + kGemvWarps * 32 * (NT * 8 + 1) * sizeof(float);
    static int resident[16] = {0};  // per device, filled on first use
    if (resident[ctx->device & 15] == 0) {
        NC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int blocks = 0;
        NC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kGemvWarps * 32, smem));
        if (blocks < 1) return refuse(kBadState, "the product kernel does not fit an SM");
        resident[ctx->device & 15] = blocks;
    }
    const GemvPlan plan = plan_gemv(ctx, element, n, k, resident[ctx->device & 15]);
    const uint64_t cells = (uint64_t)p.rows * kTileRows;
    int32_t rc;
    if ((rc = ensure(ctx, ctx->partial, (uint64_t)plan.ntiles * plan.maxp * cells * sizeof(float), false))) return rc;
    if ((rc = ensure(ctx, ctx->counters, (uint64_t)plan.ntiles * sizeof(unsigned int), true))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    p.partial = (float *)ctx->partial.ptr;
    p.counters = (unsigned int *)ctx->counters.ptr;
    p.status = (unsigned int *)ctx->status.ptr;
    p.upt = plan.upt;
    p.nwarps = plan.nwarps;
    p.q = plan.q;
    p.r = plan.r;
    p.maxp = plan.maxp;
    NC_CUDA(launch_dependent(kernel, dim3(plan.blocks), dim3(kGemvWarps * 32), smem, stream, p));
    ctx->launches++;
    return 0;
}

template <int NT>
int32_t launch_gemv(nc_context *ctx, cudaStream_t stream, uint32_t element, GemvParams &p, uint32_t n, uint32_t k) {
    return element == NC_ELEMENT_Q4K ? launch_gemv_as<true, NT>(ctx, stream, element, p, n, k)
                                     : launch_gemv_as<false, NT>(ctx, stream, element, p, n, k);
}

// The product of at most two rows that also applies its input's rms_norm scalar and stages its own output.
int32_t launch_gemv_hooked(nc_context *ctx, cudaStream_t stream, uint32_t element, GemvParams &p, uint32_t n, uint32_t k) {
    return element == NC_ELEMENT_Q4K ? launch_gemv_as<true, 1, true>(ctx, stream, element, p, n, k)
                                     : launch_gemv_as<false, 1, true>(ctx, stream, element, p, n, k);
}

int32_t check_weight(const nc_weight *w) {
    if (!w || !w->data_dev) return refuse(kBadArgument, "a product needs a weight on the device");
    const uint32_t per = block_elements(w->element);
    if (!per)
        return refuse(kBadArgument, "element %u is not a format this path multiplies (Q8_0 = 8, Q4K = 9; in GGUF order Q5K = 10, Q6K = 11, Q3K = 12, half = 1, bfloat16 = 2)",
                      w->element);
    if (w->n == 0 || w->k == 0 || w->k % per)
        return refuse(kBadArgument, "a [%u, %u] weight does not fill whole blocks of %u along its rows", w->n,
                      w->k, per);
    if (gguf_only(w->element)) {
        if (w->layout != NC_LAYOUT_GGUF) return refuse(kBadArgument, "a weight of element %u is multiplied in GGUF order; it has no sealed layout", w->element);
        return 0;
    }
    if ((uintptr_t)w->data_dev % 16)
        return refuse(kBadArgument, "a weight starts on a 16-byte boundary");
    return 0;
}

template <uint32_t ELEMENT>
void (*rows_kernel_of(uint32_t rows))(RowsParams, uint64_t) {
    return rows <= 1 ? qlinear_rows_kernel<ELEMENT, 1> : rows <= 2 ? qlinear_rows_kernel<ELEMENT, 2>
           : rows <= 4 ? qlinear_rows_kernel<ELEMENT, 4> : qlinear_rows_kernel<ELEMENT, 8>;
}

// The product of a weight kept in GGUF order (qlinear_rows.cuh): passes of up to eight rows.
int32_t rows_product(nc_context *ctx, cudaStream_t stream, const nc_weight *w, const float *x_dev, uint32_t rows, uint64_t x_stride,
                     float *out_dev, uint64_t out_stride, const nc_step *chain, uint32_t n_steps) {
    for (uint32_t first = 0; first < rows; first += kRowsKernelMost) {
        RowsParams p;
        memset(&p, 0, sizeof p);
        p.w = (const uint8_t *)w->data_dev;
        p.x = x_dev + (uint64_t)first * x_stride;
        p.out = out_dev + (uint64_t)first * out_stride;
        p.x_stride = x_stride;
        p.out_stride = out_stride;
        p.n = w->n;
        p.k = w->k;
        p.rows = std::min(kRowsKernelMost, rows - first);
        p.chain.n = n_steps;
        for (uint32_t s = 0; s < n_steps; ++s) {
            p.chain.step[s] = chain[s];
            if (chain[s].operand_dev) p.chain.step[s].operand_dev = chain[s].operand_dev + (int64_t)first * chain[s].row_stride;
        }
        const uint64_t want = ((uint64_t)w->n + 7) / 8;   // eight warps a CTA, a warp a weight row
        const unsigned int blocks = (unsigned int)std::min<uint64_t>(want, (uint64_t)ctx->sms * 8);
        if (w->element == NC_ELEMENT_Q6K) {
            void (*kernel)(RowsParams) = p.rows <= 1 ? qlinear_rows_q6k_kernel<1> : p.rows <= 2 ? qlinear_rows_q6k_kernel<2>
                                         : p.rows <= 4 ? qlinear_rows_q6k_kernel<4> : qlinear_rows_q6k_kernel<8>;
            NC_CUDA(launch_dependent(kernel, dim3(blocks), dim3(256), 0, stream, p));
        } else {
            void (*kernel)(RowsParams, uint64_t) = w->element == NC_ELEMENT_Q5K ? rows_kernel_of<NC_ELEMENT_Q5K>(p.rows)
                                                   : w->element == NC_ELEMENT_Q3K ? rows_kernel_of<NC_ELEMENT_Q3K>(p.rows)
                                                   : w->element == NC_ELEMENT_HALF ? rows_kernel_of<NC_ELEMENT_HALF>(p.rows)
                                                                                   : rows_kernel_of<NC_ELEMENT_BFLOAT16>(p.rows);
            const uint64_t row_bytes = (uint64_t)w->k / block_elements(w->element) * block_bytes(w->element);
            NC_CUDA(launch_dependent(kernel, dim3(blocks), dim3(256), 0, stream, p, row_bytes));
        }
        ctx->launches++;
    }
    return 0;
}

// The device status word (the reference's refusal word, crates/neura-kernel/src/substrate.rs:93-100):
// read after a synchronisation, non-zero when a kernel gave up on a bounded wait.
// ---------------------------------------------------------------------------------------
// Scratch of the product for callers that must not allocate (neura_cuda_linear_static).
//
// Everything neura_cuda_linear keeps in scratch that it may have to cudaMalloc (digit
// planes, digit scales, split-tile partial sums, tile counters, the status word) lives
// here in one fixed array inside the library image.  Every GPU whose context loads the
// library carries these 16 MiB until the process exits.
// ---------------------------------------------------------------------------------------
constexpr uint64_t kStaticScratchBytes = 16ull << 20;
constexpr uint32_t kStaticMaxRows = 4;
constexpr uint32_t kStaticMaxK = 32768;
constexpr uint32_t kStaticMaxN = 262144;
constexpr uint64_t kStaticCountersBytes = (uint64_t)(kStaticMaxN / kTileRows) * sizeof(unsigned int);
constexpr int kStaticDevices = 64;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// `g_static_scratch` names a host-side shadow in host code, not device memory: the device
// address has to be asked for, once per device, with that device current.
struct StaticScratch {
    unsigned char *base = nullptr;   // the array's address on this device, null until the first call
    int resident[4] = {0, 0, 0, 0};  // CTAs of each kernel variant an SM holds
};
StaticScratch g_static[kStaticDevices];

// The four kernels the allocation-free product may launch: Q8_0 / Q4_K, one or two 8-column MMA tiles.
void (*static_variant(int variant))(GemvParams) {
    switch (variant) {
    case 0: return qlinear_stream_kernel<false, 1, NC_GEMV_STAGES>;
    case 1: return qlinear_stream_kernel<false, 2, NC_GEMV_STAGES>;
    case 2: return qlinear_stream_kernel<true, 1, NC_GEMV_STAGES>;
    default: return qlinear_stream_kernel<true, 2, NC_GEMV_STAGES>;
    }
}
size_t static_variant_smem(int variant) {
    const size_t stage = variant >= 2 ? kQ4kStage : kQ8Stage;
    const int nt = (variant & 1) + 1;
    return kGemvWarps * NC_GEMV_STAGES * (stage + 8) + kGemvWarps * 32 * (nt * 8 + 1) * sizeof(float);
}

// The first call on a device: looks the array's device address up and makes the runtime load every kernel the
// entry point may launch (loading a kernel's code on first use may allocate), so that later calls only launch.
int32_t static_setup(int device) {
    StaticScratch &fixed = g_static[device];
    if (fixed.base) return 0;
    NC_CUDA(cudaSetDevice(device));
    unsigned char *address = nullptr;
    NC_CUDA(cudaGetSymbolAddress((void **)&address, g_static_scratch));
    if (!address) return refuse(kBadState, "the static scratch has no address on device %d", device);
    for (int variant = 0; variant < 4; ++variant) {
        NC_CUDA(cudaFuncSetAttribute(static_variant(variant), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)static_variant_smem(variant)));
        NC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fixed.resident[variant], static_variant(variant),
                                                              kGemvWarps * 32, static_variant_smem(variant)));
        if (fixed.resident[variant] < 1) return refuse(kBadState, "the product kernel does not fit an SM");
    }
    cudaFuncAttributes attributes;
    NC_CUDA(cudaFuncGetAttributes(&attributes, prep_kernel));
    fixed.base = address;
    return 0;
}

unsigned int *static_status_of(int device) {
    return device >= 0 && device < kStaticDevices ? (unsigned int *)g_static[device].base : nullptr;
}

// After a reported failure: the status word and the tile counters start from zero again.
int32_t static_scratch_clear(int device) {
    NC_CUDA(cudaMemset(g_static[device].base, 0, 256 + kStaticCountersBytes));
    return 0;
}

const char *status_sentence(unsigned int word) {
    if (word & 4u) return "an all-reduce gave up waiting for a peer's partial sums";
    if (word & 2u) return "a kernel gave up waiting at a barrier";
    return "a kernel gave up waiting for its own copies";
}

int32_t check_status(nc_context *ctx) {
    unsigned int word = 0, fixed = 0;
    if (ctx->status.ptr) NC_CUDA(cudaMemcpy(&word, ctx->status.ptr, sizeof word, cudaMemcpyDeviceToHost));
    unsigned int *fixed_dev = static_status_of(ctx->device);
    if (fixed_dev) NC_CUDA(cudaMemcpy(&fixed, fixed_dev, sizeof fixed, cudaMemcpyDeviceToHost));
    if (word == 0 && fixed == 0) return 0;
    if (word) NC_CUDA(cudaMemset(ctx->status.ptr, 0, sizeof word));
    if (fixed) {   // a product that gave up may have left tile counters behind: the array starts over
        int32_t rc = static_scratch_clear(ctx->device);
        if (rc) return rc;
    }
    return refuse(kDeviceRefusal, "%s (status %u); its output is not valid", status_sentence(word | fixed), word | fixed);
}


// cuTensorMapEncodeTiled, looked up through the runtime so that the library links the runtime only.
typedef CUresult (*tensor_map_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                         const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int32_t tensor_map_encoder(tensor_map_encode_fn *out) {
    static tensor_map_encode_fn encode = nullptr;
    if (!encode) {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult found;
        NC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found));
        if (!entry || found != cudaDriverEntryPointSuccess) return refuse(kBadState, "the driver does not offer cuTensorMapEncodeTiled");
        encode = (tensor_map_encode_fn)entry;
    }
    *out = encode;
    return 0;
}

// A 16-bit [rows][cols] tensor read in boxes of 64 columns x `box_rows` rows, 128-byte swizzled.
int32_t tensor_map_16bit(CUtensorMap *map, CUtensorMapDataType type, void *base, uint64_t cols, uint64_t rows, uint32_t box_rows) {
    tensor_map_encode_fn encode;
    int32_t rc;
    if ((rc = tensor_map_encoder(&encode))) return rc;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, box_rows}, steps[2] = {1, 1};
    const CUresult made = encode(map, type, 2, base, dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (made != CUDA_SUCCESS) return refuse(kBadState, "cuTensorMapEncodeTiled refused the activations (%d)", (int)made);
    return 0;
}

// An f32 [rows][cols] output written in boxes of 32 x 32, 128-byte swizzled in shared memory (rows `stride` numbers apart).
int32_t tensor_map_f32_out(CUtensorMap *map, void *base, uint64_t cols, uint64_t rows, uint64_t stride) {
    tensor_map_encode_fn encode;
    int32_t rc;
    if ((rc = tensor_map_encoder(&encode))) return rc;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride * 4};
    const cuuint32_t box[2] = {32, 32}, steps[2] = {1, 1};
    const CUresult made = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (made != CUDA_SUCCESS) return refuse(kBadState, "cuTensorMapEncodeTiled refused the output (%d)", (int)made);
    return 0;
}

// ---- the skinny product (skinny_tcgen05.cuh) ---------------------------------------------------------------
// How many rows one pass of a product carries: up to 16 as digit planes (8 a launch), or, for a Q4_K weight from
// kSkinnyFrom rows on, up to kSkMaxRows through the skinny kernel, the rows dealt evenly over the passes.
uint32_t rows_per_pass(uint32_t element, uint32_t rows) {
    if (element == NC_ELEMENT_Q4K && rows >= kSkinnyFrom) {
        const uint32_t passes = (rows + kSkMaxRows - 1) / kSkMaxRows;
        return (rows + passes - 1) / passes;
    }
    return rows < kMaxRowsPerPass ? rows : kMaxRowsPerPass;
}

struct SkinnyPlan {
    uint32_t tiles32, ntile128, splits, grid;
};

// Items are (128-row tile, K slice); a CTA per SM walks them.  The K axis is split when that fills the SMs better:
// the cost of a split is the rounds of items times the super-blocks of an item, a little more for the partial sums.
SkinnyPlan skinny_plan(const nc_context *ctx, uint32_t n, uint32_t k, bool pair, uint32_t bpad) {
    SkinnyPlan plan;
    plan.tiles32 = pair ? (n + 15) / 16 : (n + kTileRows - 1) / kTileRows;
    plan.ntile128 = (plan.tiles32 + 3) / 4;
    const uint32_t nsb = k / kSuperBlock, sms = (uint32_t)ctx->sms;
    double best = 0.0;
    plan.splits = 1;
    for (uint32_t s = 1; s <= nsb && s <= 16; ++s) {
        if (s > 1 && (uint64_t)plan.ntile128 * s * bpad * kSkTileRows * sizeof(float) > (16ull << 20)) break;
        const uint64_t rounds = ((uint64_t)plan.ntile128 * s + sms - 1) / sms;
        // (an item costs about four super-blocks' time on top of its own: the second sum's stages, the accumulator's
        // last read, the partial sums)
        const double cost = (double)rounds * (double)((nsb + s - 1) / s + (s > 1 ? 1 : 0) + 4) * (1.0 + 0.02 * (s - 1));
        if (s == 1 || cost < best) {
            best = cost;
            plan.splits = s;
        }
    }
    const uint64_t items = (uint64_t)plan.ntile128 * plan.splits;
    plan.grid = (uint32_t)(items < sms ? items : sms);
    return plan;
}

int32_t skinny_reserve(nc_context *ctx, uint32_t rows, uint32_t n, uint32_t k) {
    const uint32_t bpad = (std::min(rows, kSkMaxRows) + 7) / 8 * 8;
    const uint64_t kpad = ((uint64_t)k + 255) / 256 * 256, nsb = kpad / 256, sx_cols = skinny_sx_cols((uint32_t)nsb);
    int32_t rc;
    if ((rc = ensure(ctx, ctx->sk_xh, 2ull * kSkMaxRows * kpad * 2, false))) return rc;
    if ((rc = ensure(ctx, ctx->sk_sx, 2ull * kSkMaxRows * sx_cols * 2, true))) return rc;
    if ((rc = ensure(ctx, ctx->sk_xs, nsb * kSkMaxRows * sizeof(float), true))) return rc;
    if ((rc = ensure(ctx, ctx->sk_rs, kSkMaxRows * sizeof(float), true))) return rc;
    if (n) {
        uint64_t partial = 0, tiles = 0;
        for (int pair = 0; pair < 2; ++pair) {
            const SkinnyPlan plan = skinny_plan(ctx, n, (uint32_t)kpad, pair != 0, bpad);
            partial = std::max<uint64_t>(partial, plan.splits > 1 ? (uint64_t)plan.ntile128 * plan.splits * bpad * kSkTileRows * sizeof(float) : 0);
            tiles = std::max<uint64_t>(tiles, plan.ntile128);
        }
        if (partial && (rc = ensure(ctx, ctx->sk_partial, partial, false))) return rc;
        if ((rc = ensure(ctx, ctx->sk_counters, tiles * 4 * sizeof(unsigned int), true))) return rc;
    }
    return ensure(ctx, ctx->status, 256, true);
}

// Stages 9 to 32 rows for the skinny product, optionally rms-normed first.
int32_t skinny_stage(nc_context *ctx, cudaStream_t stream, const float *x_dev, uint32_t rows, uint64_t x_stride, uint32_t k,
                     uint32_t lo, uint32_t hi, bool norm, const float *gain, float floor, float *normed, uint64_t normed_stride) {
    int32_t rc;
    if ((rc = skinny_reserve(ctx, rows, 0, k))) return rc;
    SkinnyPrepParams p;
    memset(&p, 0, sizeof p);
    p.x = x_dev;
    p.x_stride = x_stride;
    p.xh = (__half *)ctx->sk_xh.ptr;
    p.sx = (__half *)ctx->sk_sx.ptr;
    p.xs = (float *)ctx->sk_xs.ptr;
    p.rs = (float *)ctx->sk_rs.ptr;
    p.rows = rows;
    p.bpad = (rows + 7) / 8 * 8;
    p.k = k;
    p.sx_cols = skinny_sx_cols(k / kSuperBlock);
    p.lo = lo;
    p.hi = hi;
    p.vector = ((uintptr_t)x_dev % 16 == 0 && x_stride % 4 == 0 && lo % 8 == 0) ? 1u : 0u;
    p.gain = gain;
    p.norm = norm ? 1u : 0u;
    p.floor = floor;
    p.normed = normed;
    p.normed_stride = normed_stride;
    const unsigned int prep_threads = std::min(1024u, std::max(256u, (k / kSuperBlock + 7) / 8 * 8 * 32));   // a warp a stretch, up to 32
    NC_CUDA(launch_dependent(skinny_prep_kernel, dim3(rows), dim3(prep_threads), 0, stream, p));
    ctx->launches++;
    ctx->sk_bpad = p.bpad;
    ctx->sk_sx_cols = p.sx_cols;
    Staging &slot = ctx->slots[ctx->cur];
    slot.rows = rows;
    slot.k = k;
    slot.granule = 256;
    slot.halves = 1;
    return 0;
}

int32_t skinny_product(nc_context *ctx, cudaStream_t stream, const nc_weight *w, float *out_dev, uint64_t out_stride,
                       const nc_step *chain, uint32_t n_steps) {
    const Staging &slot = ctx->slots[ctx->cur];
    const bool pair = w->layout == NC_LAYOUT_TILED_PAIR;
    const uint32_t bpad = ctx->sk_bpad;
    const SkinnyPlan plan = skinny_plan(ctx, w->n, w->k, pair, bpad);
    int32_t rc;
    if (plan.splits > 1 &&
        (rc = ensure(ctx, ctx->sk_partial, (uint64_t)plan.ntile128 * plan.splits * bpad * kSkTileRows * sizeof(float), false)))
        return rc;
    if ((rc = ensure(ctx, ctx->sk_counters, (uint64_t)plan.ntile128 * 4 * sizeof(unsigned int), true))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    SkinnyParams p;
    memset(&p, 0, sizeof p);
    if ((rc = tensor_map_16bit(&p.x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, ctx->sk_xh.ptr, w->k, 2 * bpad, 2 * bpad))) return rc;
    if ((rc = tensor_map_16bit(&p.sx_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, ctx->sk_sx.ptr, ctx->sk_sx_cols, 2 * bpad, 2 * bpad))) return rc;
    p.w = (const uint8_t *)w->data_dev;
    p.xs = (const float *)ctx->sk_xs.ptr;
    p.rs = (const float *)ctx->sk_rs.ptr;
    p.out = out_dev;
    p.out_stride = out_stride;
    p.partial = (float *)ctx->sk_partial.ptr;
    p.counters = (unsigned int *)ctx->sk_counters.ptr;
    p.status = (unsigned int *)ctx->status.ptr;
    p.n = w->n;
    p.rows = slot.rows;
    p.bpad = bpad;
    p.nsb = w->k / kSuperBlock;
    p.tiles32 = plan.tiles32;
    p.ntile128 = plan.ntile128;
    p.splits = plan.splits;
    p.pair = pair ? 1u : 0u;
    p.chain.n = n_steps;
    for (uint32_t s = 0; s < n_steps; ++s) p.chain.step[s] = chain[s];
    void (*kernel)(SkinnyParams);
    switch (bpad / 8) {
    case 1: kernel = skinny_q4k_tcgen05_kernel<1>; break;
    case 2: kernel = skinny_q4k_tcgen05_kernel<2>; break;
    case 3: kernel = skinny_q4k_tcgen05_kernel<3>; break;
    default: kernel = skinny_q4k_tcgen05_kernel<4>; break;
    }
    const uint32_t smem = skinny_smem_bytes(bpad);
    static bool raised[64][5] = {{false}};
    if (!raised[ctx->device & 63][bpad / 8]) {
        NC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised[ctx->device & 63][bpad / 8] = true;
    }
    NC_CUDA(launch_dependent(kernel, dim3(plan.grid), dim3(kSkThreads), smem, stream, p));
    ctx->launches++;
    return 0;
}

}  // namespace

extern "C" {

const char *neura_cuda_last_error(void) { return g_error.c_str(); }

int32_t neura_cuda_open(int32_t device, nc_context **out) {
    if (!out) return refuse(kBadArgument, "open needs somewhere to put the context");
    *out = nullptr;
    int count = 0;
    NC_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count)
        return refuse(kBadArgument, "device %d is not one of the %d GPUs this process sees", device, count);
    NC_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    NC_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return refuse(kBadState, "this library holds sm_100a code only and device %d is sm_%d%d", device, prop.major,
                      prop.minor);
    nc_context *ctx = new (std::nothrow) nc_context();
    if (!ctx) return refuse(kBadState, "out of host memory");
    ctx->device = device;
    ctx->sms = prop.multiProcessorCount;
    *out = ctx;
    return 0;
}

int32_t neura_cuda_close(nc_context *ctx) {
    if (!ctx) return 0;
    cudaSetDevice(ctx->device);
    if (ctx->capturing) {  // a recording cut short by an error: end it, or the thread stays in capture mode
        cudaGraph_t graph = nullptr;
        cudaStreamEndCapture(ctx->capture_stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
    }
    for (Staging &slot : ctx->slots)
        for (Region *region : {&slot.dig, &slot.cs, &slot.sums, &slot.chunks})
            if (region->ptr) cudaFree(region->ptr);
    for (Region *region : {&ctx->squares, &ctx->partial, &ctx->counters, &ctx->status, &ctx->stage_x, &ctx->stage_out, &ctx->attend_partial, &ctx->attend_counters, &ctx->argmax_scratch, &ctx->x_bf16, &ctx->pair_out,
                           &ctx->sk_xh, &ctx->sk_sx, &ctx->sk_xs, &ctx->sk_rs, &ctx->sk_partial, &ctx->sk_counters})
        if (region->ptr) cudaFree(region->ptr);
    delete ctx;
    return 0;
}

uint64_t neura_cuda_payload_bytes(uint32_t element, uint64_t elements) {
    if (element == NC_ELEMENT_SINGLE) return elements * 4;
    const uint32_t per = block_elements(element);
    if (!per) return 0;
    return (elements + per - 1) / per * block_bytes(element);
}

uint64_t neura_cuda_sealed_bytes(uint32_t element, uint32_t n, uint32_t k) {
    const uint32_t per = block_elements(element);
    if (!per || k % per || gguf_only(element)) return 0;
    const uint64_t padded = ((uint64_t)n + kTileRows - 1) / kTileRows * kTileRows;
    return padded * (k / per) * block_bytes(element);
}

int32_t neura_cuda_alloc(nc_context *ctx, uint64_t bytes, void **out_dev) {
    if (!ctx || !out_dev) return refuse(kBadArgument, "alloc needs a context and somewhere to put the pointer");
    NC_CUDA(cudaSetDevice(ctx->device));
    NC_CUDA(cudaMalloc(out_dev, bytes ? bytes : 1));
    return 0;
}

int32_t neura_cuda_free(nc_context *ctx, void *ptr_dev) {
    if (!ctx) return refuse(kBadArgument, "free needs a context");
    NC_CUDA(cudaSetDevice(ctx->device));
    NC_CUDA(cudaFree(ptr_dev));
    return 0;
}

int32_t neura_cuda_host_alloc(nc_context *ctx, uint64_t bytes, void **out_host) {
    if (!ctx || !out_host) return refuse(kBadArgument, "host_alloc needs a context and somewhere to put the pointer");
    NC_CUDA(cudaSetDevice(ctx->device));
    NC_CUDA(cudaMallocHost(out_host, bytes ? bytes : 1));
    return 0;
}

int32_t neura_cuda_host_free(nc_context *ctx, void *ptr_host) {
    if (!ctx) return refuse(kBadArgument, "host_free needs a context");
    NC_CUDA(cudaFreeHost(ptr_host));
    return 0;
}

int32_t neura_cuda_write(nc_context *ctx, void *stream, void *dst_dev, const void *src_host, uint64_t bytes) {
    if (!ctx || (bytes && (!dst_dev || !src_host))) return refuse(kBadArgument, "write needs both ends of the copy");
    NC_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return 0;
}

int32_t neura_cuda_read(nc_context *ctx, void *stream, void *dst_host, const void *src_dev, uint64_t bytes) {
    if (!ctx || (bytes && (!dst_host || !src_dev))) return refuse(kBadArgument, "read needs both ends of the copy");
    NC_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return 0;
}

int32_t neura_cuda_sync(nc_context *ctx, void *stream) {
    if (!ctx) return refuse(kBadArgument, "sync needs a context");
    NC_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return check_status(ctx);
}

int32_t neura_cuda_set_wait_limit(nc_context *ctx, uint64_t nanoseconds) {
    if (!ctx || !nanoseconds) return refuse(kBadArgument, "a wait limit needs a context and a time above zero");
    ctx->wait_nanos = nanoseconds;
    return 0;
}

int32_t neura_cuda_memory(nc_context *ctx, uint64_t *free_out, uint64_t *total_out) {
    if (!ctx) return refuse(kBadArgument, "a memory query needs a context");
    NC_CUDA(cudaSetDevice(ctx->device));
    size_t free_bytes = 0, total_bytes = 0;
    NC_CUDA(cudaMemGetInfo(&free_bytes, &total_bytes));
    if (free_out) *free_out = free_bytes;
    if (total_out) *total_out = total_bytes;
    return 0;
}

int32_t neura_cuda_reserve(nc_context *ctx, uint32_t rows, uint32_t n, uint32_t k) {
    if (!ctx || !rows || !n || !k) return refuse(kBadArgument, "reserve needs a context and a shape");
    NC_CUDA(cudaSetDevice(ctx->device));
    const uint32_t pass = rows < kMaxRowsPerPass ? rows : kMaxRowsPerPass;
    const uint64_t kpad = ((uint64_t)k + 255) / 256 * 256;
    int32_t rc;
    for (Staging &slot : ctx->slots) {   // every staging slot, so that no product grows one while a program is recorded
        if ((rc = ensure(ctx, slot.dig, kpad * 3 * pass, false))) return rc;
        if ((rc = ensure(ctx, slot.cs, kpad / 32 * 3 * pass * sizeof(float), false))) return rc;
        if ((rc = ensure(ctx, slot.sums, kpad / 256 * 3 * pass * 64, false))) return rc;
        if ((rc = ensure(ctx, slot.chunks, std::max<uint64_t>(kpad, ((uint64_t)n + 255) / 256 * 256) / 256 * sizeof(unsigned int), true))) return rc;
    }
    if ((rc = ensure(ctx, ctx->squares, (uint64_t)kMaxRowsPerPass * 1024 * sizeof(float), true))) return rc;
    // partial sums: the widest split is one unit per warp and two warps per tile ... bounded by the
    // plan for the narrowest block (32), computed with the resident grid of the largest kernel
    const uint32_t ntiles = (n + kTileRows - 1) / kTileRows;
    for (uint32_t element : {NC_ELEMENT_Q8_0, NC_ELEMENT_Q4K}) {
        if (k % block_elements(element)) continue;
        for (int resident = 1; resident <= 8; ++resident) {
            const GemvPlan plan = plan_gemv(ctx, element, n, k, resident);
            if ((rc = ensure(ctx, ctx->partial, (uint64_t)plan.ntiles * plan.maxp * pass * kTileRows * sizeof(float), false)))
                return rc;
        }
    }
    if ((rc = ensure(ctx, ctx->counters, (uint64_t)ntiles * sizeof(unsigned int), true))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    if ((rc = ensure(ctx, ctx->stage_x, (uint64_t)rows * k * sizeof(float), false))) return rc;
    if ((rc = ensure(ctx, ctx->stage_out, (uint64_t)rows * n * sizeof(float), false))) return rc;
    if (rows >= kSkinnyFrom && k % kSuperBlock == 0 && (rc = skinny_reserve(ctx, rows_per_pass(NC_ELEMENT_Q4K, rows), n, k))) return rc;
    return 0;
}

int32_t neura_cuda_reserve_bf16(nc_context *ctx, uint32_t rows, uint32_t k) {
    if (!ctx || !rows || !k) return refuse(kBadArgument, "reserve needs a context and a shape");
    NC_CUDA(cudaSetDevice(ctx->device));
    int32_t rc;
    if ((rc = ensure(ctx, ctx->x_bf16, (uint64_t)rows * k * 2, false))) return rc;
    if ((rc = ensure(ctx, ctx->pair_out, (uint64_t)ctx->sms * kGemmBM * kGemmBN * sizeof(float), false))) return rc;
    return ensure(ctx, ctx->status, 256, true);
}

int32_t neura_cuda_reserve_decoder(nc_context *ctx, uint32_t rows, uint32_t heads, uint32_t key_heads, uint32_t width,
                                   uint32_t capacity) {
    if (!ctx || !rows || !heads || !key_heads || !width || !capacity)
        return refuse(kBadArgument, "reserve needs a context and the decoder's shape");
    NC_CUDA(cudaSetDevice(ctx->device));
    int32_t rc;
    const uint64_t splits = ((uint64_t)capacity + 63) / 64;   // never fewer tiles than the attention launches
    if ((rc = ensure(ctx, ctx->attend_partial, (uint64_t)rows * heads * splits * (width + 2) * sizeof(float), false))) return rc;
    if ((rc = ensure(ctx, ctx->attend_counters, (uint64_t)rows * key_heads * sizeof(unsigned int), true))) return rc;
    if ((rc = ensure(ctx, ctx->argmax_scratch, (uint64_t)rows * 64 * 8 + (uint64_t)rows * 4 + 256, true))) return rc;
    return ensure(ctx, ctx->status, 256, true);
}

static int32_t seal_any(nc_context *ctx, void *stream, uint32_t element, uint32_t n, uint32_t k, const void *gguf_dev,
                        const void *second_dev, void *dst_dev) {
    if (!ctx || !gguf_dev || !dst_dev) return refuse(kBadArgument, "seal needs a context, a source and a destination");
    const uint32_t per = block_elements(element);
    if (!per || !n || !k || k % per || gguf_only(element))
        return refuse(kBadArgument, "a [%u, %u] tensor of element %u is not whole blocks this path seals (Q8_0 and Q4K are sealed; the other formats stay in GGUF order)", n, k, element);
    const uintptr_t align = element == NC_ELEMENT_Q4K ? 8 : 2;
    if ((uintptr_t)gguf_dev % align || (uintptr_t)second_dev % align || (uintptr_t)dst_dev % 16)
        return refuse(kBadArgument, "seal reads an 8-byte aligned tensor and writes a 16-byte aligned one");
    const uint64_t bytes = second_dev ? neura_cuda_sealed_pair_bytes(element, n, k) : neura_cuda_sealed_bytes(element, n, k);
    const uint64_t granules = element == NC_ELEMENT_Q4K ? bytes / 8 : bytes / 2;
    const uint64_t want = (granules + 255) / 256;
    const unsigned int blocks = (unsigned int)(want < (uint64_t)ctx->sms * 32 ? want : (uint64_t)ctx->sms * 32);
    if (element == NC_ELEMENT_Q4K)
        seal_q4k_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)gguf_dev, (const uint8_t *)second_dev,
                                                                  (uint8_t *)dst_dev, n, k / per, granules);
    else
        seal_q8_0_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)gguf_dev, (const uint8_t *)second_dev,
                                                                   (uint8_t *)dst_dev, n, k / per, granules);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    return 0;
}

uint64_t neura_cuda_sealed_pair_bytes(uint32_t element, uint32_t n, uint32_t k) {
    const uint32_t per = block_elements(element);
    if (!per || k % per) return 0;
    const uint64_t tiles = ((uint64_t)n + 15) / 16;
    return tiles * 32 * (k / per) * block_bytes(element);
}

int32_t neura_cuda_weight_seal(nc_context *ctx, void *stream, uint32_t element, uint32_t n, uint32_t k,
                               const void *gguf_dev, void *dst_dev) {
    return seal_any(ctx, stream, element, n, k, gguf_dev, nullptr, dst_dev);
}

int32_t neura_cuda_weight_seal_pair(nc_context *ctx, void *stream, uint32_t element, uint32_t n, uint32_t k,
                                    const void *gate_gguf_dev, const void *up_gguf_dev, void *dst_dev) {
    if (!up_gguf_dev) return refuse(kBadArgument, "a pair seals two tensors");
    return seal_any(ctx, stream, element, n, k, gate_gguf_dev, up_gguf_dev, dst_dev);
}

int32_t neura_cuda_dequant(nc_context *ctx, void *stream, const nc_weight *w, float *out_dev) {
    if (!ctx || !out_dev) return refuse(kBadArgument, "dequant needs a context and a destination");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (w->layout != NC_LAYOUT_GGUF && w->layout != NC_LAYOUT_TILED)
        return refuse(kBadArgument, "layout %u is neither the GGUF nor the tiled order (a sealed pair is dequantised from its two sources)", w->layout);
    WeightView view{(const uint8_t *)w->data_dev, w->element, w->layout, w->n, w->k};
    const uint64_t total = (uint64_t)w->n * w->k;
    const uint64_t want = (total + 255) / 256;
    const unsigned int blocks = (unsigned int)(want < (uint64_t)ctx->sms * 32 ? want : (uint64_t)ctx->sms * 32);
    dequant_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(view, out_dev);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    return 0;
}

int32_t neura_cuda_quantize(nc_context *ctx, void *stream, uint32_t element, const float *src_dev,
                            uint64_t elements, void *dst_dev) {
    if (!ctx || !src_dev || !dst_dev) return refuse(kBadArgument, "quantize needs a context, a source and a destination");
    const uint32_t per = block_elements(element);
    if (!per || !elements || elements % per)
        return refuse(kBadArgument, "%llu numbers do not fill whole blocks of element %u",
                      (unsigned long long)elements, element);
    if (element != NC_ELEMENT_Q8_0 && element != NC_ELEMENT_Q4K)
        return refuse(kBadArgument, "the device packs Q8_0 and Q4K blocks, not element %u", element);
    if ((uintptr_t)dst_dev % 2 || (uintptr_t)src_dev % 4)
        return refuse(kBadArgument, "quantize reads 4-byte aligned numbers and writes 2-byte aligned blocks");
    const uint64_t blocks = elements / per;
    const uint64_t want = (blocks + 7) / 8;
    const unsigned int grid = (unsigned int)(want < (uint64_t)ctx->sms * 16 ? want : (uint64_t)ctx->sms * 16);
    if (element == NC_ELEMENT_Q8_0)
        quantize_q8_0_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(src_dev, (uint8_t *)dst_dev, blocks);
    else
        quantize_q4k_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(src_dev, (uint8_t *)dst_dev, blocks);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    return 0;
}

int32_t neura_cuda_stage_window(nc_context *ctx, void *stream_, const float *x_dev, uint32_t rows, uint64_t x_stride,
                                uint32_t k, uint32_t element, uint32_t lo, uint32_t hi) {
    if (!ctx || !x_dev) return refuse(kBadArgument, "staging needs a context and activations");
    const uint32_t per = gguf_only(element) ? 0 : block_elements(element);   // (a product in GGUF order takes f32 rows as they are)
    if (!per || !k || k % per)
        return refuse(kBadArgument, "%u activations do not line up with blocks of element %u (Q8_0 or Q4K)", k, element);
    const uint32_t most = element == NC_ELEMENT_Q4K ? kSkMaxRows : kMaxRowsPerPass;
    if (rows == 0 || rows > most)
        return refuse(kBadArgument, "one staging holds 1 to %u rows of element %u, not %u", most, element, rows);
    if (lo >= hi || hi > k || lo % 32 || hi % 32)
        return refuse(kBadArgument, "a window [%u, %u) of %u activations starts and ends on multiples of 32 inside them", lo, hi, k);
    if (x_stride < hi - lo)
        return refuse(kBadArgument, "rows of %u activations overlap at stride %llu", hi - lo, (unsigned long long)x_stride);
    if ((uintptr_t)x_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    if (element == NC_ELEMENT_Q4K && (rows >= kSkinnyFrom || rows > kMaxRowsPerPass))
        return skinny_stage(ctx, (cudaStream_t)stream_, x_dev, rows, x_stride, k, lo, hi, false, nullptr, 0.0f, nullptr, 0);
    const uint64_t kpad = ((uint64_t)k + 255) / 256 * 256;
    const uint32_t ncols = rows * 3;
    int32_t rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].dig, kpad * ncols, false))) return rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].cs, kpad / 32 * ncols * sizeof(float), false))) return rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].sums, kpad / 256 * ncols * 64, false))) return rc;
    PrepParams prep;
    prep.x = x_dev;
    prep.x_stride = x_stride;
    prep.dig = (int8_t *)ctx->slots[ctx->cur].dig.ptr;
    prep.cs = (float *)ctx->slots[ctx->cur].cs.ptr;
    prep.sums = (uint32_t *)ctx->slots[ctx->cur].sums.ptr;
    prep.rows = rows;
    prep.k = k;
    prep.ncols = ncols;
    prep.granule = element == NC_ELEMENT_Q4K ? 256 : 32;
    prep.vector = ((uintptr_t)x_dev % 16 == 0 && x_stride % 4 == 0) ? 1u : 0u;
    prep.lo = lo;
    prep.hi = hi;
    const uint64_t prep_warps = (uint64_t)rows * (kpad / 256);
    NC_CUDA(launch_dependent(prep_kernel, dim3((unsigned int)((prep_warps + 3) / 4)), dim3(128), 0,
                             (cudaStream_t)stream_, prep));
    ctx->launches++;
    ctx->slots[ctx->cur].rows = rows;
    ctx->slots[ctx->cur].k = k;
    ctx->slots[ctx->cur].granule = prep.granule;
    ctx->slots[ctx->cur].halves = 0;
    return 0;
}

int32_t neura_cuda_stage(nc_context *ctx, void *stream_, const float *x_dev, uint32_t rows, uint64_t x_stride,
                         uint32_t k, uint32_t element) {
    if (k == 0) return refuse(kBadArgument, "staging no activations stages nothing");
    if (x_stride < k) return refuse(kBadArgument, "rows of %u activations overlap at stride %llu", k, (unsigned long long)x_stride);
    return neura_cuda_stage_window(ctx, stream_, x_dev, rows, x_stride, k, element, 0, k);
}

int32_t neura_cuda_linear_staged(nc_context *ctx, void *stream_, const nc_weight *w, float *out_dev,
                                 uint64_t out_stride, const nc_step *chain, uint32_t n_steps) {
    if (!ctx || !out_dev) return refuse(kBadArgument, "a product needs a context and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (w->layout != NC_LAYOUT_TILED && w->layout != NC_LAYOUT_TILED_PAIR)
        return refuse(kBadArgument, "the product streams a sealed weight (neura_cuda_weight_seal); this one is in GGUF order "
                                    "(a weight kept in GGUF order takes neura_cuda_linear, which needs no staging)");
    const bool pair = w->layout == NC_LAYOUT_TILED_PAIR;
    // a pair is planned as the matrix of both tensors' rows, 16 of each per 32-row tile
    const uint32_t plan_n = pair ? (w->n + 15) / 16 * 32 : w->n;
    const uint32_t granule = w->element == NC_ELEMENT_Q4K ? 256 : 32;
    if (!ctx->slots[ctx->cur].rows || ctx->slots[ctx->cur].k != w->k || ctx->slots[ctx->cur].granule != granule)
        return refuse(kBadArgument, "the staged activations (%u rows of %u for blocks of %u) do not fit a [%u, %u] weight of element %u",
                      ctx->slots[ctx->cur].rows, ctx->slots[ctx->cur].k, ctx->slots[ctx->cur].granule, w->n, w->k, w->element);
    if (out_stride < w->n)
        return refuse(kBadArgument, "rows of %u outputs overlap at stride %llu", w->n, (unsigned long long)out_stride);
    if (n_steps > NC_MAX_STEPS || (n_steps && !chain))
        return refuse(kBadArgument, "an epilogue holds at most %u steps", NC_MAX_STEPS);
    if ((uintptr_t)out_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    cudaStream_t stream = (cudaStream_t)stream_;
    if (ctx->slots[ctx->cur].halves) return skinny_product(ctx, stream, w, out_dev, out_stride, chain, n_steps);
    // a launch carries at most kRowsPerLaunch rows: beyond that the accumulators of the wider MMA tiles spill
    // and two launches over the same weights are faster than one
    for (uint32_t first = 0; first < ctx->slots[ctx->cur].rows; first += kRowsPerLaunch) {
        GemvParams p;
        memset(&p, 0, sizeof p);
        p.w = (const uint8_t *)w->data_dev;
        p.dig = (const uint8_t *)ctx->slots[ctx->cur].dig.ptr;
        p.cs = (const float *)ctx->slots[ctx->cur].cs.ptr;
        p.sums = (const uint8_t *)ctx->slots[ctx->cur].sums.ptr;
        p.out = out_dev + (uint64_t)first * out_stride;
        p.out_stride = out_stride;
        p.n = w->n;
        p.rows = std::min(kRowsPerLaunch, ctx->slots[ctx->cur].rows - first);
        p.ncols = p.rows * 3;
        p.col_stride = ctx->slots[ctx->cur].rows * 3;
        p.col0 = first * 3;
        p.pair = pair ? 1u : 0u;
        p.chain.n = n_steps;
        for (uint32_t s = 0; s < n_steps; ++s) {
            p.chain.step[s] = chain[s];
            if (chain[s].operand_dev)   // the operand is read at this launch's rows
                p.chain.step[s].operand_dev = chain[s].operand_dev + (int64_t)first * chain[s].row_stride;
        }
        switch ((p.ncols + 7) / 8) {
        case 1: rc = launch_gemv<1>(ctx, stream, w->element, p, plan_n, w->k); break;
        case 2: rc = launch_gemv<2>(ctx, stream, w->element, p, plan_n, w->k); break;
        default: rc = launch_gemv<3>(ctx, stream, w->element, p, plan_n, w->k); break;
        }
        if (rc) return rc;
    }
    return 0;
}

int32_t neura_cuda_staging_select(nc_context *ctx, uint32_t slot) {
    if (!ctx || slot >= kStagingSlots) return refuse(kBadArgument, "a context holds staging slots 0 to %u", kStagingSlots - 1);
    ctx->cur = slot;
    return 0;
}

int32_t neura_cuda_linear_staged_fused(nc_context *ctx, void *stream_, const nc_weight *w, float *out_dev, uint64_t out_stride,
                                       const nc_step *chain, uint32_t n_steps, uint32_t normed, float floor, nc_comm *reduce,
                                       const nc_then *then_) {
    if (!ctx || !out_dev) return refuse(kBadArgument, "a product needs a context and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (w->layout != NC_LAYOUT_TILED && w->layout != NC_LAYOUT_TILED_PAIR)
        return refuse(kBadArgument, "the product streams a sealed weight (neura_cuda_weight_seal); this one is in GGUF order");
    Staging &from = ctx->slots[ctx->cur];
    const bool pair = w->layout == NC_LAYOUT_TILED_PAIR;
    const uint32_t plan_n = pair ? (w->n + 15) / 16 * 32 : w->n;
    const uint32_t granule = w->element == NC_ELEMENT_Q4K ? 256 : 32;
    if (!from.rows || from.k != w->k || from.granule != granule)
        return refuse(kBadArgument, "the staged activations (%u rows of %u for blocks of %u) do not fit a [%u, %u] weight of element %u",
                      from.rows, from.k, from.granule, w->n, w->k, w->element);
    if (from.rows > 2 || from.halves) return refuse(kBadArgument, "a product that stages its own output carries 1 or 2 rows, not %u", from.rows);
    nc_then none = {NC_NO_SLOT, 0, 0, 0, nullptr, 0};
    const nc_then &want = then_ ? *then_ : none;
    const bool then = want.slot != NC_NO_SLOT;
    if (then && (want.slot >= kStagingSlots || want.slot == ctx->cur))
        return refuse(kBadArgument, "the output is staged into another slot than the one the product reads (0 to %u)", kStagingSlots - 1);
    if (out_stride < w->n || out_stride % 4 || (uintptr_t)out_dev % 16)
        return refuse(kBadArgument, "output rows of %u start 16-byte aligned and do not overlap (stride %llu)", w->n, (unsigned long long)out_stride);
    if (then && w->n % 8) return refuse(kBadArgument, "%u outputs do not stage in whole runs of eight", w->n);
    if (n_steps > NC_MAX_STEPS || (n_steps && !chain))
        return refuse(kBadArgument, "an epilogue holds at most %u steps", NC_MAX_STEPS);
    // where the output rows sit on the K axis of the product that will read them
    const uint32_t then_k = want.k ? want.k : w->n, lo = want.k ? want.lo : 0, hi = want.k ? want.hi : w->n;
    if (then && (hi - lo != w->n || hi > then_k || lo % 32 || then_k % granule))
        return refuse(kBadArgument, "rows of %u outputs are not the window [%u, %u) of %u activations in blocks of %u", w->n, lo, hi, then_k, granule);
    if (reduce) {
        if (!then) return refuse(kBadArgument, "a product that adds the ranks' sums up also stages them: name a slot");
        if (!reduce->connected) return refuse(kBadState, "the communicator is not connected to its peers");
        if (lo || w->n % 256 || (uint64_t)from.rows * w->n > reduce->max_count)
            return refuse(kBadArgument, "an exchange in the epilogue takes whole rows of a multiple of 256 numbers, at most %llu in all (got %u x %u)",
                          (unsigned long long)reduce->max_count, from.rows, w->n);
    }
    // the slot the output is staged into
    Staging &to = ctx->slots[then ? want.slot : ctx->cur];
    const uint64_t kpad = ((uint64_t)then_k + 255) / 256 * 256;
    const uint32_t ncols = from.rows * 3;
    if (then) {
        if (kpad / 256 > 1024) return refuse(kBadArgument, "rows of %u activations are more than this path stages (262144)", then_k);
        if ((rc = ensure(ctx, to.dig, kpad * ncols, false))) return rc;
        if ((rc = ensure(ctx, to.cs, kpad / 32 * ncols * sizeof(float), false))) return rc;
        if ((rc = ensure(ctx, to.sums, kpad / 256 * ncols * 64, false))) return rc;
        if ((rc = ensure(ctx, to.chunks, kpad / 256 * sizeof(unsigned int), true))) return rc;
    }
    if ((rc = ensure(ctx, ctx->squares, (uint64_t)kMaxRowsPerPass * 1024 * sizeof(float), true))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    GemvParams p;
    memset(&p, 0, sizeof p);
    p.w = (const uint8_t *)w->data_dev;
    p.dig = (const uint8_t *)from.dig.ptr;
    p.cs = (const float *)from.cs.ptr;
    p.sums = (const uint8_t *)from.sums.ptr;
    p.out = out_dev;
    p.out_stride = out_stride;
    p.n = w->n;
    p.rows = from.rows;
    p.ncols = ncols;
    p.col_stride = ncols;
    p.col0 = 0;
    p.pair = pair ? 1u : 0u;
    p.chain.n = n_steps;
    for (uint32_t s = 0; s < n_steps; ++s) p.chain.step[s] = chain[s];
    if (normed) {   // the input rows were staged with a norm's gain: their scalar is still to be applied
        p.sumsq = (const float *)ctx->squares.ptr;
        p.sumsq_chunks = (from.k + 255) / 256;
        p.floor = floor;
        p.inv_k = 1.0f / (float)from.k;
    }
    p.has_then = then ? 1u : 0u;
    StageAfter &a = p.then;
    a.prep.x = out_dev;
    a.prep.x_stride = out_stride;
    a.prep.dig = (int8_t *)to.dig.ptr;
    a.prep.cs = (float *)to.cs.ptr;
    a.prep.sums = (uint32_t *)to.sums.ptr;
    a.prep.rows = from.rows;
    a.prep.k = then_k;
    a.prep.ncols = ncols;
    a.prep.granule = granule;
    a.prep.vector = 1;
    a.prep.lo = lo;
    a.prep.hi = hi;
    a.gain = want.gain_dev;
    a.sumsq = want.squares ? (float *)ctx->squares.ptr : nullptr;
    a.counters = (unsigned int *)to.chunks.ptr;
    a.piece = pair ? 16 : 32;
    a.exchange = reduce ? reduce->view_dev : nullptr;
    a.wait_nanos = ctx->wait_nanos;
    a.status = (unsigned int *)ctx->status.ptr;
    if ((rc = launch_gemv_hooked(ctx, (cudaStream_t)stream_, w->element, p, plan_n, w->k))) return rc;
    if (then) {
        to.rows = from.rows;
        to.k = then_k;
        to.granule = granule;
        to.halves = 0;
    }
    return 0;
}

int32_t neura_cuda_linear_staged_then(nc_context *ctx, void *stream_, const nc_weight *w, float *out_dev, uint64_t out_stride,
                                      const nc_step *chain, uint32_t n_steps, uint32_t normed, float floor,
                                      uint32_t then_slot, const float *then_gain_dev, uint32_t then_squares) {
    const nc_then then = {then_slot, 0, 0, 0, then_gain_dev, then_squares};
    return neura_cuda_linear_staged_fused(ctx, stream_, w, out_dev, out_stride, chain, n_steps, normed, floor, nullptr, &then);
}

int32_t neura_cuda_linear(nc_context *ctx, void *stream_, const nc_weight *w, const float *x_dev, uint32_t rows,
                          uint64_t x_stride, float *out_dev, uint64_t out_stride, const nc_step *chain,
                          uint32_t n_steps) {
    if (!ctx || !x_dev || !out_dev) return refuse(kBadArgument, "a product needs a context, activations and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (rows == 0) return refuse(kBadArgument, "a product of no rows computes nothing");
    if (n_steps > NC_MAX_STEPS || (n_steps && !chain))
        return refuse(kBadArgument, "an epilogue holds at most %u steps", NC_MAX_STEPS);
    if (gguf_only(w->element)) {
        if (x_stride < w->k || out_stride < w->n)
            return refuse(kBadArgument, "rows of %u activations and %u outputs overlap at strides %llu and %llu", w->k, w->n,
                          (unsigned long long)x_stride, (unsigned long long)out_stride);
        if ((uintptr_t)x_dev % 4 || (uintptr_t)out_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
        return rows_product(ctx, (cudaStream_t)stream_, w, x_dev, rows, x_stride, out_dev, out_stride, chain, n_steps);
    }
    const uint32_t per = rows_per_pass(w->element, rows);
    for (uint32_t first = 0; first < rows; first += per) {
        const uint32_t pass = rows - first < per ? rows - first : per;
        if ((rc = neura_cuda_stage(ctx, stream_, x_dev + (uint64_t)first * x_stride, pass, x_stride, w->k, w->element)))
            return rc;
        nc_step steps[NC_MAX_STEPS];
        for (uint32_t s = 0; s < n_steps; ++s) {
            steps[s] = chain[s];
            if (chain[s].operand_dev)  // the operand is read at this pass's rows
                steps[s].operand_dev = chain[s].operand_dev + (int64_t)first * chain[s].row_stride;
        }
        if ((rc = neura_cuda_linear_staged(ctx, stream_, w, out_dev + (uint64_t)first * out_stride, out_stride, steps,
                                           n_steps)))
            return rc;
    }
    return 0;
}

int32_t neura_cuda_linear_bf16(nc_context *ctx, void *stream_, const nc_weight *w, const float *x_dev, uint32_t rows,
                               uint64_t x_stride, float *out_dev, uint64_t out_stride, const nc_step *chain,
                               uint32_t n_steps) {
    if (!ctx || !x_dev || !out_dev) return refuse(kBadArgument, "a product needs a context, activations and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (w->element != NC_ELEMENT_Q4K || (w->layout != NC_LAYOUT_TILED && w->layout != NC_LAYOUT_TILED_PAIR))
        return refuse(kBadArgument, "the tensor-core product takes a sealed Q4K weight (element %u, layout %u given)",
                      w->element, w->layout);
    if (rows == 0) return refuse(kBadArgument, "a product of no rows computes nothing");
    // a sealed gate|up pair is a sealed weight of twice the rows whose 32-row tiles hold 16 gate rows and the 16 up
    // rows of the same columns: the product runs over all of them into scratch, a second kernel joins the halves
    const bool pair = w->layout == NC_LAYOUT_TILED_PAIR;
    const uint32_t n_all = pair ? (w->n + 15) / 16 * 32 : w->n;
    if (x_stride < w->k || out_stride < w->n)
        return refuse(kBadArgument, "rows of %u activations and %u outputs overlap at strides %llu and %llu", w->k, w->n,
                      (unsigned long long)x_stride, (unsigned long long)out_stride);
    if (n_steps > NC_MAX_STEPS || (n_steps && !chain))
        return refuse(kBadArgument, "an epilogue holds at most %u steps", NC_MAX_STEPS);
    if ((uintptr_t)x_dev % 4 || (uintptr_t)out_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    if ((rc = ensure(ctx, ctx->x_bf16, (uint64_t)rows * w->k * 2, false))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    // few tiles (a chunk of a few hundred rows against a narrow weight) leave most SMs idle: runs of K then go to
    // different CTAs, which leave their sums in scratch for gemm_finish_kernel to add in order
    const uint32_t tiles = ((n_all + kGemmBN - 1) / kGemmBN) * ((rows + kGemmBM - 1) / kGemmBM);
    const uint32_t splits = tiles * 2 <= (uint32_t)ctx->sms ? std::min({8u, (uint32_t)ctx->sms / tiles, w->k / kSuperBlock}) : 1u;
    const bool scratch = splits > 1;   // (an unsplit pair is joined in the product's own epilogue)
    // (splits <= SMs / tiles and a tile covers at most 256 x 256 outputs, so the runs of any product fit the bound below:
    // sized once, the scratch never moves under a recorded program)
    if (scratch && (rc = ensure(ctx, ctx->pair_out, std::max<uint64_t>((uint64_t)splits * rows * n_all, (uint64_t)ctx->sms * kGemmBM * kGemmBN) * sizeof(float), false))) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    const uint64_t total = (uint64_t)rows * w->k;
    const uint64_t want = (total + 255) / 256;
    const unsigned int blocks = (unsigned int)(want < (uint64_t)ctx->sms * 16 ? want : (uint64_t)ctx->sms * 16);
    to_bf16_kernel<<<blocks, 256, 0, stream>>>(x_dev, x_stride, rows, w->k, (__nv_bfloat16 *)ctx->x_bf16.ptr);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    static bool raised[64] = {false};
    if (!raised[ctx->device & 63]) {
        NC_CUDA(cudaFuncSetAttribute(gemm_q4k_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem));
        raised[ctx->device & 63] = true;
    }
    GemmParams p;
    memset(&p, 0, sizeof p);
    if ((rc = tensor_map_16bit(&p.x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ctx->x_bf16.ptr, w->k, rows, kGemmBM))) return rc;
    p.w = (const uint8_t *)w->data_dev;
    p.x = (const __nv_bfloat16 *)ctx->x_bf16.ptr;
    p.out = scratch ? (float *)ctx->pair_out.ptr : out_dev;
    p.out_stride = scratch ? n_all : out_stride;
    p.split_stride = (uint64_t)rows * n_all;
    p.m = rows;
    p.n = n_all;
    p.k = w->k;
    p.units32 = (n_all + 31) / 32;
    p.status = (unsigned int *)ctx->status.ptr;
    Chain steps;
    memset(&steps, 0, sizeof steps);
    steps.n = n_steps;
    for (uint32_t s = 0; s < n_steps; ++s) steps.step[s] = chain[s];
    if (!scratch) p.chain = steps;
    if (pair && !scratch) {
        p.pair = 1;
        p.n_out = w->n;
    }
    // a plain product straight into the caller's rows: blocks of the output leave by bulk tensor stores where the
    // rows allow a tensor map (16-byte aligned, a multiple of 16 bytes apart)
    if (!pair && !scratch && (uintptr_t)out_dev % 16 == 0 && out_stride % 4 == 0) {
        if ((rc = tensor_map_f32_out(&p.out_map, out_dev, w->n, rows, out_stride))) return rc;
        p.tma_out = 1;
    }
    NC_CUDA(launch_dependent(gemm_q4k_tcgen05_kernel, dim3((n_all + kGemmBN - 1) / kGemmBN, (rows + kGemmBM - 1) / kGemmBM, splits),
                             dim3(kGemmThreads), kGemmSmem, stream, p));
    ctx->launches++;
    if (scratch) {
        const uint64_t cells = ((uint64_t)rows * w->n + 255) / 256;
        const unsigned int grid = (unsigned int)(cells < (uint64_t)ctx->sms * 16 ? cells : (uint64_t)ctx->sms * 16);
        gemm_finish_kernel<<<grid, 256, 0, stream>>>((const float *)ctx->pair_out.ptr, n_all, p.split_stride, splits, rows, w->n,
                                                     pair ? 1u : 0u, out_dev, out_stride, steps);
        ctx->launches++;
        NC_CUDA(cudaGetLastError());
    }
    return 0;
}

int32_t neura_cuda_rms_norm(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint64_t x_stride, uint32_t k,
                            const float *weight_dev, float floor, float *out_dev, uint64_t out_stride) {
    if (!ctx || !x_dev || !out_dev) return refuse(kBadArgument, "a norm needs a context, rows to norm and somewhere to put them");
    if (!rows || !k) return refuse(kBadArgument, "a norm of %u rows of %u numbers computes nothing", rows, k);
    if (x_stride < k || out_stride < k) return refuse(kBadArgument, "rows of %u numbers overlap at the strides given", k);
    if ((uintptr_t)x_dev % 4 || (uintptr_t)out_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    rms_norm_rows_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(x_dev, x_stride, k, weight_dev, floor, out_dev, out_stride);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    return 0;
}

int32_t neura_cuda_linear_host(nc_context *ctx, void *stream_, const nc_weight *w, const float *x_host,
                               uint32_t rows, float *out_host, const nc_step *chain, uint32_t n_steps) {
    if (!ctx || !x_host || !out_host) return refuse(kBadArgument, "a product needs a context, activations and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (rows == 0) return refuse(kBadArgument, "a product of no rows computes nothing");
    cudaStream_t stream = (cudaStream_t)stream_;
    const uint64_t x_bytes = (uint64_t)rows * w->k * sizeof(float), out_bytes = (uint64_t)rows * w->n * sizeof(float);
    if ((rc = ensure(ctx, ctx->stage_x, x_bytes, false))) return rc;
    if ((rc = ensure(ctx, ctx->stage_out, out_bytes, false))) return rc;
    NC_CUDA(cudaMemcpyAsync(ctx->stage_x.ptr, x_host, x_bytes, cudaMemcpyHostToDevice, stream));
    if ((rc = neura_cuda_linear(ctx, stream_, w, (const float *)ctx->stage_x.ptr, rows, w->k,
                                (float *)ctx->stage_out.ptr, w->n, chain, n_steps)))
        return rc;
    NC_CUDA(cudaMemcpyAsync(out_host, ctx->stage_out.ptr, out_bytes, cudaMemcpyDeviceToHost, stream));
    NC_CUDA(cudaStreamSynchronize(stream));
    return check_status(ctx);
}

}  // extern "C"

namespace {

// Checks the rows of an rms_norm + staging and fills its parameters (the scratch may grow).
int32_t norm_stage_params(nc_context *ctx, const float *x_dev, uint32_t rows, uint64_t x_stride, uint32_t k,
                          const float *weight_dev, float floor, uint32_t element, float *normed_dev,
                          uint64_t normed_stride, NormStageParams &p) {
    if (!ctx || !x_dev) return refuse(kBadArgument, "a norm needs a context and a row to norm");
    const uint32_t per = gguf_only(element) ? 0 : block_elements(element);
    if (!per || !k || k % per)
        return refuse(kBadArgument, "%u activations do not line up with blocks of element %u", k, element);
    if (rows == 0 || rows > kMaxRowsPerPass)
        return refuse(kBadArgument, "one staging holds 1 to %u rows, not %u", kMaxRowsPerPass, rows);
    if (x_stride < k || (normed_dev && normed_stride < k))
        return refuse(kBadArgument, "rows of %u numbers overlap at the strides given", k);
    if ((uintptr_t)x_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    const uint64_t kpad = ((uint64_t)k + 255) / 256 * 256;
    const uint32_t ncols = rows * 3;
    int32_t rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].dig, kpad * ncols, false))) return rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].cs, kpad / 32 * ncols * sizeof(float), false))) return rc;
    if ((rc = ensure(ctx, ctx->slots[ctx->cur].sums, kpad / 256 * ncols * 64, false))) return rc;
    p.prep.x = x_dev;
    p.prep.x_stride = x_stride;
    p.prep.dig = (int8_t *)ctx->slots[ctx->cur].dig.ptr;
    p.prep.cs = (float *)ctx->slots[ctx->cur].cs.ptr;
    p.prep.sums = (uint32_t *)ctx->slots[ctx->cur].sums.ptr;
    p.prep.rows = rows;
    p.prep.k = k;
    p.prep.ncols = ncols;
    p.prep.granule = element == NC_ELEMENT_Q4K ? 256 : 32;
    p.prep.vector = ((uintptr_t)x_dev % 16 == 0 && x_stride % 4 == 0) ? 1u : 0u;
    p.prep.lo = 0;
    p.prep.hi = k;
    p.weight = weight_dev;
    p.normed = normed_dev;
    p.normed_stride = normed_stride;
    p.floor = floor;
    return 0;
}

}  // namespace

extern "C" {

int32_t neura_cuda_rms_norm_stage(nc_context *ctx, void *stream_, const float *x_dev, uint32_t rows, uint64_t x_stride,
                                  uint32_t k, const float *weight_dev, float floor, uint32_t element,
                                  float *normed_dev, uint64_t normed_stride) {
    if (ctx && x_dev && element == NC_ELEMENT_Q4K && rows >= kSkinnyFrom) {   // many rows: staged for the skinny product
        if (rows > kSkMaxRows) return refuse(kBadArgument, "one staging holds 1 to %u rows, not %u", kSkMaxRows, rows);
        if (!k || k % kSuperBlock) return refuse(kBadArgument, "%u activations do not line up with blocks of element %u", k, element);
        if (x_stride < k || (normed_dev && normed_stride < k))
            return refuse(kBadArgument, "rows of %u numbers overlap at the strides given", k);
        if ((uintptr_t)x_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
        return skinny_stage(ctx, (cudaStream_t)stream_, x_dev, rows, x_stride, k, 0, k, true, weight_dev, floor, normed_dev, normed_stride);
    }
    NormStageParams p;
    int32_t rc;
    if ((rc = norm_stage_params(ctx, x_dev, rows, x_stride, k, weight_dev, floor, element, normed_dev, normed_stride, p)))
        return rc;
    // one warp a 256-column chunk where the row allows it: the chunks of a row are then digitised side by side
    // (with 8 warps a 5120-column row took three chunks a warp in turn; 6 % of the 32B decode step)
    const uint32_t chunks = (k + 255) / 256;
    const uint32_t threads = chunks <= 8 ? 256u : chunks >= 32 ? 1024u : chunks * 32u;
    NC_CUDA(launch_dependent(rms_norm_stage_kernel, dim3(rows), dim3(threads), 0, (cudaStream_t)stream_, p));
    ctx->launches++;
    ctx->slots[ctx->cur].rows = rows;
    ctx->slots[ctx->cur].k = k;
    ctx->slots[ctx->cur].granule = p.prep.granule;
    ctx->slots[ctx->cur].halves = 0;
    return 0;
}

static int32_t rope_cache_any(nc_context *ctx, void *stream_, float *qkv_dev, uint64_t row_stride,
                              const uint32_t *position_dev, float base, uint32_t batch, uint32_t heads,
                              uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                              float *values_dev, uint32_t shared) {
    if (!ctx || !qkv_dev || !position_dev || !keys_dev || !values_dev)
        return refuse(kBadArgument, "rope needs a context, the q|k|v rows, their positions and a cache");
    if (!batch || !heads || !key_heads || !width || width % 2 || !capacity)
        return refuse(kBadArgument, "a rotation of %u heads of width %u over %u slots turns nothing", heads, width, capacity);
    if (row_stride < (uint64_t)(heads + 2 * key_heads) * width)
        return refuse(kBadArgument, "a q|k|v row of %u numbers overlaps at stride %llu", (heads + 2 * key_heads) * width,
                      (unsigned long long)row_stride);
    RopeCacheParams p{qkv_dev, row_stride, position_dev, keys_dev, values_dev, base, batch, heads, key_heads, width, capacity, shared};
    const uint32_t work = batch * ((heads + key_heads) * (width / 2) + key_heads * width);
    NC_CUDA(launch_dependent(rope_cache_kernel, dim3((work + 255) / 256), dim3(256), 0, (cudaStream_t)stream_, p));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_rope_cache(nc_context *ctx, void *stream_, float *qkv_dev, uint64_t row_stride,
                              const uint32_t *position_dev, float base, uint32_t batch, uint32_t heads,
                              uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                              float *values_dev) {
    return rope_cache_any(ctx, stream_, qkv_dev, row_stride, position_dev, base, batch, heads, key_heads, width, capacity, keys_dev,
                          values_dev, 0);
}

int32_t neura_cuda_rope_cache_rows(nc_context *ctx, void *stream_, float *qkv_dev, uint64_t row_stride,
                                   const uint32_t *position_dev, float base, uint32_t rows, uint32_t heads,
                                   uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                                   float *values_dev) {
    return rope_cache_any(ctx, stream_, qkv_dev, row_stride, position_dev, base, rows, heads, key_heads, width, capacity, keys_dev,
                          values_dev, 1);
}

}  // extern "C"

namespace {

// Attention of one new row per sequence; with `fresh_keys` the rows at q_dev are the un-turned q | k | v of this
// step and the kernel turns them and writes the cache itself.
int32_t attend_any(nc_context *ctx, void *stream_, const float *q_dev, uint64_t q_stride, const float *keys_dev,
                   const float *values_dev, const uint32_t *position_dev, float scale, uint32_t batch, uint32_t heads,
                   uint32_t key_heads, uint32_t width, uint32_t capacity, float *out_dev, uint64_t out_stride,
                   float *fresh_keys, float *fresh_values, const float2 *rope_table, uint32_t shared = 0) {
    if (!ctx || !q_dev || !keys_dev || !values_dev || !position_dev || !out_dev)
        return refuse(kBadArgument, "attention needs a context, queries, a cache, positions and an output");
    if (!batch || !heads || !key_heads || heads % key_heads || !width || !capacity)
        return refuse(kBadArgument, "%u query heads do not share %u key heads", heads, key_heads);
    const uint32_t group = heads / key_heads;
    if (group > kAttendMaxGroup)
        return refuse(kBadArgument, "%u query heads per key head are more than the %u the attention kernel serves together",
                      group, kAttendMaxGroup);
    if (width != 64 && width != 128)
        return refuse(kBadArgument, "the attention kernel is built for heads of width 64 and 128, not %u", width);
    if (capacity > 64 * 128)
        return refuse(kBadArgument, "a cache of %u slots is more than the %u the attention kernel splits", capacity, 64 * 128);
    // up to 8 splits merge inside a thread-block cluster; longer caches merge through global memory
    // (tiles of 128 positions take 133 KB of shared memory, one CTA an SM: with many sequences that leaves the grid
    // several waves long, so once the 128-position tiles outnumber the SMs the kernel takes tiles of 64, three CTAs an
    // SM, and merges through global memory)
    const bool crowded = (uint64_t)batch * key_heads * ((capacity + 127) / 128) > (uint64_t)ctx->sms;
    const uint32_t tile = capacity <= kAttendMaxCluster * 64 || crowded ? 64 : 128;
    // a full cluster wherever the cache is long enough to give every CTA 64 positions: eight CTAs of 80 positions
    // beat five of 128 (1.2 % of the 32B decode step at 640 cache rows)
    uint32_t splits = (capacity + tile - 1) / tile;
    if (splits < kAttendMaxCluster) splits = std::max(splits, std::min(kAttendMaxCluster, (capacity + 63) / 64));
    const bool cluster = splits <= kAttendMaxCluster;
    const size_t smem = ((size_t)tile * (2 * width + 4) + (size_t)kAttendMaxGroup * width +
                         (size_t)kAttendMaxGroup * kAttendMaxChunk + (size_t)kAttendMaxGroup * 2) * sizeof(float);
    void (*kernel)(AttendParams);
    const bool turning = fresh_keys != nullptr;
    const int which = (turning ? 8 : 0) + (width == 128 ? 4 : 0) + (tile == 128 ? 2 : 0) + (cluster ? 1 : 0);
    switch (which) {
    case 0: kernel = attend_kernel<64, 64, false, false>; break;
    case 1: kernel = attend_kernel<64, 64, true, false>; break;
    case 2: kernel = attend_kernel<64, 128, false, false>; break;
    case 3: kernel = attend_kernel<64, 128, true, false>; break;
    case 4: kernel = attend_kernel<128, 64, false, false>; break;
    case 5: kernel = attend_kernel<128, 64, true, false>; break;
    case 6: kernel = attend_kernel<128, 128, false, false>; break;
    case 7: kernel = attend_kernel<128, 128, true, false>; break;
    case 8: kernel = attend_kernel<64, 64, false, true>; break;
    case 9: kernel = attend_kernel<64, 64, true, true>; break;
    case 10: kernel = attend_kernel<64, 128, false, true>; break;
    case 11: kernel = attend_kernel<64, 128, true, true>; break;
    case 12: kernel = attend_kernel<128, 64, false, true>; break;
    case 13: kernel = attend_kernel<128, 64, true, true>; break;
    case 14: kernel = attend_kernel<128, 128, false, true>; break;
    default: kernel = attend_kernel<128, 128, true, true>; break;
    }
    static bool raised[64][16] = {{false}};
    if (!raised[ctx->device & 63][which]) {
        NC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised[ctx->device & 63][which] = true;
    }
    int32_t rc;
    if (!cluster) {
        if ((rc = ensure(ctx, ctx->attend_partial, (uint64_t)batch * heads * splits * (width + 2) * sizeof(float), false))) return rc;
        if ((rc = ensure(ctx, ctx->attend_counters, (uint64_t)batch * key_heads * sizeof(unsigned int), true))) return rc;
    }
    AttendParams p{q_dev, q_stride, keys_dev, values_dev, position_dev, out_dev, out_stride,
                   (float *)ctx->attend_partial.ptr, (unsigned int *)ctx->attend_counters.ptr, scale,
                   batch, heads, key_heads, width, capacity, splits, fresh_keys, fresh_values, rope_table, shared};
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(batch * key_heads * splits);
    config.blockDim = dim3(kAttendThreads);
    config.dynamicSmemBytes = smem;
    config.stream = (cudaStream_t)stream_;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = splits;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = cluster ? 2 : 1;
    NC_CUDA(cudaLaunchKernelEx(&config, kernel, p));
    ctx->launches++;
    return 0;
}

}  // namespace

extern "C" {

int32_t neura_cuda_attend(nc_context *ctx, void *stream, const float *q_dev, uint64_t q_stride, const float *keys_dev,
                          const float *values_dev, const uint32_t *position_dev, float scale, uint32_t batch,
                          uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *out_dev,
                          uint64_t out_stride) {
    return attend_any(ctx, stream, q_dev, q_stride, keys_dev, values_dev, position_dev, scale, batch, heads, key_heads,
                      width, capacity, out_dev, out_stride, nullptr, nullptr, nullptr);
}

int32_t neura_cuda_attend_rows(nc_context *ctx, void *stream, const float *q_dev, uint64_t q_stride, const float *keys_dev,
                               const float *values_dev, const uint32_t *position_dev, float scale, uint32_t rows,
                               uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *out_dev,
                               uint64_t out_stride) {
    // many rows (a wide prompt chunk): blocks of 16 rows share every tile of the cache they read
    const bool lined_up = (uintptr_t)q_dev % 16 == 0 && q_stride % 4 == 0 && (uintptr_t)keys_dev % 16 == 0 && (uintptr_t)values_dev % 16 == 0;
    if (ctx && q_dev && keys_dev && values_dev && position_dev && out_dev && rows >= kAttendBlockFrom && lined_up && key_heads &&
        heads % key_heads == 0 && heads / key_heads <= kAttendMaxGroup && (width == 64 || width == 128) && capacity &&
        q_stride >= (uint64_t)heads * width && out_stride >= (uint64_t)heads * width) {
        const uint32_t group = heads / key_heads;
        const size_t smem = attend_block_smem(width, group);
        void (*kernel)(AttendBlockParams) = nullptr;
        switch ((width == 128 ? 8 : 0) + group - 1) {
#define NC_BLOCK_CASE(G) case G - 1: kernel = attend_block_kernel<64, G>; break; case 8 + G - 1: kernel = attend_block_kernel<128, G>; break;
            NC_BLOCK_CASE(1) NC_BLOCK_CASE(2) NC_BLOCK_CASE(3) NC_BLOCK_CASE(4) NC_BLOCK_CASE(5) NC_BLOCK_CASE(6) NC_BLOCK_CASE(7) NC_BLOCK_CASE(8)
#undef NC_BLOCK_CASE
        }
        static bool raised[64][16] = {{false}};
        if (!raised[ctx->device & 63][(width == 128 ? 8 : 0) + group - 1]) {
            NC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            raised[ctx->device & 63][(width == 128 ? 8 : 0) + group - 1] = true;
        }
        AttendBlockParams p{q_dev, q_stride, keys_dev, values_dev, position_dev, out_dev, out_stride, scale, rows, heads, key_heads, capacity};
        NC_CUDA(launch_dependent(kernel, dim3((rows + kBlockRows - 1) / kBlockRows * key_heads), dim3(kBlockThreads), smem,
                                 (cudaStream_t)stream, p));
        ctx->launches++;
        return 0;
    }
    return attend_any(ctx, stream, q_dev, q_stride, keys_dev, values_dev, position_dev, scale, rows, heads, key_heads,
                      width, capacity, out_dev, out_stride, nullptr, nullptr, nullptr, 1);
}

int32_t neura_cuda_rope_table(nc_context *ctx, void *stream, const uint32_t *position_dev, float base, uint32_t batch,
                              uint32_t width, float *table_dev) {
    if (!ctx || !position_dev || !table_dev || !batch || !width || width % 2)
        return refuse(kBadArgument, "the angles need a context, cursors, an even head width and a table");
    if ((uintptr_t)table_dev % 8) return refuse(kBadArgument, "the table of (cosine, sine) pairs starts on an 8-byte boundary");
    const uint32_t total = batch * (width / 2);
    NC_CUDA(launch_dependent(rope_table_kernel, dim3((total + 63) / 64), dim3(64), 0, (cudaStream_t)stream, position_dev, base,
                             batch, width, (float2 *)table_dev));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_rope_attend(nc_context *ctx, void *stream, const float *qkv_dev, uint64_t row_stride,
                               const uint32_t *position_dev, const float *table_dev, float scale, uint32_t batch,
                               uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                               float *values_dev, float *out_dev, uint64_t out_stride) {
    if (!keys_dev || !values_dev || !table_dev)
        return refuse(kBadArgument, "attention needs the cache it writes the new row to and the step's angles");
    return attend_any(ctx, stream, qkv_dev, row_stride, keys_dev, values_dev, position_dev, scale, batch, heads, key_heads,
                      width, capacity, out_dev, out_stride, keys_dev, values_dev, (const float2 *)table_dev);
}

int32_t neura_cuda_argmax_segments(nc_context *ctx, void *stream_, const float *x_dev, uint32_t rows, uint32_t width,
                                   uint64_t stride, uint32_t segment, uint64_t segment_stride, uint32_t *out_dev) {
    if (!ctx || !x_dev || !out_dev || !rows || !width) return refuse(kBadArgument, "argmax needs a context, rows and an output");
    if (!segment || width % segment) return refuse(kBadArgument, "rows of %u numbers do not split in segments of %u", width, segment);
    const uint32_t slices = width >= 8192 ? 64 : 1;
    int32_t rc;
    if ((rc = ensure(ctx, ctx->argmax_scratch, (uint64_t)rows * slices * 8 + (uint64_t)rows * 4 + 256, true))) return rc;
    ArgmaxParams p;
    p.x = x_dev;
    p.stride = stride;
    p.segment = segment;
    p.segment_stride = segment_stride;
    p.width = width;
    p.slices = slices;
    p.out = out_dev;
    p.counters = (unsigned int *)ctx->argmax_scratch.ptr;
    p.slice_value = (float *)((unsigned char *)ctx->argmax_scratch.ptr + (((uint64_t)rows * 4 + 255) / 256) * 256);
    p.slice_index = (uint32_t *)(p.slice_value + (uint64_t)rows * slices);
    NC_CUDA(launch_dependent(argmax_kernel, dim3(rows * slices), dim3(256), 0, (cudaStream_t)stream_, p));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_argmax(nc_context *ctx, void *stream_, const float *x_dev, uint32_t rows, uint32_t width,
                          uint64_t stride, uint32_t *out_dev) {
    if (stride < width) return refuse(kBadArgument, "rows of %u numbers overlap at stride %llu", width, (unsigned long long)stride);
    return neura_cuda_argmax_segments(ctx, stream_, x_dev, rows, width, stride, width, 0, out_dev);
}

int32_t neura_cuda_embed(nc_context *ctx, void *stream_, const nc_weight *table, const uint32_t *tokens_dev,
                         uint32_t rows, float *out_dev, uint64_t out_stride) {
    if (!ctx || !tokens_dev || !out_dev || !rows) return refuse(kBadArgument, "a gather needs a context, tokens and an output");
    int32_t rc;
    if ((rc = check_weight(table))) return rc;
    if (out_stride < table->k) return refuse(kBadArgument, "rows of %u numbers overlap at stride %llu", table->k, (unsigned long long)out_stride);
    WeightView view{(const uint8_t *)table->data_dev, table->element, table->layout, table->n, table->k};
    const uint32_t work = rows * table->k;
    NC_CUDA(launch_dependent(embed_kernel, dim3((work + 255) / 256), dim3(256), 0, (cudaStream_t)stream_, view, tokens_dev,
                             rows, out_dev, out_stride));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_advance(nc_context *ctx, void *stream_, uint32_t *position_dev, uint32_t rows, uint32_t by) {
    if (!ctx || !position_dev || !rows) return refuse(kBadArgument, "advance needs a context and positions");
    NC_CUDA(launch_dependent(advance_kernel, dim3((rows + 127) / 128), dim3(128), 0, (cudaStream_t)stream_, position_dev, rows, by));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_comm_create(nc_context *ctx, uint64_t max_count, nc_comm **out, void *handle_out) {
    if (!ctx || !out || !handle_out || !max_count) return refuse(kBadArgument, "a communicator needs a context, a size and somewhere to put its handle");
    NC_CUDA(cudaSetDevice(ctx->device));
    nc_comm *comm = new (std::nothrow) nc_comm();
    if (!comm) return refuse(kBadState, "out of host memory");
    comm->device = ctx->device;
    comm->max_count = (max_count + 3) / 4 * 4;
    comm->slot_bytes = (comm->max_count * sizeof(float) + 255) / 256 * 256;
    comm->chunks_most = (uint32_t)((comm->max_count + 255) / 256);
    comm->header_bytes = (kCommChunkFlagsAt + 32 * comm->chunks_most + 255) / 256 * 256;
    const uint64_t bytes = comm->header_bytes + 2 * kMaxRanks * comm->slot_bytes;   // two slots of one seat per sender
    cudaError_t e = cudaMalloc((void **)&comm->mine, bytes);
    if (e == cudaSuccess) e = cudaMemset(comm->mine, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&comm->view_dev, sizeof(ExchangeView));
    cudaIpcMemHandle_t handle;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&handle, comm->mine);
    if (e != cudaSuccess) {
        if (comm->mine) cudaFree(comm->mine);
        if (comm->view_dev) cudaFree(comm->view_dev);
        delete comm;
        return cuda_refuse(e, "neura_cuda_comm_create");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    memcpy(handle_out, &handle, sizeof handle);
    *out = comm;
    return 0;
}

static int32_t comm_publish_view(nc_comm *comm) {
    ExchangeView view;
    memset(&view, 0, sizeof view);
    view.mine = comm->mine;
    for (uint32_t r = 0; r < comm->world; ++r) view.peer[r] = comm->peer[r];
    view.slot_bytes = comm->slot_bytes;
    view.header_bytes = comm->header_bytes;
    view.world = comm->world;
    view.rank = comm->rank;
    view.chunks_most = comm->chunks_most;
    NC_CUDA(cudaMemcpy(comm->view_dev, &view, sizeof view, cudaMemcpyHostToDevice));
    return 0;
}

int32_t neura_cuda_comm_connect(nc_context *ctx, nc_comm *comm, uint32_t rank, uint32_t world, const void *handles) {
    if (!ctx || !comm || !handles) return refuse(kBadArgument, "connect needs a context, a communicator and the ranks' handles");
    if (world < 2 || world > kMaxRanks || rank >= world)
        return refuse(kBadArgument, "rank %u of %u is not a place in a group of 2 to %u", rank, world, kMaxRanks);
    if (comm->connected) return refuse(kBadState, "this communicator is already connected");
    NC_CUDA(cudaSetDevice(ctx->device));
    for (uint32_t r = 0; r < world; ++r) {
        if (r == rank) {
            comm->peer[r] = comm->mine;
            continue;
        }
        cudaIpcMemHandle_t handle;
        memcpy(&handle, (const unsigned char *)handles + 64 * r, sizeof handle);
        NC_CUDA(cudaIpcOpenMemHandle((void **)&comm->peer[r], handle, cudaIpcMemLazyEnablePeerAccess));
    }
    comm->world = world;
    comm->rank = rank;
    comm->connected = true;
    return comm_publish_view(comm);
}

int32_t neura_cuda_comm_connect_local(nc_context *ctx, nc_comm *comm, uint32_t rank, uint32_t world, nc_comm *const *all) {
    if (!ctx || !comm || !all) return refuse(kBadArgument, "connect needs a context, a communicator and the group's communicators");
    if (world < 2 || world > kMaxRanks || rank >= world)
        return refuse(kBadArgument, "rank %u of %u is not a place in a group of 2 to %u", rank, world, kMaxRanks);
    if (comm->connected) return refuse(kBadState, "this communicator is already connected");
    if (all[rank] != comm) return refuse(kBadArgument, "place %u of the group holds another communicator", rank);
    NC_CUDA(cudaSetDevice(ctx->device));
    for (uint32_t r = 0; r < world; ++r) {
        if (!all[r] || !all[r]->mine) return refuse(kBadArgument, "place %u of the group is empty", r);
        if (all[r]->slot_bytes != comm->slot_bytes)
            return refuse(kBadArgument, "the communicators of a group are created for the same count");
        if (all[r]->device != comm->device) {   // another GPU of this process: its memory has to be reachable from here
            int reachable = 0;
            NC_CUDA(cudaDeviceCanAccessPeer(&reachable, comm->device, all[r]->device));
            if (!reachable) return refuse(kBadState, "device %d cannot reach the memory of device %d", comm->device, all[r]->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(all[r]->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_refuse(e, "cudaDeviceEnablePeerAccess");
            cudaGetLastError();
        }
        comm->peer[r] = all[r]->mine;
    }
    comm->world = world;
    comm->rank = rank;
    comm->connected = true;
    comm->local = true;
    return comm_publish_view(comm);
}

int32_t neura_cuda_allreduce(nc_context *ctx, void *stream_, nc_comm *comm, float *inout_dev, uint32_t count) {
    if (!ctx || !comm || !inout_dev || !count) return refuse(kBadArgument, "an all-reduce needs a context, a communicator and numbers");
    if (!comm->connected) return refuse(kBadState, "the communicator is not connected to its peers");
    if (count % 4 || count > comm->max_count || (uintptr_t)inout_dev % 16)
        return refuse(kBadArgument, "an all-reduce takes a 16-byte aligned multiple of 4 numbers, at most %llu (got %u)",
                      (unsigned long long)comm->max_count, count);
    int32_t rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    AllreduceParams p;
    memset(&p, 0, sizeof p);
    p.mine = comm->mine;
    for (uint32_t r = 0; r < comm->world; ++r) p.peer[r] = comm->peer[r];
    p.inout = inout_dev;
    p.slot_bytes = comm->slot_bytes;
    p.header_bytes = comm->header_bytes;
    p.count = count;
    p.world = comm->world;
    p.rank = comm->rank;
    p.status = (unsigned int *)ctx->status.ptr;
    p.wait_nanos = ctx->wait_nanos;
    const unsigned int threads = count / 4 >= 1024 ? 1024 : ((count / 4 + 31) / 32 * 32 < 32 ? 32 : (count / 4 + 31) / 32 * 32);
    NC_CUDA(launch_dependent(allreduce_kernel, dim3(1), dim3(threads), 0, (cudaStream_t)stream_, p));
    ctx->launches++;
    return 0;
}

int32_t neura_cuda_allreduce_norm_stage(nc_context *ctx, void *stream_, nc_comm *comm, float *inout_dev, uint32_t rows,
                                        uint32_t k, const float *weight_dev, float floor, uint32_t element) {
    if (!ctx || !comm || !inout_dev || !rows || !k) return refuse(kBadArgument, "an all-reduce needs a context, a communicator and rows");
    if (!comm->connected) return refuse(kBadState, "the communicator is not connected to its peers");
    const uint64_t count = (uint64_t)rows * k;
    if (count % 4 || count > comm->max_count || (uintptr_t)inout_dev % 16)
        return refuse(kBadArgument, "an all-reduce takes a 16-byte aligned multiple of 4 numbers, at most %llu (got %llu)",
                      (unsigned long long)comm->max_count, (unsigned long long)count);
    NormStageParams then;
    int32_t rc;
    if ((rc = norm_stage_params(ctx, inout_dev, rows, k, k, weight_dev, floor, element, nullptr, 0, then))) return rc;
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    AllreduceParams p;
    memset(&p, 0, sizeof p);
    p.mine = comm->mine;
    for (uint32_t r = 0; r < comm->world; ++r) p.peer[r] = comm->peer[r];
    p.inout = inout_dev;
    p.slot_bytes = comm->slot_bytes;
    p.header_bytes = comm->header_bytes;
    p.count = (uint32_t)count;
    p.world = comm->world;
    p.rank = comm->rank;
    p.status = (unsigned int *)ctx->status.ptr;
    p.wait_nanos = ctx->wait_nanos;
    NC_CUDA(launch_dependent(allreduce_norm_stage_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream_, p, then));
    ctx->launches++;
    ctx->slots[ctx->cur].rows = rows;
    ctx->slots[ctx->cur].k = k;
    ctx->slots[ctx->cur].granule = then.prep.granule;
    ctx->slots[ctx->cur].halves = 0;
    return 0;
}

int32_t neura_cuda_comm_destroy(nc_context *ctx, nc_comm *comm) {
    if (!comm) return 0;
    if (ctx) cudaSetDevice(ctx->device);
    for (uint32_t r = 0; r < comm->world && !comm->local; ++r)
        if (r != comm->rank && comm->peer[r]) cudaIpcCloseMemHandle(comm->peer[r]);
    if (comm->mine) cudaFree(comm->mine);
    if (comm->view_dev) cudaFree(comm->view_dev);
    delete comm;
    return 0;
}

int32_t neura_cuda_linear_static(nc_context *ctx, void *stream_, const nc_weight *w, const float *x_dev,
                                 uint32_t rows, uint64_t x_stride, float *out_dev, uint64_t out_stride,
                                 const nc_step *chain, uint32_t n_steps) {
    if (!ctx || !x_dev || !out_dev) return refuse(kBadArgument, "a product needs a context, activations and an output");
    int32_t rc;
    if ((rc = check_weight(w))) return rc;
    if (w->layout != NC_LAYOUT_TILED)
        return refuse(kBadArgument, "the product streams a sealed weight (neura_cuda_weight_seal); this one is in GGUF order");
    if (rows == 0 || rows > kStaticMaxRows || w->k > kStaticMaxK || w->n > kStaticMaxN)
        return refuse(kBadArgument,
                      "the allocation-free product holds scratch for at most %u rows against a [%u, %u] weight; "
                      "%u rows against [%u, %u] need neura_cuda_linear",
                      kStaticMaxRows, kStaticMaxN, kStaticMaxK, rows, w->n, w->k);
    if (x_stride < w->k || out_stride < w->n)
        return refuse(kBadArgument, "rows of %u activations and %u outputs overlap at strides %llu and %llu", w->k, w->n,
                      (unsigned long long)x_stride, (unsigned long long)out_stride);
    if (n_steps > NC_MAX_STEPS || (n_steps && !chain))
        return refuse(kBadArgument, "an epilogue holds at most %u steps", NC_MAX_STEPS);
    if ((uintptr_t)x_dev % 4 || (uintptr_t)out_dev % 4) return refuse(kBadArgument, "f32 rows start on a 4-byte boundary");
    if (ctx->device < 0 || ctx->device >= kStaticDevices) return refuse(kBadState, "device %d is outside the table of scratch addresses", ctx->device);
    cudaStream_t stream = (cudaStream_t)stream_;

    // one-time set-up per device (the first call on a device; make it before any stream capture)
    if ((rc = static_setup(ctx->device))) return rc;
    StaticScratch &fixed = g_static[ctx->device];
    unsigned char *base = fixed.base;

    // carve: [status 256][counters][digit scales][digit planes][partial sums ...]
    const uint32_t ncols = rows * 3;
    const uint64_t kpad = ((uint64_t)w->k + 255) / 256 * 256;
    const uint64_t cs_bytes = (uint64_t)(kStaticMaxK / 32) * kStaticMaxRows * 3 * sizeof(float);
    const uint64_t dig_bytes = (uint64_t)kStaticMaxK * kStaticMaxRows * 3;
    const uint64_t sums_bytes = (uint64_t)(kStaticMaxK / 256) * kStaticMaxRows * 3 * 64;
    unsigned int *status = (unsigned int *)base;
    unsigned int *counters = (unsigned int *)(base + 256);
    float *cs = (float *)(base + 256 + kStaticCountersBytes);
    uint8_t *dig = base + 256 + kStaticCountersBytes + cs_bytes;
    uint32_t *sums = (uint32_t *)(base + 256 + kStaticCountersBytes + cs_bytes + dig_bytes);
    float *partial = (float *)(base + 256 + kStaticCountersBytes + cs_bytes + dig_bytes + sums_bytes);
    const uint64_t partial_room = kStaticScratchBytes - (256 + kStaticCountersBytes + cs_bytes + dig_bytes + sums_bytes);

    const bool q4k = w->element == NC_ELEMENT_Q4K;
    const int nt = (int)((ncols + 7) / 8);  // 1 or 2 for up to four rows
    const int variant = (q4k ? 2 : 0) + (nt - 1);
    void (*kernel)(GemvParams) = static_variant(variant);
    const size_t smem = static_variant_smem(variant);
    const GemvPlan plan = plan_gemv(ctx, w->element, w->n, w->k, fixed.resident[variant]);
    const uint64_t partial_need = (uint64_t)plan.ntiles * plan.maxp * rows * kTileRows * sizeof(float);
    if (partial_need > partial_room)
        return refuse(kBadArgument, "this product splits into %llu bytes of partial sums and the static scratch holds %llu",
                      (unsigned long long)partial_need, (unsigned long long)partial_room);

    // The array keeps what the last call left.  Nothing has to be cleared here: the array loads as zeros, the warp
    // that finishes a split tile puts the tile's counter back to zero, and the status word stays raised until
    // neura_cuda_sync has reported it (which then clears the counters a product that gave up may have left).
    PrepParams prep;
    prep.x = x_dev;
    prep.x_stride = x_stride;
    prep.dig = (int8_t *)dig;
    prep.cs = cs;
    prep.sums = sums;
    prep.rows = rows;
    prep.k = w->k;
    prep.ncols = ncols;
    prep.granule = q4k ? 256 : 32;
    prep.vector = ((uintptr_t)x_dev % 16 == 0 && x_stride % 4 == 0) ? 1u : 0u;
    prep.lo = 0;
    prep.hi = w->k;
    const uint64_t prep_warps = (uint64_t)rows * (kpad / 256);
    prep_kernel<<<(unsigned int)((prep_warps + 3) / 4), 128, 0, stream>>>(prep);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());

    GemvParams p;
    memset(&p, 0, sizeof p);
    p.w = (const uint8_t *)w->data_dev;
    p.dig = dig;
    p.cs = cs;
    p.sums = (const uint8_t *)sums;
    p.out = out_dev;
    p.partial = partial;
    p.counters = counters;
    p.status = status;
    p.out_stride = out_stride;
    p.n = w->n;
    p.rows = rows;
    p.ncols = ncols;
    p.col_stride = ncols;
    p.col0 = 0;
    p.upt = plan.upt;
    p.nwarps = plan.nwarps;
    p.q = plan.q;
    p.r = plan.r;
    p.maxp = plan.maxp;
    p.chain.n = n_steps;
    for (uint32_t s = 0; s < n_steps; ++s) p.chain.step[s] = chain[s];
    kernel<<<plan.blocks, kGemvWarps * 32, smem, stream>>>(p);
    ctx->launches++;
    NC_CUDA(cudaGetLastError());
    return 0;
}

uint64_t neura_cuda_launches(const nc_context *ctx) { return ctx ? ctx->launches : 0; }

int32_t neura_cuda_capture_begin(nc_context *ctx, void *stream) {
    if (!ctx) return refuse(kBadArgument, "capture needs a context");
    if (ctx->capturing) return refuse(kBadState, "this context is already recording a program");
    if (!stream) return refuse(kBadArgument, "a program is recorded on a stream of its own, not the default stream");
    NC_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->capture_stream = (cudaStream_t)stream;
    ctx->capture_mark = ctx->launches;
    return 0;
}

int32_t neura_cuda_capture_end(nc_context *ctx, void *stream, nc_program **out) {
    if (!ctx || !out) return refuse(kBadArgument, "capture needs a context and somewhere to put the program");
    if (!ctx->capturing) return refuse(kBadState, "no program is being recorded");
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    NC_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &graph));
    nc_program *program = new (std::nothrow) nc_program();
    if (!program) return refuse(kBadState, "out of host memory");
    program->graph = graph;
    program->launches = ctx->launches - ctx->capture_mark;
    ctx->launches = ctx->capture_mark;  // recording launched nothing
    cudaError_t e = cudaGraphInstantiate(&program->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete program;
        return cuda_refuse(e, "cudaGraphInstantiate");
    }
    *out = program;
    return 0;
}

int32_t neura_cuda_program_run(nc_context *ctx, void *stream, nc_program *program) {
    if (!ctx || !program || !program->exec) return refuse(kBadArgument, "run needs a context and a recorded program");
    NC_CUDA(cudaGraphLaunch(program->exec, (cudaStream_t)stream));
    ctx->launches += program->launches;
    return 0;
}

int32_t neura_cuda_stream_create(nc_context *ctx, void **out_stream) {
    if (!ctx || !out_stream) return refuse(kBadArgument, "stream_create needs a context and somewhere to put the stream");
    cudaStream_t stream;
    NC_CUDA(cudaSetDevice(ctx->device));
    NC_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    *out_stream = (void *)stream;
    return 0;
}

int32_t neura_cuda_stream_destroy(nc_context *ctx, void *stream) {
    if (!ctx) return refuse(kBadArgument, "stream_destroy needs a context");
    if (stream) NC_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    return 0;
}

int32_t neura_cuda_program_free(nc_context *ctx, nc_program *program) {
    (void)ctx;
    if (!program) return 0;
    if (program->exec) cudaGraphExecDestroy(program->exec);
    if (program->graph) cudaGraphDestroy(program->graph);
    delete program;
    return 0;
}


// ---- a decode step as one persistent kernel (megakernel.cuh) -----------------------------------------------
}  // extern "C"

struct nc_decoder {
    int device = 0;
    MkParams params = {};
    bool q4k = false;
    unsigned int grid = 0;
    std::vector<void *> owned;   // device blocks freed with the decoder
    std::vector<uint32_t> kinds; // the phase table's kinds, for the trace
};

namespace {

int32_t decoder_alloc(nc_decoder *d, uint64_t bytes, bool zero, void **out) {
    void *ptr = nullptr;
    NC_CUDA(cudaMalloc(&ptr, bytes ? bytes : 1));
    d->owned.push_back(ptr);
    if (zero) NC_CUDA(cudaMemset(ptr, 0, bytes ? bytes : 1));
    *out = ptr;
    return 0;
}

// The (q, r) split of a product over all the warps of the persistent grid.
void plan_phase(GemvParams &g, uint32_t element, uint32_t plan_n, uint32_t k, uint64_t warps) {
    const uint32_t ntiles = (plan_n + kTileRows - 1) / kTileRows;
    g.upt = k / block_elements(element);
    const uint64_t units = (uint64_t)ntiles * g.upt;
    const uint64_t least = element == NC_ELEMENT_Q4K ? 1 : 4;
    if (warps > units / least) warps = units / least;
    if (warps < 1) warps = 1;
    g.nwarps = (uint32_t)warps;
    g.q = (uint32_t)(units / warps);
    g.r = (uint32_t)(units % warps);
    g.maxp = (g.upt + g.q - 1) / g.q + 1;
}

}  // namespace

extern "C" {

int32_t neura_cuda_decoder_free(nc_context *ctx, nc_decoder *decoder) {
    (void)ctx;
    if (!decoder) return 0;
    cudaSetDevice(decoder->device);
    for (void *ptr : decoder->owned) cudaFree(ptr);
    delete decoder;
    return 0;
}

int32_t neura_cuda_decoder_compile(nc_context *ctx, const nc_decoder_desc *desc, nc_decoder **out) {
    return neura_cuda_decoder_compile_rank(ctx, desc, nullptr, 1, 0, out);
}

int32_t neura_cuda_decoder_compile_rank(nc_context *ctx, const nc_decoder_desc *desc, nc_comm *comm, uint32_t world, uint32_t rank,
                                        nc_decoder **out) {
    if (!ctx || !desc || !out) return refuse(kBadArgument, "compile needs a context, a description and somewhere to put the decoder");
    *out = nullptr;
    const nc_decoder_desc &c = *desc;
    if (world < 1 || world > kMaxRanks || rank >= world) return refuse(kBadArgument, "rank %u of %u ranks", rank, world);
    if ((world > 1) != (comm != nullptr)) return refuse(kBadArgument, "a rank of a group compiles with the group's communicator, a single device without one");
    if (comm && (!comm->connected || comm->world != world || comm->rank != rank))
        return refuse(kBadState, "the communicator is not connected as rank %u of %u", rank, world);
    if (!c.layers || !c.layer || !c.tokens_dev || !c.position_dev || !c.logits_dev || !c.output_norm_dev)
        return refuse(kBadArgument, "a decoder needs its layers, token ids, cursors, logits and output norm");
    if (c.batch < 1 || c.batch > 2)
        return refuse(kBadArgument, "the persistent step carries 1 or 2 sequences, not %u", c.batch);
    if (!c.heads || !c.key_heads || c.heads % c.key_heads || c.heads / c.key_heads > kAttendMaxGroup)
        return refuse(kBadArgument, "%u query heads do not share %u key heads", c.heads, c.key_heads);
    if (c.head_width != 64 && c.head_width != 128)
        return refuse(kBadArgument, "the attention phase is built for heads of width 64 and 128, not %u", c.head_width);
    if (!c.capacity || c.capacity > kMkTile * kAttendMaxChunk)
        return refuse(kBadArgument, "a cache of %u slots is more than the %u the attention phase splits", c.capacity,
                      kMkTile * kAttendMaxChunk);
    const uint32_t element = c.head.element;
    const uint32_t per = block_elements(element);
    if (!per) return refuse(kBadArgument, "element %u is not a block format this path multiplies", element);
    const uint32_t query_width = c.heads * c.head_width, key_width = c.key_heads * c.head_width;
    const uint32_t ncols = c.batch * 3;
    const bool q4k = element == NC_ELEMENT_Q4K;
    if (c.hidden % per || c.hidden % 8)
        return refuse(kBadArgument, "a hidden width of %u is not whole blocks of %u", c.hidden, per);
    auto fits = [&](const nc_weight &w, uint32_t n, uint32_t k, uint32_t layout, const char *name) -> int32_t {
        int32_t rc = check_weight(&w);
        if (rc) return rc;
        if (w.element != element || w.layout != layout || w.n != n || w.k != k)
            return refuse(kBadArgument, "%s is [%u, %u] of element %u in layout %u where the decoder wants [%u, %u] of element %u in layout %u",
                          name, w.n, w.k, w.element, w.layout, n, k, element, layout);
        return 0;
    };
    int32_t rc;
    // a rank's share of a row-parallel projection's K axis: the whole blocks that cover elements
    // [rank, rank + 1) * width of the group's axis, the share itself at [lo, hi) inside them
    struct Window { uint32_t k, lo, hi; };
    auto window_of = [&](uint32_t width) {
        const uint32_t k0 = rank * width, k1 = k0 + width, b0 = k0 / per, b1 = (k1 + per - 1) / per;
        return Window{(b1 - b0) * per, k0 - b0 * per, k1 - b0 * per};
    };
    const Window attended_at = window_of(query_width), held_at = window_of(c.feed_forward);
    if (world > 1 && (query_width % 32 || c.feed_forward % 32 || c.hidden % 256 || (uint64_t)c.batch * c.hidden > comm->max_count))
        return refuse(kBadArgument, "a rank's shares of %u and %u columns start on multiples of 32, and the exchange takes rows of a multiple of 256 numbers, %llu in all",
                      query_width, c.feed_forward, (unsigned long long)comm->max_count);
    if ((rc = fits(c.head, c.vocab, c.hidden, NC_LAYOUT_TILED, "the head"))) return rc;
    if ((rc = check_weight(&c.embedding))) return rc;
    if (c.embedding.n != c.vocab * world || c.embedding.k != c.hidden)
        return refuse(kBadArgument, "the embedding is [%u, %u] where the decoder wants [%u, %u]", c.embedding.n, c.embedding.k, c.vocab * world, c.hidden);
    for (uint32_t l = 0; l < c.layers; ++l) {
        const nc_decoder_layer &layer = c.layer[l];
        if ((rc = fits(layer.qkv, query_width + 2 * key_width, c.hidden, NC_LAYOUT_TILED, "a q|k|v projection"))) return rc;
        if ((rc = fits(layer.attn_output, c.hidden, attended_at.k, NC_LAYOUT_TILED, "an attention output projection"))) return rc;
        if ((rc = fits(layer.gate_up, c.feed_forward, c.hidden, NC_LAYOUT_TILED_PAIR, "a gate|up pair"))) return rc;
        if ((rc = fits(layer.down, c.hidden, held_at.k, NC_LAYOUT_TILED, "a down projection"))) return rc;
        if (!layer.attn_norm_dev || !layer.ffn_norm_dev || !layer.keys_dev || !layer.values_dev)
            return refuse(kBadArgument, "layer %u lacks a norm weight or its cache", l);
    }
    NC_CUDA(cudaSetDevice(ctx->device));
    if ((rc = ensure(ctx, ctx->status, 256, true))) return rc;
    nc_decoder *d = new (std::nothrow) nc_decoder();
    if (!d) return refuse(kBadState, "out of host memory");
    d->device = ctx->device;
    d->q4k = q4k;
    d->grid = (unsigned int)ctx->sms;
    const uint64_t warps = (uint64_t)ctx->sms * kMkWarps;
    auto fail = [&](int32_t code) { neura_cuda_decoder_free(ctx, d); return code; };

    // activations and scratch
    float *hidden, *qkv, *attended, *held, *partial, *attend_partial, *slice_value, *sumsq;
    uint32_t *slice_index;
    unsigned int *counters, *attend_counters, *argmax_counters, *barrier;
    const uint32_t qkv_width = query_width + 2 * key_width;
    const uint32_t max_splits = (c.capacity + kMkTile - 1) / kMkTile;
    const uint32_t widest = std::max(std::max(c.vocab, 2 * ((c.feed_forward + 15) / 16 * 16)), std::max(c.hidden, qkv_width));
    const uint32_t ntiles_max = (widest + kTileRows - 1) / kTileRows + 1;
#define NC_TRY(call) do { int32_t rc_ = (call); if (rc_) return fail(rc_); } while (0)
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * c.hidden * 4, true, (void **)&hidden));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * qkv_width * 4, true, (void **)&qkv));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * query_width * 4, true, (void **)&attended));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * c.feed_forward * 4, true, (void **)&held));
    NC_TRY(decoder_alloc(d, (uint64_t)ntiles_max * sizeof(unsigned int), true, (void **)&counters));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * c.heads * max_splits * (c.head_width + 2) * 4, true, (void **)&attend_partial));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * c.key_heads * sizeof(unsigned int), true, (void **)&attend_counters));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * d->grid * 4, true, (void **)&slice_value));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * d->grid * 4, true, (void **)&slice_index));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * sizeof(unsigned int), true, (void **)&argmax_counters));
    float *best_value;
    uint32_t *best_index;
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * 4, true, (void **)&best_value));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * 4, true, (void **)&best_index));
    NC_TRY(decoder_alloc(d, 256, true, (void **)&barrier));
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * ((c.hidden + 255) / 256) * 4, true, (void **)&sumsq));
    float2 *rope_table;
    NC_TRY(decoder_alloc(d, (uint64_t)c.batch * (c.head_width / 2) * sizeof(float2), true, (void **)&rope_table));
    unsigned long long *trace;

    // the staged form of each kind of activation row: what the products read (prep.cuh)
    struct Staged {
        int8_t *dig;
        float *cs;
        uint32_t *sums;
        unsigned int *counters;
        float *rows;
        uint32_t width;          // the K axis of the product that reads the staged rows
        uint32_t stride, lo, hi; // the rows themselves: their stride, and where they sit on that axis
    };
    auto staged = [&](float *rows, uint32_t stride, const Window &at, Staged &out) -> int32_t {
        const uint32_t width = at.k;
        out.stride = stride;
        out.lo = at.lo;
        out.hi = at.hi;
        const uint64_t kpad = ((uint64_t)width + 255) / 256 * 256;
        int32_t rc_;
        if ((rc_ = decoder_alloc(d, kpad * ncols, true, (void **)&out.dig))) return rc_;
        if ((rc_ = decoder_alloc(d, kpad / 32 * ncols * 4, true, (void **)&out.cs))) return rc_;
        if ((rc_ = decoder_alloc(d, kpad / 256 * ncols * 64, true, (void **)&out.sums))) return rc_;
        if ((rc_ = decoder_alloc(d, (uint64_t)c.batch * (kpad / 256) * sizeof(unsigned int), true, (void **)&out.counters))) return rc_;
        out.rows = rows;
        out.width = width;
        return 0;
    };
    Staged of_hidden, of_attended, of_held;
    NC_TRY(staged(hidden, c.hidden, Window{c.hidden, 0, c.hidden}, of_hidden));
    NC_TRY(staged(attended, query_width, attended_at, of_attended));
    NC_TRY(staged(held, c.feed_forward, held_at, of_held));

    // the phase table
    std::vector<MkPhase> phases;
    uint64_t partial_cells = 0;
    auto blank = [](uint32_t kind) {
        MkPhase ph;
        memset(&ph, 0, sizeof ph);
        ph.kind = kind;
        ph.prefetch = kMkNone;
        return ph;
    };
    // how the rows a phase writes become the operand of the next product
    auto stage_after = [&](MkPhase &ph, const Staged &to, uint32_t piece, const float *gain, bool squares) {
        ph.has_after = 1;
        StageAfter &a = ph.after;
        a.prep.x = to.rows;
        a.prep.x_stride = to.stride;
        a.prep.dig = to.dig;
        a.prep.cs = to.cs;
        a.prep.sums = to.sums;
        a.prep.rows = c.batch;
        a.prep.k = to.width;
        a.prep.ncols = ncols;
        a.prep.granule = q4k ? 256 : 32;
        a.prep.vector = 1;
        a.prep.lo = to.lo;
        a.prep.hi = to.hi;
        a.gain = gain;
        a.sumsq = squares ? sumsq : nullptr;
        a.counters = to.counters;
        a.piece = piece;
        // the hidden rows a rank's row-parallel products write are partial sums: whoever completes a chunk adds the ranks' up
        a.exchange = comm && ph.kind == MK_GEMV && to.rows == hidden ? comm->view_dev : nullptr;
        a.wait_nanos = ctx->wait_nanos;
        a.status = (unsigned int *)ctx->status.ptr;
        if (ph.kind == MK_GEMV) {
            ph.g.then = a;
            ph.g.has_then = 1;
        }
    };
    auto product = [&](const nc_weight &w, const Staged &from, bool normed, float *out_rows, uint64_t out_stride,
                       const float *residual) -> MkPhase & {
        MkPhase ph = blank(MK_GEMV);
        ph.k = w.k;
        GemvParams &g = ph.g;
        const bool pair = w.layout == NC_LAYOUT_TILED_PAIR;
        const uint32_t plan_n = pair ? (w.n + 15) / 16 * 32 : w.n;
        g.w = (const uint8_t *)w.data_dev;
        g.dig = (const uint8_t *)from.dig;
        g.cs = from.cs;
        g.sums = (const uint8_t *)from.sums;
        g.out = out_rows;
        g.out_stride = out_stride;
        g.counters = counters;
        g.status = (unsigned int *)ctx->status.ptr;
        g.n = w.n;
        g.rows = c.batch;
        g.ncols = ncols;
        g.col_stride = ncols;
        g.col0 = 0;
        g.pair = pair ? 1u : 0u;
        if (normed) {
            g.sumsq = sumsq;
            g.sumsq_chunks = (from.width + 255) / 256;
            g.floor = c.floor;
            g.inv_k = 1.0f / (float)from.width;
        }
        if (residual) {
            g.chain.n = 1;
            g.chain.step[0].op = NC_OP_ADD;
            g.chain.step[0].swapped = 0;
            g.chain.step[0].operand_dev = residual;
            g.chain.step[0].row_stride = (int64_t)out_stride;
            g.chain.step[0].col_stride = 1;
        }
        plan_phase(g, element, plan_n, w.k, warps);
        const uint64_t ntiles = (plan_n + kTileRows - 1) / kTileRows;
        partial_cells = std::max(partial_cells, ntiles * g.maxp * c.batch * kTileRows);
        phases.push_back(ph);
        return phases.back();
    };
    {
        MkPhase ph = blank(MK_EMBED);
        ph.table = WeightView{(const uint8_t *)c.embedding.data_dev, c.embedding.element, c.embedding.layout, c.embedding.n, c.embedding.k};
        ph.out = hidden;
        ph.out_stride = c.hidden;
        phases.push_back(ph);
        MkPhase first = blank(MK_STAGE);
        stage_after(first, of_hidden, 256, c.layer[0].attn_norm_dev, true);
        phases.push_back(first);
    }
    for (uint32_t l = 0; l < c.layers; ++l) {
        const nc_decoder_layer &layer = c.layer[l];
        const float *next_norm = l + 1 < c.layers ? c.layer[l + 1].attn_norm_dev : c.output_norm_dev;
        product(layer.qkv, of_hidden, true, qkv, qkv_width, nullptr);
        {
            MkPhase ph = blank(MK_ATTEND);
            ph.keys = layer.keys_dev;
            ph.values = layer.values_dev;
            stage_after(ph, of_attended, 256, nullptr, false);
            phases.push_back(ph);
        }
        const float *residual = rank == 0 ? hidden : nullptr;   // rank 0 carries the residual into the ranks' sum
        stage_after(product(layer.attn_output, of_attended, false, hidden, c.hidden, residual), of_hidden, 32, layer.ffn_norm_dev, true);
        stage_after(product(layer.gate_up, of_hidden, true, held, c.feed_forward, nullptr), of_held, 16, nullptr, false);
        stage_after(product(layer.down, of_held, false, hidden, c.hidden, residual), of_hidden, 32, next_norm, true);
    }
    product(c.head, of_hidden, true, c.logits_dev, c.vocab, nullptr);
    {
        MkPhase ph = blank(MK_ARGMAX);
        ph.x = c.logits_dev;
        ph.x_stride = c.vocab;
        ph.k = c.vocab;
        phases.push_back(ph);
        if (comm) {   // the ranks hold shares of the vocabulary: one more phase picks among their winners
            MkPhase choose = blank(MK_CHOOSE);
            choose.k = c.vocab;
            choose.after.exchange = comm->view_dev;
            choose.after.wait_nanos = ctx->wait_nanos;
            choose.after.status = (unsigned int *)ctx->status.ptr;
            phases.back().flags = 1;   // the argmax phase leaves its winners for the next phase
            phases.push_back(choose);
        }
    }
    // when a phase ends, its warps start the copies of the next product, unless the attention phase
    // (which borrows the ring) comes first
    for (size_t i = 0; i < phases.size(); ++i) {
        for (size_t j = i + 1; j < phases.size(); ++j) {
            if (phases[j].kind == MK_ATTEND) break;
            if (phases[j].kind == MK_GEMV) { phases[i].prefetch = (uint32_t)j; break; }
        }
    }
    NC_TRY(decoder_alloc(d, partial_cells * sizeof(float), false, (void **)&partial));
    for (MkPhase &ph : phases)
        if (ph.kind == MK_GEMV) ph.g.partial = partial;
    MkPhase *table = nullptr;
    NC_TRY(decoder_alloc(d, (phases.size() + 1) * sizeof(unsigned long long), true, (void **)&trace));
    for (const MkPhase &ph : phases) d->kinds.push_back(ph.kind);
    NC_TRY(decoder_alloc(d, phases.size() * sizeof(MkPhase), false, (void **)&table));
    cudaError_t e = cudaMemcpy(table, phases.data(), phases.size() * sizeof(MkPhase), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(cuda_refuse(e, "cudaMemcpy of the phase table"));
#undef NC_TRY

    MkParams &p = d->params;
    p.phases = table;
    p.nphases = (uint32_t)phases.size();
    p.barrier = barrier;
    p.status = (unsigned int *)ctx->status.ptr;
    p.tokens = c.tokens_dev;
    p.position = c.position_dev;
    p.rows = c.batch;
    p.granule = q4k ? 256 : 32;
    p.qkv = qkv;
    p.qkv_stride = qkv_width;
    p.attended = attended;
    p.attended_stride = query_width;
    p.attend_partial = attend_partial;
    p.attend_counters = attend_counters;
    p.heads = c.heads;
    p.key_heads = c.key_heads;
    p.width = c.head_width;
    p.capacity = c.capacity;
    p.max_splits = max_splits;
    p.scale = c.scale;
    p.rope_base = c.rope_base;
    p.floor = c.floor;
    p.rope_table = rope_table;
    p.slice_value = slice_value;
    p.slice_index = slice_index;
    p.argmax_counters = argmax_counters;
    p.best_value = best_value;
    p.best_index = best_index;
    p.trace = trace;

    // the kernel must be resident on every SM at once
    const void *kernel = q4k ? (const void *)decode_megakernel<true> : (const void *)decode_megakernel<false>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMkSmem);
    if (e != cudaSuccess) return fail(cuda_refuse(e, "cudaFuncSetAttribute"));
    int resident = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kMkThreads, kMkSmem);
    if (e != cudaSuccess) return fail(cuda_refuse(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor"));
    if (resident < 1) return fail(refuse(kBadState, "the persistent step does not fit an SM"));
    *out = d;
    return 0;
}

int32_t neura_cuda_decoder_trace(nc_context *ctx, nc_decoder *decoder, uint32_t capacity, uint32_t *kinds_out,
                                 uint64_t *nanos_out, uint32_t *phases_out) {
    if (!ctx || !decoder || !phases_out) return refuse(kBadArgument, "a trace needs a context, a decoder and somewhere to put the count");
    const uint32_t phases = (uint32_t)decoder->kinds.size();
    *phases_out = phases;
    if (!kinds_out || !nanos_out || capacity < phases) return 0;   // the caller asked for the count
    std::vector<unsigned long long> stamps(phases + 1);
    NC_CUDA(cudaMemcpy(stamps.data(), decoder->params.trace, stamps.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    for (uint32_t i = 0; i < phases; ++i) {
        kinds_out[i] = decoder->kinds[i];
        nanos_out[i] = stamps[i + 1] >= stamps[i] ? stamps[i + 1] - stamps[i] : 0;
    }
    return 0;
}

int32_t neura_cuda_decoder_step(nc_context *ctx, void *stream_, nc_decoder *decoder) {
    if (!ctx || !decoder) return refuse(kBadArgument, "a step needs a context and a compiled decoder");
    cudaStream_t stream = (cudaStream_t)stream_;
    NC_CUDA(cudaMemsetAsync(decoder->params.barrier, 0, 256, stream));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(decoder->grid);
    config.blockDim = dim3(kMkThreads);
    config.dynamicSmemBytes = kMkSmem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (decoder->q4k) NC_CUDA(cudaLaunchKernelEx(&config, decode_megakernel<true>, decoder->params));
    else NC_CUDA(cudaLaunchKernelEx(&config, decode_megakernel<false>, decoder->params));
    ctx->launches++;
    return 0;
}

}  // extern "C"
