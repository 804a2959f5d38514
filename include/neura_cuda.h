/*
 * libneura_cuda — C ABI of the B200 (sm_100a) quantized-linear path for Neura.
 *
 * The reference (formetaohy/Neura) has no FFI boundary of its own: its operator
 * API for this path is `Graph::matmul` over a block-quantised parameter
 * (crates/neura-graph/src/op.rs:17), executed by `Runtime::{open, load, write,
 * run, read}` (crates/neura-runtime/src/runtime.rs:183,356,1020,833,1064) on a
 * device heap that holds GGUF blocks verbatim (crates/neura-runtime/src/store.rs:77-157).
 * Each entry point below names the reference item it stands in for; a thin Rust
 * crate binds them one to one.
 *
 * Conventions
 *  - every call returns int32_t: 0 = ok, negative = host-side refusal (the
 *    sentence is in neura_cuda_last_error(), thread-local), positive = CUDA error code;
 *  - pointers named *_dev are device pointers of the context's GPU, *_host are host pointers;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *  - a context is used by one host thread at a time and its calls share one
 *    scratch area: work submitted through one context must be stream-ordered;
 *  - the library never falls back to the CPU.
 */
#ifndef NEURA_CUDA_H
#define NEURA_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element codes: discriminants of neura_abi::Element (crates/neura-abi/src/element.rs:3-17). */
#define NC_ELEMENT_SINGLE 0u
#define NC_ELEMENT_BFLOAT16 2u
#define NC_ELEMENT_Q8_0 8u
#define NC_ELEMENT_Q4K 9u
#define NC_ELEMENT_Q6K 11u /* heads and embeddings of common GGUF mixes: multiplied where the GGUF left it (NC_LAYOUT_GGUF) */
/* The other weight formats a GGUF of this model family may hold (element.rs:3-17), all multiplied in GGUF order by
 * the plain row-at-a-time product: */
#define NC_ELEMENT_HALF 1u   /* IEEE half numbers, two to a word (as a weight; NC_ELEMENT_BFLOAT16 likewise) */
#define NC_ELEMENT_Q5K 10u   /* 256 numbers in 176 bytes */
#define NC_ELEMENT_Q3K 12u   /* 256 numbers in 110 bytes */

/* How the blocks of a weight tensor are laid out in device memory. */
#define NC_LAYOUT_GGUF 0u   /* verbatim GGUF: row after row, blocks in order (what store.rs:131-135 copies) */
#define NC_LAYOUT_TILED 1u  /* neura_cuda_weight_seal output: same bytes, permuted per 32-row tile for the MMA kernels */
#define NC_LAYOUT_TILED_PAIR 2u /* neura_cuda_weight_seal_pair output: two [n, k] tensors, 16 rows of each per tile */

/* Pointwise op codes of the fused epilogue: neura-pointwise declaration order
 * (crates/neura-pointwise/src/op.rs:141-170). */
#define NC_OP_ADD 0u
#define NC_OP_MUL 1u
#define NC_OP_SUB 2u
#define NC_OP_DIV 3u
#define NC_OP_MAXIMUM 4u
#define NC_OP_MINIMUM 5u
#define NC_OP_RELU 6u
#define NC_OP_SQRT 7u
#define NC_OP_RECIP 8u
#define NC_OP_EXP 9u
#define NC_OP_LOG 10u
#define NC_OP_TANH 11u
#define NC_OP_SIGMOID 12u
#define NC_OP_NEG 13u
#define NC_OP_ABS 14u
#define NC_OP_IDENTITY 15u
#define NC_OP_SIN 16u
#define NC_OP_COS 17u
#define NC_OP_POW 18u
#define NC_OP_FLOOR 19u
#define NC_OP_GELU 20u
#define NC_OP_SILU 21u

#define NC_MAX_STEPS 4u

typedef struct nc_context nc_context;

/* A weight matrix on the device: the subset of ValueRecord{base, element, dims, strides}
 * (crates/neura-abi/src/record.rs:151-165) a linear layer needs.  `n` output
 * features (GGUF ne[1]), `k` input features (GGUF ne[0], contiguous inside a row). */
typedef struct nc_weight {
    const void *data_dev;
    uint32_t element; /* NC_ELEMENT_Q8_0 | NC_ELEMENT_Q4K, or one of the formats kept in GGUF order: Q6K, Q5K, Q3K, HALF, BFLOAT16 */
    uint32_t layout;  /* NC_LAYOUT_* */
    uint32_t n;
    uint32_t k;
} nc_weight;

/* One step of the fused epilogue: StepRecord{op, operand, swapped}
 * (crates/neura-abi/src/record.rs:72-76), applied like `chained`
 * (crates/neura-kernel/src/pointwise.rs:90-104).  The operand is read at the
 * output coordinate through broadcast strides (in elements; 0 broadcasts). */
typedef struct nc_step {
    uint32_t op;
    uint32_t swapped;         /* 1: the operand is the op's first argument */
    const float *operand_dev; /* NULL for a unary op */
    int64_t row_stride;
    int64_t col_stride;
} nc_step;

/* Thread-local sentence for the last negative return (the reference panics with
 * a sentence on host contract violations, e.g. store.rs:90-123). */
const char *neura_cuda_last_error(void);

/* Runtime::open (runtime.rs:183): binds the calling thread's work to one GPU and
 * allocates the context's scratch (activation staging, split-tile partials). */
int32_t neura_cuda_open(int32_t device, nc_context **out);
int32_t neura_cuda_close(nc_context *ctx);

/* Element::payload_bytes (element.rs:231-241); 0 for an element the path does not hold. */
uint64_t neura_cuda_payload_bytes(uint32_t element, uint64_t elements);
/* Bytes neura_cuda_weight_seal writes for an [n, k] matrix (rows padded to 16). */
uint64_t neura_cuda_sealed_bytes(uint32_t element, uint32_t n, uint32_t k);

/* Device memory and copies: GpuBuffer / Runtime::write / Runtime::read
 * (crates/neura-gpu/src/buffer.rs:30-177, runtime.rs:1020,1064).  The copies are
 * asynchronous on `stream`; neura_cuda_sync completes them (Run::complete, runtime.rs:123). */
int32_t neura_cuda_alloc(nc_context *ctx, uint64_t bytes, void **out_dev);
int32_t neura_cuda_free(nc_context *ctx, void *ptr_dev);
int32_t neura_cuda_host_alloc(nc_context *ctx, uint64_t bytes, void **out_host); /* pinned */
int32_t neura_cuda_host_free(nc_context *ctx, void *ptr_host);
int32_t neura_cuda_write(nc_context *ctx, void *stream, void *dst_dev, const void *src_host, uint64_t bytes);
int32_t neura_cuda_read(nc_context *ctx, void *stream, void *dst_host, const void *src_dev, uint64_t bytes);
int32_t neura_cuda_sync(nc_context *ctx, void *stream);

/* Free and total bytes of the context's GPU (what a host sizes its heap request from, MemoryRequest,
 * runtime.rs:150-167). */
int32_t neura_cuda_memory(nc_context *ctx, uint64_t *free_out, uint64_t *total_out);

/* How long a kernel of this context waits for another party before it gives up: a peer's flag in an
 * all-reduce, the other CTAs at the grid barrier of the persistent step (the reference's hang deadline,
 * FRAME_TIMEOUT, crates/neura-gpu/src/native.rs:20-35).  Default two seconds.  A kernel that gives up
 * raises the context's status word and returns; the next neura_cuda_sync reports it as a refusal and
 * clears it, and the context stays usable.  (Waits for a kernel's own asynchronous copies keep a fixed
 * two-second limit.) */
int32_t neura_cuda_set_wait_limit(nc_context *ctx, uint64_t nanoseconds);

/* Grows the context's scratch ahead of time so that later linear calls of up to
 * `rows` activation rows against matrices of up to [n, k] never allocate. */
int32_t neura_cuda_reserve(nc_context *ctx, uint32_t rows, uint32_t n, uint32_t k);

/* The same for neura_cuda_linear_bf16: the bf16 copy of up to `rows` rows of `k` activations and the scratch its
 * split products share, so that a program recorded around such products never sees them move. */
int32_t neura_cuda_reserve_bf16(nc_context *ctx, uint32_t rows, uint32_t k);

/* The same for the decoder's other scratch: the partial results of an attention over a cache of
 * `capacity` rows and the candidates of an argmax over `rows` rows, so that a decode step can be
 * recorded without having run eagerly first.  (The reference sizes these at plan time,
 * crates/neura-plan/src/layout.rs:22-55.) */
int32_t neura_cuda_reserve_decoder(nc_context *ctx, uint32_t rows, uint32_t heads, uint32_t key_heads, uint32_t width,
                                   uint32_t capacity);

/* The load step after pour_one (store.rs:77-157): permutes a verbatim GGUF tensor
 * into the tiled layout the MMA kernels stream.  Out of place; `dst_dev` holds
 * neura_cuda_sealed_bytes().  Dequantised values are unchanged bit for bit. */
int32_t neura_cuda_weight_seal(nc_context *ctx, void *stream, uint32_t element, uint32_t n, uint32_t k,
                               const void *gguf_dev, void *dst_dev);

/* The gate and up projections of an MLP sealed as one weight (examples/qwen/mlp.rs:31-33:
 * `mul(silu(matmul(x, gate)), matmul(x, up))`).  A product with the result (layout
 * NC_LAYOUT_TILED_PAIR, n = rows of each tensor) writes out[c] = chain(silu(gate_c . x) * (up_c . x)):
 * both tensors are streamed once by one kernel and the SwiGLU costs no pass of its own.
 * `dst_dev` holds neura_cuda_sealed_pair_bytes(). */
uint64_t neura_cuda_sealed_pair_bytes(uint32_t element, uint32_t n, uint32_t k);
int32_t neura_cuda_weight_seal_pair(nc_context *ctx, void *stream, uint32_t element, uint32_t n, uint32_t k,
                                    const void *gate_gguf_dev, const void *up_gguf_dev, void *dst_dev);

/* unpack (crates/neura-precision/src/ggml.rs:22-38, q8_0_values :211-216,
 * q4_k_values :336-350): out_dev[n*k] f32, bit-exact, for either layout. */
int32_t neura_cuda_dequant(nc_context *ctx, void *stream, const nc_weight *w, float *out_dev);

/* pack (ggml.rs:8-20, q8_0 :201-209, affine_block :149-199) on the device, the
 * counterpart of the reference's device packer (crates/neura-kernel/src/task/convert.rs:355-431):
 * `elements` f32 (a multiple of the block) -> GGUF blocks, bit-exact with the host packer. */
int32_t neura_cuda_quantize(nc_context *ctx, void *stream, uint32_t element, const float *src_dev,
                            uint64_t elements, void *dst_dev);

/* run_matmul + chained (crates/neura-kernel/src/task/matmul.rs:376-517, pointwise.rs:90-104):
 *   out[r*out_stride + c] = chain(sum_k W[c][k] * x[r*x_stride + k]),  r < rows, c < w->n
 * f32 activations, f32 accumulation, f32 output (promote(Single, Q*) = Single, element.rs:306-323).
 * A Q8_0 or Q4K weight is sealed (NC_LAYOUT_TILED, or a sealed pair); a Q6K, Q5K, Q3K, half or bfloat16 weight stays in
 * GGUF order.
 * The kernel follows the row count the way the reference's planner picks its tiles (Product::planned,
 * crates/neura-plan/src/product.rs:103-195): up to eight rows the streaming product (the reference's folded tiles),
 * from nine rows on a Q4K weight takes the skinny tensor-core product that streams the weight once for up to 32 rows
 * (its staged-run tiles), more rows go in passes.  The bf16 tensor path is neura_cuda_linear_bf16: the reference, too,
 * takes its cooperative-matrix tiles only when asked to measure them (product.rs:109-113, 191-195). */
int32_t neura_cuda_linear(nc_context *ctx, void *stream, const nc_weight *w, const float *x_dev, uint32_t rows,
                          uint64_t x_stride, float *out_dev, uint64_t out_stride, const nc_step *chain,
                          uint32_t n_steps);

/* The tensor path, template_run_matmul_cooperative (crates/neura-kernel/src/task/matmul.rs:1344-1565),
 * for prefill: many rows at once.  The f32 activations are rounded to bf16 (round to nearest even,
 * crates/neura-precision/src/lib.rs:325-329), the Q4K weight is dequantised exactly and rounded to
 * bf16 tile by tile in shared memory, products accumulate in f32 (tcgen05 MMAs into tensor memory):
 *   out[r*out_stride + c] = chain(sum_k bf16(W[c][k]) * bf16(x[r*x_stride + k]))
 * Needs a sealed Q4K weight; any number of rows.  A sealed gate|up pair (NC_LAYOUT_TILED_PAIR) gives
 *   out[r*out_stride + c] = chain(silu(gate_c . x_r) * (up_c . x_r))
 * as neura_cuda_linear does (the epilogue joins the halves; a product of few tiles splits K over CTAs and leaves
 * the joining, like the chain, to a second kernel over scratch of the context). */
int32_t neura_cuda_linear_bf16(nc_context *ctx, void *stream, const nc_weight *w, const float *x_dev, uint32_t rows,
                               uint64_t x_stride, float *out_dev, uint64_t out_stride, const nc_step *chain,
                               uint32_t n_steps);

/* The two halves of neura_cuda_linear, for callers that feed several weights with the
 * same activations (q/k/v, gate/up: examples/qwen/attention.rs:106-125, mlp.rs:31-32).
 * neura_cuda_stage rewrites up to 16 rows of f32 activations into the context's
 * staging area in the form the MMA kernels read (three int8 digit planes per row, an
 * exponent per block of the weight format `element`); neura_cuda_linear_staged runs
 * the product of the staged rows with `w`.  The staging is overwritten by the next
 * neura_cuda_stage or neura_cuda_linear on the context. */
int32_t neura_cuda_stage(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint64_t x_stride,
                         uint32_t k, uint32_t element);
/* neura_cuda_stage for a row-parallel shard (no counterpart in the reference, which runs on one
 * device): the rows hold elements [lo, hi) of the K axis of a weight of `k` columns and the rest of
 * K is staged as zero.  A rank of a tensor-parallel group keeps the whole super-blocks that cover
 * its K range and stages its activations at their offset inside them; lo and hi are multiples of 32. */
int32_t neura_cuda_stage_window(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint64_t x_stride,
                                uint32_t k, uint32_t element, uint32_t lo, uint32_t hi);
int32_t neura_cuda_linear_staged(nc_context *ctx, void *stream, const nc_weight *w, float *out_dev,
                                 uint64_t out_stride, const nc_step *chain, uint32_t n_steps);

/* ---- the steps either side of the products in a decoder layer (one new row per sequence) ---- */

/* rms_norm (crates/neura-decoder/src/op.rs:3-5 -> crates/neura-kernel/src/task/norm.rs:55-131):
 *   y = x / sqrt(mean(x^2) + floor) * weight
 * fused with neura_cuda_stage of y for weights of block format `element`, so that the products
 * that follow (q/k/v, gate/up, the head) take neura_cuda_linear_staged directly.  `weight_dev`
 * may be NULL; `normed_dev`, when not NULL, also receives y as f32. */
int32_t neura_cuda_rms_norm_stage(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint64_t x_stride,
                                  uint32_t k, const float *weight_dev, float floor, uint32_t element,
                                  float *normed_dev, uint64_t normed_stride);

/* rms_norm alone, for any number of rows (the rows of a wide prompt chunk on their way to neura_cuda_linear_bf16):
 *   out[r*out_stride + c] = x[r*x_stride + c] / sqrt(mean_c(x[r]^2) + floor) * weight[c]
 * `weight_dev` may be NULL; `out_dev` may be `x_dev`. */
int32_t neura_cuda_rms_norm(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint64_t x_stride,
                            uint32_t k, const float *weight_dev, float floor, float *out_dev, uint64_t out_stride);

/* rope over the full head width (crates/neura-decoder/src/rope.rs:3-12 -> crates/neura-kernel/src/task/rope.rs:48-122,
 * half rotation, angle = position * base^(-2c/width)) applied in place to the query and key parts of
 * fused q|k|v rows, then Cache::write (crates/neura-decoder/src/cache.rs:267-310): the turned key and
 * the value of sequence b go to slot position_dev[b] of keys/values [batch][key_heads][capacity][width]. */
int32_t neura_cuda_rope_cache(nc_context *ctx, void *stream, float *qkv_dev, uint64_t row_stride,
                              const uint32_t *position_dev, float base, uint32_t batch, uint32_t heads,
                              uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                              float *values_dev);

/* Cache::attend (crates/neura-decoder/src/cache.rs:311-406 -> crates/neura-kernel/src/task/attention.rs:309-617):
 * causal grouped-query attention of the new row of each sequence over slots 0..position_dev[b];
 * query head h reads key head h / (heads / key_heads); f32 throughout. */
int32_t neura_cuda_attend(nc_context *ctx, void *stream, const float *q_dev, uint64_t q_stride, const float *keys_dev,
                          const float *values_dev, const uint32_t *position_dev, float scale, uint32_t batch,
                          uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *out_dev,
                          uint64_t out_stride);

/* The same two steps for a chunk of a prompt (Batch::prefill and its fill programs,
 * crates/neura-generate/src/batch.rs:1595-1599, :298-325; examples/qwen/main.rs:21 fills in chunks of 32 and 8): the
 * `rows` rows are consecutive tokens of ONE sequence, row i at position_dev[i]; keys_dev / values_dev point at that
 * sequence's cache [key_heads][capacity][width].  neura_cuda_rope_cache_rows writes all the rows' keys and values;
 * neura_cuda_attend_rows then lets row i attend to slots 0..position_dev[i], the rows before it in the chunk included. */
int32_t neura_cuda_rope_cache_rows(nc_context *ctx, void *stream, float *qkv_dev, uint64_t row_stride,
                                   const uint32_t *position_dev, float base, uint32_t rows, uint32_t heads,
                                   uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                                   float *values_dev);
int32_t neura_cuda_attend_rows(nc_context *ctx, void *stream, const float *q_dev, uint64_t q_stride, const float *keys_dev,
                               const float *values_dev, const uint32_t *position_dev, float scale, uint32_t rows,
                               uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *out_dev,
                               uint64_t out_stride);

/* Sampling::Greedy -> graph.argmax (crates/neura-generate/src/sampling.rs:79-81,
 * crates/neura-kernel/src/task/choice.rs:46-52): the lowest index wins a tie. */
int32_t neura_cuda_argmax(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint32_t width,
                          uint64_t stride, uint32_t *out_dev);

/* The same over rows whose columns arrive in segments (the shares of a column-parallel head gathered
 * from the ranks of a tensor-parallel group, no counterpart in the reference): column c of row r is
 * x_dev[(c / segment) * segment_stride + r * stride + c % segment]. */
int32_t neura_cuda_argmax_segments(nc_context *ctx, void *stream, const float *x_dev, uint32_t rows, uint32_t width,
                                   uint64_t stride, uint32_t segment, uint64_t segment_stride, uint32_t *out_dev);

/* The angles of one decode step: table_dev[b][c] = (cosine, sine) of position_dev[b] in channel c < width / 2
 * (the angle of rope.rs:48-122).  They are the same in every layer, so a step computes them once. */
int32_t neura_cuda_rope_table(nc_context *ctx, void *stream, const uint32_t *position_dev, float base, uint32_t batch,
                              uint32_t width, float *table_dev);

/* neura_cuda_rope_cache and neura_cuda_attend as one launch: `qkv_dev` holds the un-turned q | k | v rows of this
 * step (they are left as they are); the queries are turned by table_dev (neura_cuda_rope_table) as the kernel loads
 * them, and the new key (turned) and value go to slot position_dev[b] of the cache before the row attends to
 * positions 0..position_dev[b].  Bit for bit what the two launches give. */
int32_t neura_cuda_rope_attend(nc_context *ctx, void *stream, const float *qkv_dev, uint64_t row_stride,
                               const uint32_t *position_dev, const float *table_dev, float scale, uint32_t batch,
                               uint32_t heads, uint32_t key_heads, uint32_t width, uint32_t capacity, float *keys_dev,
                               float *values_dev, float *out_dev, uint64_t out_stride);

/* graph.gather of a quantised embedding table (crates/neura-kernel/src/task/select.rs:29-49 with
 * fetch_q8_0 / fetch_q4_k, fetch.rs:236-267): out[r] = dequantised row tokens_dev[r], bit-exact;
 * the table may be in either layout (a tied head is sealed). */
int32_t neura_cuda_embed(nc_context *ctx, void *stream, const nc_weight *table, const uint32_t *tokens_dev,
                         uint32_t rows, float *out_dev, uint64_t out_stride);

/* cursor += by for every sequence (Batch::step's advance, crates/neura-generate/src/batch.rs:1716-1725),
 * on the device so that a recorded decode step replays without host writes. */
int32_t neura_cuda_advance(nc_context *ctx, void *stream, uint32_t *position_dev, uint32_t rows, uint32_t by);

/* ---- tensor-parallel exchange over NVLink peer memory (no counterpart in the reference, which runs on one device) ---- */

/* A communicator of one process per GPU on one box.  neura_cuda_comm_create allocates this rank's
 * buffer (room for all-reduces of up to `max_count` f32) and writes its 64-byte CUDA IPC handle to
 * `handle_out`; the caller gathers the handles of all ranks (any host channel) and gives them, in
 * rank order, to neura_cuda_comm_connect, which maps the peers' buffers. */
typedef struct nc_comm nc_comm;
int32_t neura_cuda_comm_create(nc_context *ctx, uint64_t max_count, nc_comm **out, void *handle_out);
int32_t neura_cuda_comm_connect(nc_context *ctx, nc_comm *comm, uint32_t rank, uint32_t world, const void *handles);
/* The same for a group whose communicators all live in this process (one host thread per GPU, or a test
 * with several seats on one GPU): `all` holds the `world` communicators in rank order, all[rank] == comm;
 * peers on other GPUs are reached through peer access, which this call enables. */
int32_t neura_cuda_comm_connect_local(nc_context *ctx, nc_comm *comm, uint32_t rank, uint32_t world, nc_comm *const *all);
int32_t neura_cuda_comm_destroy(nc_context *ctx, nc_comm *comm);

/* inout_dev[i] <- sum over the ranks of their inout_dev[i], added in rank order (every rank gets
 * the same bits).  One kernel: every rank pushes its partial sums into its seat of every peer's buffer
 * (plain peer stores over NVLink; nothing is read remotely), the only waiting is on the peers' sequence
 * flags, bounded by the context's wait limit; a rank that gives up leaves its input untouched, the
 * next neura_cuda_sync returns the refusal, and the call can be issued again (it repeats its sequence
 * number and completes once the missing peer has pushed).  Every rank must
 * issue the same calls in the same order.  `count` is a multiple of 4, `inout_dev` 16-byte aligned. */
int32_t neura_cuda_allreduce(nc_context *ctx, void *stream, nc_comm *comm, float *inout_dev, uint32_t count);

/* neura_cuda_allreduce of `rows` rows of `k` numbers followed, in the same launch, by neura_cuda_rms_norm_stage
 * of the summed rows (a row-parallel projection is followed by the next block's norm in every decoder layer). */
int32_t neura_cuda_allreduce_norm_stage(nc_context *ctx, void *stream, nc_comm *comm, float *inout_dev, uint32_t rows,
                                        uint32_t k, const float *weight_dev, float floor, uint32_t element);

/* No counterpart in the reference.  neura_cuda_linear for callers that may not touch the
 * device allocator: a game loop stepping generation under a frame budget (where a
 * cudaMalloc, or the device-wide wait a cudaFree implies, would blow the frame), or a host
 * engine that owns all device memory and admits no third-party allocation.  Same result as
 * neura_cuda_linear, but every byte of scratch comes from one fixed 16 MiB array inside the
 * library image (each GPU that loads the library holds it until exit) and the call makes no
 * cudaMalloc, cudaFree or other allocating call.
 *  - limits: 1 to 4 rows, w->k <= 32768, w->n <= 262144; anything larger is refused with a
 *    sentence in neura_cuda_last_error();
 *  - the first call on a device looks the array's device address up (cudaGetSymbolAddress) and has
 *    the CUDA runtime load the kernels the entry point can launch (loading a kernel on first use may
 *    allocate): make that first call at set-up time, outside any stream capture; later calls only launch;
 *  - a kernel that gives up on a bounded wait raises a status word kept in the array; neura_cuda_sync
 *    reports it like any other refusal;
 *  - all calls on a device share the array: two calls whose kernels can overlap on the GPU
 *    (different streams without an ordering between them) race; order them. */
int32_t neura_cuda_linear_static(nc_context *ctx, void *stream, const nc_weight *w, const float *x_dev,
                                 uint32_t rows, uint64_t x_stride, float *out_dev, uint64_t out_stride,
                                 const nc_step *chain, uint32_t n_steps);

/* Staging slots.  A context keeps three staged forms of activation rows; neura_cuda_stage, neura_cuda_stage_window
 * and neura_cuda_rms_norm_stage write, and the staged products read, the selected one (slot 0 until told otherwise). */
#define NC_NO_SLOT 0xffffffffu
int32_t neura_cuda_staging_select(nc_context *ctx, uint32_t slot);

/* neura_cuda_linear_staged over the selected slot (1 or 2 rows) with the staging of the NEXT product folded into
 * its epilogue (the planner's fusion of a product with the pointwise tasks that follow it,
 * crates/neura-plan/src/lower.rs:415-423, taken one step further): when then_slot is a slot, the warp that
 * completes a 256-column chunk of the output rows digitises it into that slot at once, multiplied by
 * then_gain_dev (a coming rms_norm's weight, or NULL), and with then_squares leaves the chunk's sum of squares
 * with the context.  `normed` says that the rows being read were staged that way: the product multiplies its
 * outputs by their norm's scalar 1 / sqrt(mean(x^2) + floor) (a product is linear in a row scale), so
 *   rms_norm_stage(x, g) ; linear_staged(W)   ==   [x staged with gain g and squares] ; linear_staged_then(W, normed)
 * up to the rounding of the staging.  then_slot = NC_NO_SLOT stages nothing. */
int32_t neura_cuda_linear_staged_then(nc_context *ctx, void *stream, const nc_weight *w, float *out_dev, uint64_t out_stride,
                                      const nc_step *chain, uint32_t n_steps, uint32_t normed, float floor,
                                      uint32_t then_slot, const float *then_gain_dev, uint32_t then_squares);

/* neura_cuda_linear_staged_then for a rank of a tensor-parallel group (no counterpart in the reference, which runs on
 * one device).  Two additions:
 *  - `then` says where the output rows sit on the K axis of the product that will read them: elements [lo, hi) of
 *    an axis of `k` (a row-parallel weight keeps the whole blocks that cover its share of K, neura_cuda_stage_window);
 *    k = 0 means the rows as they are;
 *  - `reduce`, when not NULL, says that the rows this rank computes are partial sums over its share of K: the warp
 *    that completes a 256-column chunk pushes it to every peer (plain peer stores over NVLink), waits (bounded by the
 *    context's wait limit) for the peers' chunks and adds them up in rank order, so that `out_dev` ends up holding the
 *    sums on every rank, bit for bit the same, and it is the sums that get staged.  One launch where a row-parallel
 *    projection had three (product, all-reduce, staging).  Rows of a multiple of 256 numbers; every rank issues the
 *    same calls in the same order; a chunk whose wait runs out raises the status word (neura_cuda_sync reports it)
 *    and leaves the call incomplete, after which the group makes a new communicator. */
typedef struct nc_then {
    uint32_t slot;            /* the staging slot the output rows go to; NC_NO_SLOT stages nothing */
    uint32_t k, lo, hi;       /* the rows are elements [lo, hi) of a K axis of k; k = 0: the rows as they are */
    const float *gain_dev;    /* a coming rms_norm's weight [hi - lo], or NULL */
    uint32_t squares;         /* 1: leave the chunks' sums of squares with the context */
} nc_then;
int32_t neura_cuda_linear_staged_fused(nc_context *ctx, void *stream, const nc_weight *w, float *out_dev, uint64_t out_stride,
                                       const nc_step *chain, uint32_t n_steps, uint32_t normed, float floor, nc_comm *reduce,
                                       const nc_then *then);

/* The same product called the way Runtime::{write, run, read} are (runtime.rs:1020,833,1064):
 * activations come from and results return to host memory; blocks until done. */
int32_t neura_cuda_linear_host(nc_context *ctx, void *stream, const nc_weight *w, const float *x_host,
                               uint32_t rows, float *out_host, const nc_step *chain, uint32_t n_steps);

/* Runtime::compile / Runtime::run (runtime.rs:528,833): the calls issued on `stream`
 * between capture_begin and capture_end are recorded into a program (a CUDA graph)
 * instead of running; program_run replays them with one launch.  `stream` must not be
 * the default stream.  Scratch cannot grow while recording: neura_cuda_reserve first. */
typedef struct nc_program nc_program;
int32_t neura_cuda_capture_begin(nc_context *ctx, void *stream);
int32_t neura_cuda_capture_end(nc_context *ctx, void *stream, nc_program **out);
int32_t neura_cuda_program_run(nc_context *ctx, void *stream, nc_program *program);
int32_t neura_cuda_program_free(nc_context *ctx, nc_program *program);

/* ---- a whole decode step as one persistent kernel ---------------------------------------------------
 * The reference compiles a step into one device megakernel that walks task records
 * (Runtime::compile, runtime.rs:528; crates/neura-kernel/src/substrate.rs).  neura_cuda_decoder_compile
 * does the same for a Qwen-shaped decoder (examples/qwen/model.rs:77-103): it lays the step out as a
 * table of phases (embedding gather; per layer: rms_norm + q|k|v product, RoPE + cache write + attention,
 * output product + residual, rms_norm + gate|up product with SwiGLU, down product + residual; final
 * rms_norm + head product; argmax; cursor += 1) that ONE cooperative kernel walks, one CTA per SM, with a
 * grid barrier between phases.  neura_cuda_decoder_step is Batch::answer (batch.rs:1716-1725) for every
 * sequence: it reads tokens_dev and position_dev, writes the chosen ids back to tokens_dev, the logits
 * to logits_dev and moves the cursors.  Limits: 1 or 2 sequences, hidden and query width <= 8192. */
typedef struct nc_decoder_layer {
    nc_weight qkv;          /* q, k, v rows stacked, NC_LAYOUT_TILED */
    nc_weight attn_output;  /* NC_LAYOUT_TILED */
    nc_weight gate_up;      /* NC_LAYOUT_TILED_PAIR, n = feed_forward */
    nc_weight down;         /* NC_LAYOUT_TILED */
    const float *attn_norm_dev, *ffn_norm_dev; /* [hidden] */
    float *keys_dev, *values_dev;              /* [batch][key_heads][capacity][head_width] */
} nc_decoder_layer;

typedef struct nc_decoder_desc {
    uint32_t layers, hidden, heads, key_heads, head_width, feed_forward, vocab;
    uint32_t batch, capacity;
    float floor, rope_base, scale;
    nc_weight embedding;     /* [vocab, hidden], either layout */
    nc_weight head;          /* [vocab, hidden], NC_LAYOUT_TILED */
    const float *output_norm_dev;
    const nc_decoder_layer *layer; /* host array of `layers` entries */
    uint32_t *tokens_dev, *position_dev; /* [batch] */
    float *logits_dev;                   /* [batch][vocab] */
} nc_decoder_desc;

typedef struct nc_decoder nc_decoder;
int32_t neura_cuda_decoder_compile(nc_context *ctx, const nc_decoder_desc *desc, nc_decoder **out);
/* The same for rank `rank` of a tensor-parallel group of `world` devices (no counterpart in the reference, which
 * runs on one device).  `desc` describes the rank's shares: heads, key_heads, feed_forward and vocab are the
 * rank's (the head holds rows [rank, rank + 1) * vocab of the group's vocabulary, the embedding all vocab * world
 * rows); attn_output and down keep the whole blocks that cover the rank's share of their K axes.  The output and
 * down products add the ranks' partial sums up inside the step (the exchange of neura_cuda_linear_staged_fused,
 * plain peer stores, bounded waits), rank 0 carries the residual, and a last phase picks among the ranks' argmax
 * winners, so every rank leaves the same token ids in tokens_dev.  `comm` is connected, holds batch * hidden numbers
 * and serves no other call while a step runs.  A wait that runs out raises the status word (neura_cuda_sync
 * reports it) and ends the step at its next barrier. */
int32_t neura_cuda_decoder_compile_rank(nc_context *ctx, const nc_decoder_desc *desc, nc_comm *comm, uint32_t world,
                                        uint32_t rank, nc_decoder **out);
int32_t neura_cuda_decoder_step(nc_context *ctx, void *stream, nc_decoder *decoder);
int32_t neura_cuda_decoder_free(nc_context *ctx, nc_decoder *decoder);

/* Where the last completed step spent its time (the reference's Trace of a run,
 * crates/neura-runtime/src/runtime.rs:95-121): for each phase of the table its kind (1 embedding,
 * 2 product, 3 attention, 4 staging, 5 argmax) and the nanoseconds from the moment CTA 0 entered it to
 * the moment it entered the next one (so a phase's barrier counts with it).  Writes the number of phases
 * to phases_out; fills the arrays when `capacity` holds them.  Synchronise the stream first. */
int32_t neura_cuda_decoder_trace(nc_context *ctx, nc_decoder *decoder, uint32_t capacity, uint32_t *kinds_out,
                                 uint64_t *nanos_out, uint32_t *phases_out);

/* Streams for callers without a CUDA runtime of their own (Queue, crates/neura-gpu/src/context.rs:287). */
int32_t neura_cuda_stream_create(nc_context *ctx, void **out_stream);
int32_t neura_cuda_stream_destroy(nc_context *ctx, void *stream);

/* Kernel launches issued through this context since it was opened (replays included). */
uint64_t neura_cuda_launches(const nc_context *ctx);

#ifdef __cplusplus
}
#endif
#endif /* NEURA_CUDA_H */
