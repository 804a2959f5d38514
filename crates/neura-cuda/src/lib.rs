//! Neura's quantized-linear path on an NVIDIA B200, behind the calls `neura-runtime` offers for it.
//!
//! `neura-runtime` drives this path through `Runtime::{open, load, write, run, read}`
//! (`crates/neura-runtime/src/runtime.rs:183,356,1020,833,1064`) over a heap that holds GGUF blocks verbatim
//! (`crates/neura-runtime/src/store.rs:77-157`); the products are `Graph::matmul` over `decoder::matrix` parameters
//! (`crates/neura-graph/src/op.rs:17`, `crates/neura-decoder/src/parameter.rs:5-41`).  `CudaRuntime` keeps those
//! names and argument meanings over `libneura_cuda` (`sys.rs` is its C ABI): weights are poured verbatim and sealed
//! on the device, a product is `linear`, a recorded run of calls is a `Program`.
//!
//! Like the reference, contract violations are panics with the library's sentence (`store.rs:90-123`); only `open`
//! returns a `Result` (`GpuUnavailable`, `crates/neura-gpu/src/context.rs:56-123`).  One thread drives one runtime.
//! There is no CPU path: where the library or a B200 is missing, `open` fails.

pub mod sys;

use core::ffi::c_void;
use std::ffi::CStr;
use std::ptr;

pub use neura_abi::Element;

/// Why a runtime could not be opened (`GpuUnavailable` in the reference).
#[derive(Debug, Clone)]
pub struct CudaUnavailable {
    pub code: i32,
    pub sentence: String,
}

impl std::fmt::Display for CudaUnavailable {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "[{}] {}", self.code, self.sentence)
    }
}

impl std::error::Error for CudaUnavailable {}

fn last_error() -> String {
    // the library keeps the sentence of the last refusal per thread
    unsafe { CStr::from_ptr(sys::neura_cuda_last_error()) }.to_string_lossy().into_owned()
}

/// Host contract violations panic with a sentence, as the reference's do.
fn check(code: i32) {
    if code != 0 {
        panic!("neura-cuda [{code}]: {}", last_error());
    }
}

fn element_code(element: Element) -> u32 {
    element as u32
}

/// A run of bytes in device memory owned by a runtime (`GpuBuffer`, `crates/neura-gpu/src/buffer.rs:30-177`).
pub struct DeviceBuffer {
    ptr: *mut c_void,
    bytes: u64,
}

impl DeviceBuffer {
    pub fn bytes(&self) -> u64 {
        self.bytes
    }
    pub fn as_f32(&self) -> *mut f32 {
        self.ptr.cast()
    }
    pub fn as_u32(&self) -> *mut u32 {
        self.ptr.cast()
    }
}

/// A block-quantised `[n, k]` matrix on the device: what `decoder::matrix` declares and `load` pours.
#[derive(Clone, Copy)]
pub struct Weight {
    record: sys::NcWeight,
}

impl Weight {
    pub fn rows(&self) -> u32 {
        self.record.n
    }
    pub fn columns(&self) -> u32 {
        self.record.k
    }
    pub fn record(&self) -> &sys::NcWeight {
        &self.record
    }
}

/// One step of a product's fused epilogue (`StepRecord`, `crates/neura-abi/src/record.rs:72-76`); `op` is a
/// `neura-pointwise` code (`crates/neura-pointwise/src/op.rs:141-170`), the operand is read at the output coordinate
/// through broadcast strides.
#[derive(Clone, Copy)]
pub struct Step {
    pub op: u32,
    pub swapped: bool,
    pub operand: *const f32,
    pub row_stride: i64,
    pub col_stride: i64,
}

impl Step {
    pub fn unary(op: u32) -> Self {
        Step { op, swapped: false, operand: ptr::null(), row_stride: 0, col_stride: 0 }
    }
    /// An operand of the output's own shape, rows `row_stride` apart.
    pub fn with(op: u32, operand: &DeviceBuffer, row_stride: i64) -> Self {
        Step { op, swapped: false, operand: operand.as_f32(), row_stride, col_stride: 1 }
    }
}

fn records(chain: &[Step]) -> Vec<sys::NcStep> {
    assert!(chain.len() <= sys::NC_MAX_STEPS as usize, "an epilogue holds at most {} steps", sys::NC_MAX_STEPS);
    chain
        .iter()
        .map(|step| sys::NcStep {
            op: step.op,
            swapped: step.swapped as u32,
            operand_dev: step.operand,
            row_stride: step.row_stride,
            col_stride: step.col_stride,
        })
        .collect()
}

/// A recorded run of calls (`Program`, `crates/neura-runtime/src/program.rs:124`): replayed with one launch.
pub struct Program {
    handle: *mut sys::NcProgram,
}

/// One GPU and one stream of work: the role of `neura_runtime::Runtime` for this path.
pub struct CudaRuntime {
    ctx: *mut sys::NcContext,
    stream: *mut c_void,
}

impl CudaRuntime {
    /// `Runtime::open` (`runtime.rs:183`): binds the calling thread's work to GPU `device`.
    pub fn open(device: i32) -> Result<Self, CudaUnavailable> {
        let mut ctx = ptr::null_mut();
        let code = unsafe { sys::neura_cuda_open(device, &mut ctx) };
        if code != 0 {
            return Err(CudaUnavailable { code, sentence: last_error() });
        }
        let mut stream = ptr::null_mut();
        let code = unsafe { sys::neura_cuda_stream_create(ctx, &mut stream) };
        if code != 0 {
            let sentence = last_error();
            unsafe { sys::neura_cuda_close(ctx) };
            return Err(CudaUnavailable { code, sentence });
        }
        Ok(CudaRuntime { ctx, stream })
    }

    /// `Element::payload_bytes` (`crates/neura-abi/src/element.rs:231-241`) as the library counts it.
    pub fn payload_bytes(element: Element, elements: u64) -> u64 {
        unsafe { sys::neura_cuda_payload_bytes(element_code(element), elements) }
    }

    /// Free and total bytes of the GPU (what a `MemoryRequest` is sized from, `runtime.rs:150-167`).
    pub fn memory(&self) -> (u64, u64) {
        let (mut free, mut total) = (0u64, 0u64);
        check(unsafe { sys::neura_cuda_memory(self.ctx, &mut free, &mut total) });
        (free, total)
    }

    /// How long a kernel waits for another party before it gives up (the reference's `FRAME_TIMEOUT`,
    /// `crates/neura-gpu/src/native.rs:20-35`).
    pub fn set_wait_limit(&self, nanoseconds: u64) {
        check(unsafe { sys::neura_cuda_set_wait_limit(self.ctx, nanoseconds) });
    }

    // ---- memory ----------------------------------------------------------------------------------------
    pub fn alloc(&self, bytes: u64) -> DeviceBuffer {
        let mut ptr = ptr::null_mut();
        check(unsafe { sys::neura_cuda_alloc(self.ctx, bytes, &mut ptr) });
        DeviceBuffer { ptr, bytes }
    }

    pub fn free(&self, buffer: DeviceBuffer) {
        check(unsafe { sys::neura_cuda_free(self.ctx, buffer.ptr) });
    }

    /// `Runtime::write` (`runtime.rs:1020`): host numbers into a device value.  Returns when the copy is done.
    pub fn write(&self, buffer: &DeviceBuffer, values: &[f32]) {
        assert!(values.len() as u64 * 4 <= buffer.bytes, "writing {} numbers into a value of {} bytes", values.len(), buffer.bytes);
        check(unsafe { sys::neura_cuda_write(self.ctx, self.stream, buffer.ptr, values.as_ptr().cast(), values.len() as u64 * 4) });
        self.sync();
    }

    pub fn write_u32(&self, buffer: &DeviceBuffer, values: &[u32]) {
        assert!(values.len() as u64 * 4 <= buffer.bytes, "writing {} numbers into a value of {} bytes", values.len(), buffer.bytes);
        check(unsafe { sys::neura_cuda_write(self.ctx, self.stream, buffer.ptr, values.as_ptr().cast(), values.len() as u64 * 4) });
        self.sync();
    }

    /// `Runtime::read` (`runtime.rs:1064`): blocking readback.
    pub fn read(&self, buffer: &DeviceBuffer, count: usize) -> Vec<f32> {
        assert!(count as u64 * 4 <= buffer.bytes, "reading {count} numbers out of a value of {} bytes", buffer.bytes);
        let mut out = vec![0.0f32; count];
        check(unsafe { sys::neura_cuda_read(self.ctx, self.stream, out.as_mut_ptr().cast(), buffer.ptr, count as u64 * 4) });
        self.sync();
        out
    }

    pub fn read_u32(&self, buffer: &DeviceBuffer, count: usize) -> Vec<u32> {
        assert!(count as u64 * 4 <= buffer.bytes, "reading {count} numbers out of a value of {} bytes", buffer.bytes);
        let mut out = vec![0u32; count];
        check(unsafe { sys::neura_cuda_read(self.ctx, self.stream, out.as_mut_ptr().cast(), buffer.ptr, count as u64 * 4) });
        self.sync();
        out
    }

    /// `Run::complete` (`runtime.rs:123`): waits for the stream; a kernel that gave up on a bounded wait since the
    /// last call surfaces here, as the reference's refusal word does at a read (`runtime.rs:75-85`).
    pub fn sync(&self) {
        check(unsafe { sys::neura_cuda_sync(self.ctx, self.stream) });
    }

    /// Sizes the context's scratch for products of up to `rows` rows against matrices of up to `[n, k]`, so that
    /// later calls (and recorded programs) never allocate.
    pub fn reserve(&self, rows: u32, n: u32, k: u32) {
        check(unsafe { sys::neura_cuda_reserve(self.ctx, rows, n, k) });
    }

    /// What `linear_bf16` keeps between its kernels for up to `rows` rows of `k` activations, sized before a program
    /// is recorded around such products.
    pub fn reserve_bf16(&self, rows: u32, k: u32) {
        check(unsafe { sys::neura_cuda_reserve_bf16(self.ctx, rows, k) });
    }

    pub fn reserve_decoder(&self, rows: u32, heads: u32, key_heads: u32, width: u32, capacity: u32) {
        check(unsafe { sys::neura_cuda_reserve_decoder(self.ctx, rows, heads, key_heads, width, capacity) });
    }

    // ---- weights ---------------------------------------------------------------------------------------
    /// `Runtime::load` for one tensor: pours the GGUF payload verbatim (`store.rs:131-135`) and seals it into the
    /// layout the streaming kernels read.  The shape contract is `decoder::matrix`'s: GGUF `ne[0] = k` (columns),
    /// `ne[1] = n` (rows) (`crates/neura-decoder/src/parameter.rs:7-13`).  A Q6_K tensor stays in GGUF order.
    pub fn load(&self, element: Element, n: u32, k: u32, gguf: &[u8]) -> Weight {
        let need = Self::payload_bytes(element, n as u64 * k as u64);
        assert!(need > 0, "{} is not a block format this path loads", element.name());
        assert!(gguf.len() as u64 >= need, "a [{n}, {k}] tensor packs {need} bytes and the source holds {}", gguf.len());
        let raw = self.alloc(need.max(16));
        check(unsafe { sys::neura_cuda_write(self.ctx, self.stream, raw.ptr, gguf.as_ptr().cast(), need) });
        self.sync();
        let code = element_code(element);
        if code == sys::NC_ELEMENT_Q6K {
            return Weight { record: sys::NcWeight { data_dev: raw.ptr, element: code, layout: sys::NC_LAYOUT_GGUF, n, k } };
        }
        let sealed = self.alloc(unsafe { sys::neura_cuda_sealed_bytes(code, n, k) });
        check(unsafe { sys::neura_cuda_weight_seal(self.ctx, self.stream, code, n, k, raw.ptr, sealed.ptr) });
        self.sync();
        self.free(raw);
        Weight { record: sys::NcWeight { data_dev: sealed.ptr, element: code, layout: sys::NC_LAYOUT_TILED, n, k } }
    }

    /// `load` for the gate and up projections of an MLP (`examples/qwen/mlp.rs:31-33`): a product with the result is
    /// `silu(gate x) * (up x)`, both tensors streamed once.
    pub fn load_pair(&self, element: Element, n: u32, k: u32, gate: &[u8], up: &[u8]) -> Weight {
        let need = Self::payload_bytes(element, n as u64 * k as u64);
        assert!(gate.len() as u64 >= need && up.len() as u64 >= need, "a [{n}, {k}] tensor packs {need} bytes");
        let (g, u) = (self.alloc(need.max(16)), self.alloc(need.max(16)));
        check(unsafe { sys::neura_cuda_write(self.ctx, self.stream, g.ptr, gate.as_ptr().cast(), need) });
        check(unsafe { sys::neura_cuda_write(self.ctx, self.stream, u.ptr, up.as_ptr().cast(), need) });
        self.sync();
        let code = element_code(element);
        let sealed = self.alloc(unsafe { sys::neura_cuda_sealed_pair_bytes(code, n, k) });
        check(unsafe { sys::neura_cuda_weight_seal_pair(self.ctx, self.stream, code, n, k, g.ptr, u.ptr, sealed.ptr) });
        self.sync();
        self.free(g);
        self.free(u);
        Weight { record: sys::NcWeight { data_dev: sealed.ptr, element: code, layout: sys::NC_LAYOUT_TILED_PAIR, n, k } }
    }

    /// `unpack` (`crates/neura-precision/src/lib.rs:25`) run on the device: `[n, k]` f32, bit-exact.
    pub fn dequant(&self, weight: &Weight, out: &DeviceBuffer) {
        check(unsafe { sys::neura_cuda_dequant(self.ctx, self.stream, &weight.record, out.as_f32()) });
    }

    // ---- the product -----------------------------------------------------------------------------------
    /// `graph.matmul(x, permute(W))` plus the fused chain (`run_matmul` + `chained`,
    /// `crates/neura-kernel/src/task/matmul.rs:376-517`, `pointwise.rs:90-104`); asynchronous on the runtime's stream.
    /// `x` holds `rows` rows `x_stride` numbers apart, `out` rows `out_stride` apart.
    #[allow(clippy::too_many_arguments)]
    pub fn linear(&self, weight: &Weight, x: &DeviceBuffer, rows: u32, x_stride: u64, out: &DeviceBuffer, out_stride: u64, chain: &[Step]) {
        let steps = records(chain);
        check(unsafe {
            sys::neura_cuda_linear(self.ctx, self.stream, &weight.record, x.as_f32(), rows, x_stride, out.as_f32(), out_stride,
                                   steps.as_ptr(), steps.len() as u32)
        });
    }

    /// The tensor path for prefill (`template_run_matmul_cooperative`, `matmul.rs:1344-1565`): bf16 operands, f32
    /// accumulation, a sealed Q4_K weight.
    #[allow(clippy::too_many_arguments)]
    pub fn linear_bf16(&self, weight: &Weight, x: &DeviceBuffer, rows: u32, x_stride: u64, out: &DeviceBuffer, out_stride: u64, chain: &[Step]) {
        let steps = records(chain);
        check(unsafe {
            sys::neura_cuda_linear_bf16(self.ctx, self.stream, &weight.record, x.as_f32(), rows, x_stride, out.as_f32(), out_stride,
                                        steps.as_ptr(), steps.len() as u32)
        });
    }

    /// `write` + `run` + `read` in one call: host activations in, host results out (blocking).
    pub fn linear_host(&self, weight: &Weight, x: &[f32], rows: u32, chain: &[Step]) -> Vec<f32> {
        assert_eq!(x.len() as u64, rows as u64 * weight.record.k as u64, "rows of {} activations", weight.record.k);
        let steps = records(chain);
        let mut out = vec![0.0f32; rows as usize * weight.record.n as usize];
        check(unsafe {
            sys::neura_cuda_linear_host(self.ctx, self.stream, &weight.record, x.as_ptr(), rows, out.as_mut_ptr(), steps.as_ptr(),
                                        steps.len() as u32)
        });
        out
    }

    /// The two halves of `linear` for callers that feed several weights with the same activations (q/k/v, gate/up).
    pub fn stage(&self, x: &DeviceBuffer, rows: u32, x_stride: u64, k: u32, element: Element) {
        check(unsafe { sys::neura_cuda_stage(self.ctx, self.stream, x.as_f32(), rows, x_stride, k, element_code(element)) });
    }

    pub fn linear_staged(&self, weight: &Weight, out: &DeviceBuffer, out_stride: u64, chain: &[Step]) {
        let steps = records(chain);
        check(unsafe {
            sys::neura_cuda_linear_staged(self.ctx, self.stream, &weight.record, out.as_f32(), out_stride, steps.as_ptr(), steps.len() as u32)
        });
    }

    // ---- the steps either side of the products in a decoder layer ----------------------------------------
    /// `decoder::rms` (`crates/neura-decoder/src/op.rs:3-5`) fused with `stage` of its result.
    #[allow(clippy::too_many_arguments)]
    pub fn rms_norm_stage(&self, x: &DeviceBuffer, rows: u32, x_stride: u64, k: u32, weight: Option<&DeviceBuffer>, floor: f32, element: Element) {
        let gain = weight.map_or(ptr::null(), |w| w.as_f32().cast_const());
        check(unsafe {
            sys::neura_cuda_rms_norm_stage(self.ctx, self.stream, x.as_f32(), rows, x_stride, k, gain, floor, element_code(element),
                                           ptr::null_mut(), 0)
        });
    }

    /// `decoder::rms` alone (`crates/neura-decoder/src/op.rs:3-5`): f32 rows out, any number of rows (a wide prompt chunk
    /// on its way to `linear_bf16`).
    #[allow(clippy::too_many_arguments)]
    pub fn rms_norm(&self, x: &DeviceBuffer, rows: u32, x_stride: u64, k: u32, weight: Option<&DeviceBuffer>, floor: f32, out: &DeviceBuffer,
                    out_stride: u64) {
        let gain = weight.map_or(ptr::null(), |w| w.as_f32().cast_const());
        check(unsafe { sys::neura_cuda_rms_norm(self.ctx, self.stream, x.as_f32(), rows, x_stride, k, gain, floor, out.as_f32(), out_stride) });
    }

    /// `decoder::partial` over the full width + `Cache::write` (`crates/neura-decoder/src/rope.rs:3-12`, `cache.rs:267-310`).
    #[allow(clippy::too_many_arguments)]
    pub fn rope_cache(&self, qkv: &DeviceBuffer, row_stride: u64, position: &DeviceBuffer, base: f32, batch: u32, heads: u32, key_heads: u32,
                      width: u32, capacity: u32, keys: &DeviceBuffer, values: &DeviceBuffer) {
        check(unsafe {
            sys::neura_cuda_rope_cache(self.ctx, self.stream, qkv.as_f32(), row_stride, position.as_u32(), base, batch, heads, key_heads, width,
                                       capacity, keys.as_f32(), values.as_f32())
        });
    }

    /// `Cache::attend` (`crates/neura-decoder/src/cache.rs:311-406`) for one new row per sequence.
    #[allow(clippy::too_many_arguments)]
    pub fn attend(&self, q: &DeviceBuffer, q_stride: u64, keys: &DeviceBuffer, values: &DeviceBuffer, position: &DeviceBuffer, scale: f32, batch: u32,
                  heads: u32, key_heads: u32, width: u32, capacity: u32, out: &DeviceBuffer, out_stride: u64) {
        check(unsafe {
            sys::neura_cuda_attend(self.ctx, self.stream, q.as_f32(), q_stride, keys.as_f32(), values.as_f32(), position.as_u32(), scale, batch,
                                   heads, key_heads, width, capacity, out.as_f32(), out_stride)
        });
    }

    /// `Sampling::Greedy` (`crates/neura-generate/src/sampling.rs:79-81`): the lowest index wins a tie.
    pub fn argmax(&self, x: &DeviceBuffer, rows: u32, width: u32, stride: u64, out: &DeviceBuffer) {
        check(unsafe { sys::neura_cuda_argmax(self.ctx, self.stream, x.as_f32(), rows, width, stride, out.as_u32()) });
    }

    /// `graph.gather` of a quantised embedding table (`crates/neura-kernel/src/task/select.rs:29-49`), bit-exact.
    pub fn embed(&self, table: &Weight, tokens: &DeviceBuffer, rows: u32, out: &DeviceBuffer, out_stride: u64) {
        check(unsafe { sys::neura_cuda_embed(self.ctx, self.stream, &table.record, tokens.as_u32(), rows, out.as_f32(), out_stride) });
    }

    /// `Batch::step`'s advance (`crates/neura-generate/src/batch.rs:1716-1725`) on the device.
    pub fn advance(&self, position: &DeviceBuffer, rows: u32, by: u32) {
        check(unsafe { sys::neura_cuda_advance(self.ctx, self.stream, position.as_u32(), rows, by) });
    }

    // ---- recorded programs -----------------------------------------------------------------------------
    /// `Runtime::compile` (`runtime.rs:528`): the calls `record` issues are recorded instead of run.
    pub fn compile(&self, record: impl FnOnce(&CudaRuntime)) -> Program {
        check(unsafe { sys::neura_cuda_capture_begin(self.ctx, self.stream) });
        record(self);
        let mut handle = ptr::null_mut();
        check(unsafe { sys::neura_cuda_capture_end(self.ctx, self.stream, &mut handle) });
        Program { handle }
    }

    /// `Runtime::run` (`runtime.rs:833`): replays a program with one launch (asynchronous).
    pub fn run(&self, program: &Program) {
        check(unsafe { sys::neura_cuda_program_run(self.ctx, self.stream, program.handle) });
    }

    pub fn release(&self, program: Program) {
        check(unsafe { sys::neura_cuda_program_free(self.ctx, program.handle) });
    }

    /// Kernel launches issued through this runtime since it was opened.
    pub fn launches(&self) -> u64 {
        unsafe { sys::neura_cuda_launches(self.ctx) }
    }
}

impl Drop for CudaRuntime {
    fn drop(&mut self) {
        unsafe {
            sys::neura_cuda_stream_destroy(self.ctx, self.stream);
            sys::neura_cuda_close(self.ctx);
        }
    }
}
