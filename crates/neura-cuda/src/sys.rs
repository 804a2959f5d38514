//! The C ABI of `libneura_cuda` (`include/neura_cuda.h`), one declaration per entry point, in the header's order.
//! Nothing here is safe to call without reading the header's contract for the entry point; `lib.rs` wraps the calls
//! the decoder path makes.

#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_void};

/// Element codes: the discriminants of `neura_abi::Element` (`crates/neura-abi/src/element.rs:3-17`).
pub const NC_ELEMENT_SINGLE: u32 = 0;
pub const NC_ELEMENT_HALF: u32 = 1;
pub const NC_ELEMENT_BFLOAT16: u32 = 2;
pub const NC_ELEMENT_Q8_0: u32 = 8;
pub const NC_ELEMENT_Q4K: u32 = 9;
pub const NC_ELEMENT_Q5K: u32 = 10;
pub const NC_ELEMENT_Q6K: u32 = 11;
pub const NC_ELEMENT_Q3K: u32 = 12;

pub const NC_LAYOUT_GGUF: u32 = 0;
pub const NC_LAYOUT_TILED: u32 = 1;
pub const NC_LAYOUT_TILED_PAIR: u32 = 2;

pub const NC_MAX_STEPS: u32 = 4;
pub const NC_NO_SLOT: u32 = 0xffff_ffff;

#[repr(C)]
pub struct NcContext {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct NcComm {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct NcProgram {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct NcDecoder {
    _opaque: [u8; 0],
}

/// `nc_weight`: the subset of `ValueRecord` a linear layer needs (`crates/neura-abi/src/record.rs:151-165`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NcWeight {
    pub data_dev: *const c_void,
    pub element: u32,
    pub layout: u32,
    pub n: u32,
    pub k: u32,
}

/// `nc_step`: `StepRecord{op, operand, swapped}` (`crates/neura-abi/src/record.rs:72-76`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NcStep {
    pub op: u32,
    pub swapped: u32,
    pub operand_dev: *const f32,
    pub row_stride: i64,
    pub col_stride: i64,
}

/// `nc_then`: where a product's output rows go next (`neura_cuda_linear_staged_fused`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NcThen {
    pub slot: u32,
    pub k: u32,
    pub lo: u32,
    pub hi: u32,
    pub gain_dev: *const f32,
    pub squares: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct NcDecoderLayer {
    pub qkv: NcWeight,
    pub attn_output: NcWeight,
    pub gate_up: NcWeight,
    pub down: NcWeight,
    pub attn_norm_dev: *const f32,
    pub ffn_norm_dev: *const f32,
    pub keys_dev: *mut f32,
    pub values_dev: *mut f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct NcDecoderDesc {
    pub layers: u32,
    pub hidden: u32,
    pub heads: u32,
    pub key_heads: u32,
    pub head_width: u32,
    pub feed_forward: u32,
    pub vocab: u32,
    pub batch: u32,
    pub capacity: u32,
    pub floor: f32,
    pub rope_base: f32,
    pub scale: f32,
    pub embedding: NcWeight,
    pub head: NcWeight,
    pub output_norm_dev: *const f32,
    pub layer: *const NcDecoderLayer,
    pub tokens_dev: *mut u32,
    pub position_dev: *mut u32,
    pub logits_dev: *mut f32,
}

extern "C" {
    pub fn neura_cuda_last_error() -> *const c_char;
    pub fn neura_cuda_open(device: i32, out: *mut *mut NcContext) -> i32;
    pub fn neura_cuda_close(ctx: *mut NcContext) -> i32;
    pub fn neura_cuda_payload_bytes(element: u32, elements: u64) -> u64;
    pub fn neura_cuda_sealed_bytes(element: u32, n: u32, k: u32) -> u64;
    pub fn neura_cuda_alloc(ctx: *mut NcContext, bytes: u64, out_dev: *mut *mut c_void) -> i32;
    pub fn neura_cuda_free(ctx: *mut NcContext, ptr_dev: *mut c_void) -> i32;
    pub fn neura_cuda_host_alloc(ctx: *mut NcContext, bytes: u64, out_host: *mut *mut c_void) -> i32;
    pub fn neura_cuda_host_free(ctx: *mut NcContext, ptr_host: *mut c_void) -> i32;
    pub fn neura_cuda_write(ctx: *mut NcContext, stream: *mut c_void, dst_dev: *mut c_void, src_host: *const c_void, bytes: u64) -> i32;
    pub fn neura_cuda_read(ctx: *mut NcContext, stream: *mut c_void, dst_host: *mut c_void, src_dev: *const c_void, bytes: u64) -> i32;
    pub fn neura_cuda_sync(ctx: *mut NcContext, stream: *mut c_void) -> i32;
    pub fn neura_cuda_memory(ctx: *mut NcContext, free_out: *mut u64, total_out: *mut u64) -> i32;
    pub fn neura_cuda_set_wait_limit(ctx: *mut NcContext, nanoseconds: u64) -> i32;
    pub fn neura_cuda_reserve(ctx: *mut NcContext, rows: u32, n: u32, k: u32) -> i32;
    pub fn neura_cuda_reserve_decoder(ctx: *mut NcContext, rows: u32, heads: u32, key_heads: u32, width: u32, capacity: u32) -> i32;
    pub fn neura_cuda_reserve_bf16(ctx: *mut NcContext, rows: u32, k: u32) -> i32;
    pub fn neura_cuda_weight_seal(ctx: *mut NcContext, stream: *mut c_void, element: u32, n: u32, k: u32, gguf_dev: *const c_void, dst_dev: *mut c_void) -> i32;
    pub fn neura_cuda_sealed_pair_bytes(element: u32, n: u32, k: u32) -> u64;
    pub fn neura_cuda_weight_seal_pair(ctx: *mut NcContext, stream: *mut c_void, element: u32, n: u32, k: u32, gate_gguf_dev: *const c_void, up_gguf_dev: *const c_void, dst_dev: *mut c_void) -> i32;
    pub fn neura_cuda_dequant(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, out_dev: *mut f32) -> i32;
    pub fn neura_cuda_quantize(ctx: *mut NcContext, stream: *mut c_void, element: u32, src_dev: *const f32, elements: u64, dst_dev: *mut c_void) -> i32;
    pub fn neura_cuda_linear(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, x_dev: *const f32, rows: u32, x_stride: u64, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32) -> i32;
    pub fn neura_cuda_linear_bf16(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, x_dev: *const f32, rows: u32, x_stride: u64, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32) -> i32;
    pub fn neura_cuda_stage(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, x_stride: u64, k: u32, element: u32) -> i32;
    pub fn neura_cuda_stage_window(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, x_stride: u64, k: u32, element: u32, lo: u32, hi: u32) -> i32;
    pub fn neura_cuda_linear_staged(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32) -> i32;
    pub fn neura_cuda_rms_norm_stage(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, x_stride: u64, k: u32, weight_dev: *const f32, floor: f32, element: u32, normed_dev: *mut f32, normed_stride: u64) -> i32;
    pub fn neura_cuda_rms_norm(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, x_stride: u64, k: u32, weight_dev: *const f32, floor: f32, out_dev: *mut f32, out_stride: u64) -> i32;
    pub fn neura_cuda_rope_cache(ctx: *mut NcContext, stream: *mut c_void, qkv_dev: *mut f32, row_stride: u64, position_dev: *const u32, base: f32, batch: u32, heads: u32, key_heads: u32, width: u32, capacity: u32, keys_dev: *mut f32, values_dev: *mut f32) -> i32;
    pub fn neura_cuda_attend(ctx: *mut NcContext, stream: *mut c_void, q_dev: *const f32, q_stride: u64, keys_dev: *const f32, values_dev: *const f32, position_dev: *const u32, scale: f32, batch: u32, heads: u32, key_heads: u32, width: u32, capacity: u32, out_dev: *mut f32, out_stride: u64) -> i32;
    pub fn neura_cuda_rope_cache_rows(ctx: *mut NcContext, stream: *mut c_void, qkv_dev: *mut f32, row_stride: u64, position_dev: *const u32, base: f32, rows: u32, heads: u32, key_heads: u32, width: u32, capacity: u32, keys_dev: *mut f32, values_dev: *mut f32) -> i32;
    pub fn neura_cuda_attend_rows(ctx: *mut NcContext, stream: *mut c_void, q_dev: *const f32, q_stride: u64, keys_dev: *const f32, values_dev: *const f32, position_dev: *const u32, scale: f32, rows: u32, heads: u32, key_heads: u32, width: u32, capacity: u32, out_dev: *mut f32, out_stride: u64) -> i32;
    pub fn neura_cuda_argmax(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, width: u32, stride: u64, out_dev: *mut u32) -> i32;
    pub fn neura_cuda_argmax_segments(ctx: *mut NcContext, stream: *mut c_void, x_dev: *const f32, rows: u32, width: u32, stride: u64, segment: u32, segment_stride: u64, out_dev: *mut u32) -> i32;
    pub fn neura_cuda_rope_table(ctx: *mut NcContext, stream: *mut c_void, position_dev: *const u32, base: f32, batch: u32, width: u32, table_dev: *mut f32) -> i32;
    pub fn neura_cuda_rope_attend(ctx: *mut NcContext, stream: *mut c_void, qkv_dev: *const f32, row_stride: u64, position_dev: *const u32, table_dev: *const f32, scale: f32, batch: u32, heads: u32, key_heads: u32, width: u32, capacity: u32, keys_dev: *mut f32, values_dev: *mut f32, out_dev: *mut f32, out_stride: u64) -> i32;
    pub fn neura_cuda_embed(ctx: *mut NcContext, stream: *mut c_void, table: *const NcWeight, tokens_dev: *const u32, rows: u32, out_dev: *mut f32, out_stride: u64) -> i32;
    pub fn neura_cuda_advance(ctx: *mut NcContext, stream: *mut c_void, position_dev: *mut u32, rows: u32, by: u32) -> i32;
    pub fn neura_cuda_comm_create(ctx: *mut NcContext, max_count: u64, out: *mut *mut NcComm, handle_out: *mut c_void) -> i32;
    pub fn neura_cuda_comm_connect(ctx: *mut NcContext, comm: *mut NcComm, rank: u32, world: u32, handles: *const c_void) -> i32;
    pub fn neura_cuda_comm_connect_local(ctx: *mut NcContext, comm: *mut NcComm, rank: u32, world: u32, all: *const *mut NcComm) -> i32;
    pub fn neura_cuda_comm_destroy(ctx: *mut NcContext, comm: *mut NcComm) -> i32;
    pub fn neura_cuda_allreduce(ctx: *mut NcContext, stream: *mut c_void, comm: *mut NcComm, inout_dev: *mut f32, count: u32) -> i32;
    pub fn neura_cuda_allreduce_norm_stage(ctx: *mut NcContext, stream: *mut c_void, comm: *mut NcComm, inout_dev: *mut f32, rows: u32, k: u32, weight_dev: *const f32, floor: f32, element: u32) -> i32;
    pub fn neura_cuda_linear_static(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, x_dev: *const f32, rows: u32, x_stride: u64, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32) -> i32;
    pub fn neura_cuda_staging_select(ctx: *mut NcContext, slot: u32) -> i32;
    pub fn neura_cuda_linear_staged_then(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32, normed: u32, floor: f32, then_slot: u32, then_gain_dev: *const f32, then_squares: u32) -> i32;
    pub fn neura_cuda_linear_staged_fused(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, out_dev: *mut f32, out_stride: u64, chain: *const NcStep, n_steps: u32, normed: u32, floor: f32, reduce: *mut NcComm, then: *const NcThen) -> i32;
    pub fn neura_cuda_linear_host(ctx: *mut NcContext, stream: *mut c_void, w: *const NcWeight, x_host: *const f32, rows: u32, out_host: *mut f32, chain: *const NcStep, n_steps: u32) -> i32;
    pub fn neura_cuda_capture_begin(ctx: *mut NcContext, stream: *mut c_void) -> i32;
    pub fn neura_cuda_capture_end(ctx: *mut NcContext, stream: *mut c_void, out: *mut *mut NcProgram) -> i32;
    pub fn neura_cuda_program_run(ctx: *mut NcContext, stream: *mut c_void, program: *mut NcProgram) -> i32;
    pub fn neura_cuda_program_free(ctx: *mut NcContext, program: *mut NcProgram) -> i32;
    pub fn neura_cuda_decoder_compile(ctx: *mut NcContext, desc: *const NcDecoderDesc, out: *mut *mut NcDecoder) -> i32;
    pub fn neura_cuda_decoder_compile_rank(ctx: *mut NcContext, desc: *const NcDecoderDesc, comm: *mut NcComm, world: u32, rank: u32, out: *mut *mut NcDecoder) -> i32;
    pub fn neura_cuda_decoder_step(ctx: *mut NcContext, stream: *mut c_void, decoder: *mut NcDecoder) -> i32;
    pub fn neura_cuda_decoder_free(ctx: *mut NcContext, decoder: *mut NcDecoder) -> i32;
    pub fn neura_cuda_decoder_trace(ctx: *mut NcContext, decoder: *mut NcDecoder, capacity: u32, kinds_out: *mut u32, nanos_out: *mut u64, phases_out: *mut u32) -> i32;
    pub fn neura_cuda_stream_create(ctx: *mut NcContext, out_stream: *mut *mut c_void) -> i32;
    pub fn neura_cuda_stream_destroy(ctx: *mut NcContext, stream: *mut c_void) -> i32;
    pub fn neura_cuda_launches(ctx: *const NcContext) -> u64;
}
