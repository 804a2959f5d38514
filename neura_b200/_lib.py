"""ctypes loader for libneura_cuda.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# NEURA_CUDA_LIB names another build of the same library (a build with other compile-time knobs, for A/B timing)
LIB_PATH = os.environ.get("NEURA_CUDA_LIB") or os.path.join(HERE, "lib", "libneura_cuda.so")

# every symbol include/neura_cuda.h declares
SYMBOLS = [
    "neura_cuda_last_error", "neura_cuda_open", "neura_cuda_close", "neura_cuda_payload_bytes",
    "neura_cuda_sealed_bytes", "neura_cuda_alloc", "neura_cuda_free", "neura_cuda_host_alloc",
    "neura_cuda_host_free", "neura_cuda_write", "neura_cuda_read", "neura_cuda_sync", "neura_cuda_reserve",
    "neura_cuda_weight_seal", "neura_cuda_dequant", "neura_cuda_quantize", "neura_cuda_linear",
    "neura_cuda_linear_host", "neura_cuda_launches", "neura_cuda_stage", "neura_cuda_linear_staged",
    "neura_cuda_capture_begin", "neura_cuda_capture_end", "neura_cuda_program_run", "neura_cuda_program_free",
    "neura_cuda_stream_create", "neura_cuda_stream_destroy", "neura_cuda_linear_static",
    "neura_cuda_rms_norm_stage", "neura_cuda_rope_cache", "neura_cuda_attend", "neura_cuda_argmax", "neura_cuda_embed",
    "neura_cuda_advance", "neura_cuda_stage_window", "neura_cuda_argmax_segments", "neura_cuda_sealed_pair_bytes",
    "neura_cuda_weight_seal_pair", "neura_cuda_linear_bf16", "neura_cuda_comm_create",
    "neura_cuda_comm_connect", "neura_cuda_comm_destroy", "neura_cuda_allreduce", "neura_cuda_reserve_decoder",
    "neura_cuda_decoder_compile", "neura_cuda_decoder_step", "neura_cuda_decoder_free", "neura_cuda_decoder_trace", "neura_cuda_rope_attend", "neura_cuda_rope_table", "neura_cuda_allreduce_norm_stage", "neura_cuda_staging_select",
    "neura_cuda_linear_staged_then", "neura_cuda_set_wait_limit", "neura_cuda_memory", "neura_cuda_comm_connect_local",
    "neura_cuda_linear_staged_fused", "neura_cuda_rope_cache_rows", "neura_cuda_attend_rows",
    "neura_cuda_decoder_compile_rank", "neura_cuda_rms_norm", "neura_cuda_reserve_bf16",
]


class NcWeight(ctypes.Structure):
    _fields_ = [
        ("data_dev", ctypes.c_void_p),
        ("element", ctypes.c_uint32),
        ("layout", ctypes.c_uint32),
        ("n", ctypes.c_uint32),
        ("k", ctypes.c_uint32),
    ]


class NcStep(ctypes.Structure):
    _fields_ = [
        ("op", ctypes.c_uint32),
        ("swapped", ctypes.c_uint32),
        ("operand_dev", ctypes.c_void_p),
        ("row_stride", ctypes.c_int64),
        ("col_stride", ctypes.c_int64),
    ]


class NcThen(ctypes.Structure):
    _fields_ = [
        ("slot", ctypes.c_uint32), ("k", ctypes.c_uint32), ("lo", ctypes.c_uint32), ("hi", ctypes.c_uint32),
        ("gain_dev", ctypes.c_void_p), ("squares", ctypes.c_uint32),
    ]


class NcDecoderLayer(ctypes.Structure):
    _fields_ = [
        ("qkv", NcWeight), ("attn_output", NcWeight), ("gate_up", NcWeight), ("down", NcWeight),
        ("attn_norm_dev", ctypes.c_void_p), ("ffn_norm_dev", ctypes.c_void_p),
        ("keys_dev", ctypes.c_void_p), ("values_dev", ctypes.c_void_p),
    ]


class NcDecoderDesc(ctypes.Structure):
    _fields_ = [
        ("layers", ctypes.c_uint32), ("hidden", ctypes.c_uint32), ("heads", ctypes.c_uint32),
        ("key_heads", ctypes.c_uint32), ("head_width", ctypes.c_uint32), ("feed_forward", ctypes.c_uint32),
        ("vocab", ctypes.c_uint32), ("batch", ctypes.c_uint32), ("capacity", ctypes.c_uint32),
        ("floor", ctypes.c_float), ("rope_base", ctypes.c_float), ("scale", ctypes.c_float),
        ("embedding", NcWeight), ("head", NcWeight), ("output_norm_dev", ctypes.c_void_p),
        ("layer", ctypes.POINTER(NcDecoderLayer)),
        ("tokens_dev", ctypes.c_void_p), ("position_dev", ctypes.c_void_p), ("logits_dev", ctypes.c_void_p),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Loads the library (once) and declares the signatures of the C ABI."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m neura_b200.build` (nvcc, sm_100a); "
            "this package has no other implementation of the path"
        )
    lib = ctypes.CDLL(LIB_PATH)
    i32, u32, u64, p = ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p
    pp = ctypes.POINTER(ctypes.c_void_p)
    sig = {
        "neura_cuda_last_error": (ctypes.c_char_p, []),
        "neura_cuda_open": (i32, [i32, pp]),
        "neura_cuda_close": (i32, [p]),
        "neura_cuda_payload_bytes": (u64, [u32, u64]),
        "neura_cuda_sealed_bytes": (u64, [u32, u32, u32]),
        "neura_cuda_alloc": (i32, [p, u64, pp]),
        "neura_cuda_free": (i32, [p, p]),
        "neura_cuda_host_alloc": (i32, [p, u64, pp]),
        "neura_cuda_host_free": (i32, [p, p]),
        "neura_cuda_write": (i32, [p, p, p, p, u64]),
        "neura_cuda_read": (i32, [p, p, p, p, u64]),
        "neura_cuda_sync": (i32, [p, p]),
        "neura_cuda_reserve": (i32, [p, u32, u32, u32]),
        "neura_cuda_reserve_decoder": (i32, [p, u32, u32, u32, u32, u32]),
        "neura_cuda_reserve_bf16": (i32, [p, u32, u32]),
        "neura_cuda_decoder_compile": (i32, [p, ctypes.POINTER(NcDecoderDesc), pp]),
        "neura_cuda_decoder_compile_rank": (i32, [p, ctypes.POINTER(NcDecoderDesc), p, u32, u32, pp]),
        "neura_cuda_decoder_step": (i32, [p, p, p]),
        "neura_cuda_decoder_free": (i32, [p, p]),
        "neura_cuda_decoder_trace": (i32, [p, p, u32, p, p, p]),
        "neura_cuda_weight_seal": (i32, [p, p, u32, u32, u32, p, p]),
        "neura_cuda_dequant": (i32, [p, p, ctypes.POINTER(NcWeight), p]),
        "neura_cuda_quantize": (i32, [p, p, u32, p, u64, p]),
        "neura_cuda_linear": (i32, [p, p, ctypes.POINTER(NcWeight), p, u32, u64, p, u64, ctypes.POINTER(NcStep), u32]),
        "neura_cuda_linear_host": (i32, [p, p, ctypes.POINTER(NcWeight), p, u32, p, ctypes.POINTER(NcStep), u32]),
        "neura_cuda_launches": (u64, [p]),
        "neura_cuda_stage": (i32, [p, p, p, u32, u64, u32, u32]),
        "neura_cuda_linear_staged": (i32, [p, p, ctypes.POINTER(NcWeight), p, u64, ctypes.POINTER(NcStep), u32]),
        "neura_cuda_capture_begin": (i32, [p, p]),
        "neura_cuda_capture_end": (i32, [p, p, pp]),
        "neura_cuda_program_run": (i32, [p, p, p]),
        "neura_cuda_program_free": (i32, [p, p]),
        "neura_cuda_stream_create": (i32, [p, pp]),
        "neura_cuda_stream_destroy": (i32, [p, p]),
        "neura_cuda_rms_norm_stage": (i32, [p, p, p, u32, u64, u32, p, ctypes.c_float, u32, p, u64]),
        "neura_cuda_rms_norm": (i32, [p, p, p, u32, u64, u32, p, ctypes.c_float, p, u64]),
        "neura_cuda_rope_cache": (i32, [p, p, p, u64, p, ctypes.c_float, u32, u32, u32, u32, u32, p, p]),
        "neura_cuda_attend": (i32, [p, p, p, u64, p, p, p, ctypes.c_float, u32, u32, u32, u32, u32, p, u64]),
        "neura_cuda_rope_cache_rows": (i32, [p, p, p, u64, p, ctypes.c_float, u32, u32, u32, u32, u32, p, p]),
        "neura_cuda_attend_rows": (i32, [p, p, p, u64, p, p, p, ctypes.c_float, u32, u32, u32, u32, u32, p, u64]),
        "neura_cuda_rope_attend": (i32, [p, p, p, u64, p, p, ctypes.c_float, u32, u32, u32, u32, u32, p, p, p, u64]),
        "neura_cuda_rope_table": (i32, [p, p, p, ctypes.c_float, u32, u32, p]),
        "neura_cuda_allreduce_norm_stage": (i32, [p, p, p, p, u32, u32, p, ctypes.c_float, u32]),
        "neura_cuda_staging_select": (i32, [p, u32]),
        "neura_cuda_linear_staged_then": (i32, [p, p, ctypes.POINTER(NcWeight), p, u64, ctypes.POINTER(NcStep), u32, u32,
                                             ctypes.c_float, u32, p, u32]),
        "neura_cuda_argmax": (i32, [p, p, p, u32, u32, u64, p]),
        "neura_cuda_embed": (i32, [p, p, ctypes.POINTER(NcWeight), p, u32, p, u64]),
        "neura_cuda_advance": (i32, [p, p, p, u32, u32]),
        "neura_cuda_argmax_segments": (i32, [p, p, p, u32, u32, u64, u32, u64, p]),
        "neura_cuda_sealed_pair_bytes": (u64, [u32, u32, u32]),
        "neura_cuda_weight_seal_pair": (i32, [p, p, u32, u32, u32, p, p, p]),
        "neura_cuda_linear_bf16": (i32, [p, p, ctypes.POINTER(NcWeight), p, u32, u64, p, u64, ctypes.POINTER(NcStep), u32]),
        "neura_cuda_comm_create": (i32, [p, u64, pp, p]),
        "neura_cuda_comm_connect": (i32, [p, p, u32, u32, p]),
        "neura_cuda_comm_destroy": (i32, [p, p]),
        "neura_cuda_allreduce": (i32, [p, p, p, p, u32]),
        "neura_cuda_set_wait_limit": (i32, [p, u64]),
        "neura_cuda_linear_staged_fused": (i32, [p, p, ctypes.POINTER(NcWeight), p, u64, ctypes.POINTER(NcStep), u32, u32,
                                              ctypes.c_float, p, ctypes.POINTER(NcThen)]),
        "neura_cuda_memory": (i32, [p, ctypes.POINTER(u64), ctypes.POINTER(u64)]),
        "neura_cuda_comm_connect_local": (i32, [p, p, u32, u32, pp]),
        "neura_cuda_stage_window": (i32, [p, p, p, u32, u64, u32, u32, u32, u32]),
        "neura_cuda_linear_static": (i32, [p, p, ctypes.POINTER(NcWeight), p, u32, u64, p, u64, ctypes.POINTER(NcStep), u32]),
    }
    for name in SYMBOLS:
        fn = getattr(lib, name)  # raises AttributeError if the library does not export it
        fn.restype, fn.argtypes = sig[name]
    _lib = lib
    return lib
