"""CPU oracle for the quantized-linear path (test infrastructure, never the product).

ctypes bindings over ``libneura_oracle.so`` (``neura_oracle.c`` beside this file, a
plain-C restatement of the reference's host arithmetic; each C function cites
the reference file and lines it follows).  Only the tests, the smoke check and
the benchmark's CPU-baseline leg import this package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Sequence

import numpy as np

SINGLE = 0
HALF = 1
BFLOAT16 = 2
Q8_0 = 8
Q4K = 9
Q5K = 10
Q6K = 11
Q3K = 12

# neura-pointwise op codes in declaration order (crates/neura-pointwise/src/op.rs:141-170)
ADD, MUL, SUB, DIV, MAXIMUM, MINIMUM, RELU, SQRT, RECIP, EXP = range(10)
LOG, TANH, SIGMOID, NEG, ABS, IDENTITY, SIN, COS, POW, FLOOR, GELU, SILU = range(10, 22)

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libneura_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (see the Makefile); returns the library path."""
    src = os.path.join(_HERE, "neura_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libneura_oracle.so"])
    return _SO


class _Step(ctypes.Structure):
    _fields_ = [
        ("op", ctypes.c_uint32),
        ("swapped", ctypes.c_uint32),
        ("operand", ctypes.c_void_p),
        ("row_stride", ctypes.c_int64),
        ("col_stride", ctypes.c_int64),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        u32, u64, f32 = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_float
        p = ctypes.c_void_p
        _lib.nro_f32_to_f16.restype = ctypes.c_uint16
        _lib.nro_f32_to_f16.argtypes = [f32]
        _lib.nro_f16_to_f32.restype = f32
        _lib.nro_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.nro_bf16_rne.restype = ctypes.c_uint16
        _lib.nro_bf16_rne.argtypes = [f32]
        _lib.nro_payload_bytes.restype = u64
        _lib.nro_payload_bytes.argtypes = [u32, u64]
        _lib.nro_packed_bytes.restype = u64
        _lib.nro_packed_bytes.argtypes = [u32, u64]
        _lib.nro_uniform.argtypes = [p, f32, f32, u64, p]
        _lib.nro_normal.argtypes = [p, f32, f32, u64, p]
        _lib.nro_pack.argtypes = [u32, p, u64, p]
        _lib.nro_unpack.argtypes = [u32, u64, p, p]
        _lib.nro_fetch.restype = f32
        _lib.nro_fetch.argtypes = [u32, p, u64]
        _lib.nro_op_apply.restype = f32
        _lib.nro_op_apply.argtypes = [u32, f32, f32]
        for name in ("nro_linear", "nro_linear_bf16"):
            getattr(_lib, name).argtypes = [u32, p, u64, u64, p, u64, u64, p, u64, p, u32, ctypes.c_int]
        _lib.nro_matmul_f32.argtypes = [p, u64, u64, p, u64, p, ctypes.c_int]
        _lib.nro_rms_norm.argtypes = [p, p, f32, u64, u64, p]
        _lib.nro_rope.argtypes = [p, p, f32, u64, u64, u64]
        _lib.nro_attend.argtypes = [p, p, p, p, f32, u64, u64, u64, u64, u64, p]
        _lib.nro_argmax.argtypes = [p, u64, u64, p]
        _lib.nro_embed.argtypes = [u32, p, u64, p, u64, p]
    return _lib


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


class Stream:
    """The reference's xorshift32 stream (crates/neura-graph/src/init.rs:86-91).

    The tests seed it with ``seed | 1`` (crates/neura-runtime/tests/support/mod.rs:41-48);
    consecutive draws continue one stream, as ``Init::samples`` does with ``&mut entropy``.
    """

    def __init__(self, seed: int):
        self.state = ctypes.c_uint32((seed | 1) & 0xFFFFFFFF)

    def uniform(self, count: int, low: float = -1.0, high: float = 1.0) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        lib().nro_uniform(ctypes.addressof(self.state), low, high, count, _ptr(out))
        return out

    def normal(self, count: int, mean: float = 0.0, deviation: float = 1.0) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        lib().nro_normal(ctypes.addressof(self.state), mean, deviation, count, _ptr(out))
        return out


def random(count: int, seed: int) -> np.ndarray:
    """support::random (tests/support/mod.rs:41-48): uniform(-1, 1) from seed|1."""
    return Stream(seed).uniform(count)


def payload_bytes(element: int, elements: int) -> int:
    return int(lib().nro_payload_bytes(element, elements))


def pack(element: int, values: np.ndarray) -> np.ndarray:
    values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    out = np.empty(int(lib().nro_packed_bytes(element, values.size)), dtype=np.uint8)
    if lib().nro_pack(element, _ptr(values), values.size, _ptr(out)):
        raise ValueError(f"element {element} is not a block format the oracle packs")
    return out


def unpack(element: int, count: int, data: np.ndarray) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    need = payload_bytes(element, count)
    if data.size < need:
        raise ValueError(f"unpacking {count} numbers out of {data.size} bytes where they pack {need}")
    out = np.empty(count, dtype=np.float32)
    if lib().nro_unpack(element, count, _ptr(data), _ptr(out)):
        raise ValueError(f"element {element} is not a block format the oracle unpacks")
    return out


def pack_rows(element: int, weight: np.ndarray) -> np.ndarray:
    """Pack an [N, K] matrix the way a GGUF stores it: K contiguous, row after row."""
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    n, k = weight.shape
    per = 32 if element == Q8_0 else 1 if element in (HALF, BFLOAT16) else 256
    if k % per:
        raise ValueError(f"rows of {k} numbers do not fill whole blocks of {per}")
    return pack(element, weight.reshape(-1))[: payload_bytes(element, n * k)]


def fetch(element: int, data: np.ndarray, at: int) -> float:
    return float(lib().nro_fetch(element, _ptr(np.ascontiguousarray(data)), at))


def op_apply(op: int, a: float, b: float = 0.0) -> float:
    return float(lib().nro_op_apply(op, a, b))


def _steps(chain: Sequence[tuple] | None):
    """chain: sequence of (op, operand ndarray or None, swapped) -> ctypes array + keepalive."""
    chain = list(chain or [])
    keep = []
    arr = (_Step * max(1, len(chain)))()
    for i, step in enumerate(chain):
        op, operand = step[0], step[1]
        swapped = bool(step[2]) if len(step) > 2 else False
        arr[i].op, arr[i].swapped = op, int(swapped)
        if operand is None:
            arr[i].operand, arr[i].row_stride, arr[i].col_stride = None, 0, 0
        else:
            operand = np.ascontiguousarray(operand, dtype=np.float32)
            keep.append(operand)
            if operand.ndim == 1:  # a row vector broadcast over rows
                rs, cs = 0, (1 if operand.shape[0] > 1 else 0)
            else:
                rs = operand.shape[1] if operand.shape[0] > 1 else 0
                cs = 1 if operand.shape[1] > 1 else 0
            arr[i].operand, arr[i].row_stride, arr[i].col_stride = _ptr(operand), rs, cs
    return arr, len(chain), keep


def linear(element: int, packed: np.ndarray, n: int, k: int, x: np.ndarray, chain=None, threads: int = 1,
           bf16: bool = False) -> np.ndarray:
    """out[r, c] = chain(sum_k unpack(W)[c, k] * x[r, k]) in the reference tests' order
    (crates/neura-runtime/tests/runtime.rs:72-83); bf16=True rounds both operands to bf16 first."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    if packed.size < payload_bytes(element, n * k):
        raise ValueError("the packed weight is shorter than its shape")
    out = np.empty((x.shape[0], n), dtype=np.float32)
    arr, count, keep = _steps(chain)
    fn = lib().nro_linear_bf16 if bf16 else lib().nro_linear
    rc = fn(element, _ptr(packed), n, k, _ptr(x), x.shape[0], k, _ptr(out), n, arr, count, threads)
    if rc:
        raise ValueError("the oracle refused the product")
    del keep
    return out


def matmul_f32(weight: np.ndarray, x: np.ndarray, threads: int = 1) -> np.ndarray:
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    n, k = weight.shape
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    out = np.empty((x.shape[0], n), dtype=np.float32)
    lib().nro_matmul_f32(_ptr(weight), n, k, _ptr(x), x.shape[0], _ptr(out), threads)
    return out


def rms_norm(x: np.ndarray, weight: np.ndarray | None, floor: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, width = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    lib().nro_rms_norm(_ptr(x), None if w is None else _ptr(w), floor, rows, width, _ptr(out))
    return out


def rope(x: np.ndarray, position: np.ndarray, base: float) -> np.ndarray:
    """x [rows, heads, width] turned in place semantics (a copy is returned)."""
    out = np.array(x, dtype=np.float32, order="C", copy=True)
    rows, heads, width = out.shape
    pos = np.ascontiguousarray(position, dtype=np.uint32)
    lib().nro_rope(_ptr(out), _ptr(pos), base, rows, heads, width)
    return out


def attend(q: np.ndarray, keys: np.ndarray, values: np.ndarray, count: np.ndarray, scale: float) -> np.ndarray:
    """q [batch, heads, width]; keys/values [batch, key_heads, capacity, width]; count[b] live positions."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    keys = np.ascontiguousarray(keys, dtype=np.float32)
    values = np.ascontiguousarray(values, dtype=np.float32)
    batch, heads, width = q.shape
    _, key_heads, capacity, _ = keys.shape
    cnt = np.ascontiguousarray(count, dtype=np.uint32)
    out = np.empty_like(q)
    lib().nro_attend(_ptr(q), _ptr(keys), _ptr(values), _ptr(cnt), scale, batch, heads, key_heads, capacity, width,
                     _ptr(out))
    return out


def argmax(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, width = x.reshape(-1, x.shape[-1]).shape
    out = np.empty(rows, dtype=np.uint32)
    lib().nro_argmax(_ptr(x), rows, width, _ptr(out))
    return out


def embed(element: int, packed: np.ndarray, width: int, tokens: np.ndarray) -> np.ndarray:
    tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
    out = np.empty((tokens.size, width), dtype=np.float32)
    if lib().nro_embed(element, _ptr(np.ascontiguousarray(packed, dtype=np.uint8)), width, _ptr(tokens), tokens.size,
                       _ptr(out)):
        raise ValueError("the oracle refused the gather")
    return out
