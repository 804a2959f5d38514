"""Host-side mirror of the reference's runtime surface for the quantized-linear path.

The reference drives this path through ``Runtime::{open, load, write, run, read}``
(crates/neura-runtime/src/runtime.rs:183,356,1020,833,1064) with weights poured
verbatim from a GGUF (crates/neura-runtime/src/store.rs:77-157) and products
declared by ``Graph::matmul`` over ``decoder::matrix`` parameters
(crates/neura-graph/src/op.rs:17, crates/neura-decoder/src/parameter.rs:5-41).
This module keeps those names and argument meanings over the C ABI of
``libneura_cuda``; host contract violations raise ``NeuraCudaError`` with the
library's sentence where the reference panics with one.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import NcStep, NcWeight

SINGLE, HALF, BFLOAT16, Q8_0, Q4K, Q5K, Q6K, Q3K = 0, 1, 2, 8, 9, 10, 11, 12
GGUF_ONLY = (HALF, BFLOAT16, Q5K, Q6K, Q3K)   # multiplied where the GGUF left them; Q8_0 and Q4K are sealed
LAYOUT_GGUF, LAYOUT_TILED, LAYOUT_TILED_PAIR = 0, 1, 2

# neura-pointwise op codes (crates/neura-pointwise/src/op.rs:141-170)
ADD, MUL, SUB, DIV, MAXIMUM, MINIMUM, RELU, SQRT, RECIP, EXP = range(10)
LOG, TANH, SIGMOID, NEG, ABS, IDENTITY, SIN, COS, POW, FLOOR, GELU, SILU = range(10, 22)

_BLOCK = {Q8_0: (32, 34), Q4K: (256, 144), Q6K: (256, 210), Q5K: (256, 176), Q3K: (256, 110), HALF: (1, 2), BFLOAT16: (1, 2)}


class NeuraCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


def _check(code: int) -> None:
    if code != 0:
        raise NeuraCudaError(code, _lib.load().neura_cuda_last_error().decode("utf-8", "replace"))


def payload_bytes(element: int, elements: int) -> int:
    """Element::payload_bytes (crates/neura-abi/src/element.rs:231-241)."""
    return int(_lib.load().neura_cuda_payload_bytes(element, elements))


NO_SLOT = 0xFFFFFFFF   # NC_NO_SLOT


@dataclass
class DeviceTensor:
    """A run of f32 (or raw bytes) in device memory owned by a Runtime."""
    ptr: int
    nbytes: int
    shape: tuple

    @property
    def rows(self) -> int:
        return int(np.prod(self.shape[:-1])) if len(self.shape) > 1 else 1


@dataclass
class Weight:
    """A sealed [n, k] block-quantised matrix: what ``decoder::matrix`` declares and ``load`` pours."""
    ptr: int
    element: int
    layout: int
    n: int
    k: int
    nbytes: int

    def record(self) -> NcWeight:
        return NcWeight(self.ptr, self.element, self.layout, self.n, self.k)


@dataclass
class Step:
    """One epilogue step (StepRecord, crates/neura-abi/src/record.rs:72-76)."""
    op: int
    operand: Optional[DeviceTensor] = None
    swapped: bool = False
    row_stride: Optional[int] = None
    col_stride: Optional[int] = None


class Runtime:
    """One GPU, one stream of work: the role of neura_runtime::Runtime for this path."""

    def __init__(self, device: int = 0, stream: int = 0):
        self._lib = _lib.load()
        handle = ctypes.c_void_p()
        _check(self._lib.neura_cuda_open(device, ctypes.byref(handle)))
        self._ctx = handle
        self.device = device
        self.stream = ctypes.c_void_p(stream)
        self._owned: list[int] = []

    # -- lifetime ---------------------------------------------------------------
    def close(self) -> None:
        if self._ctx:
            for ptr in self._owned:
                self._lib.neura_cuda_free(self._ctx, ctypes.c_void_p(ptr))
            self._owned.clear()
            self._lib.neura_cuda_close(self._ctx)
            self._ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- memory -----------------------------------------------------------------
    def alloc(self, nbytes: int) -> int:
        out = ctypes.c_void_p()
        _check(self._lib.neura_cuda_alloc(self._ctx, nbytes, ctypes.byref(out)))
        self._owned.append(out.value)
        return out.value

    def free(self, ptr: int) -> None:
        self._owned.remove(ptr)
        _check(self._lib.neura_cuda_free(self._ctx, ctypes.c_void_p(ptr)))

    def tensor(self, *shape: int) -> DeviceTensor:
        nbytes = int(np.prod(shape)) * 4
        return DeviceTensor(self.alloc(nbytes), nbytes, tuple(shape))

    def write(self, tensor: DeviceTensor, values: np.ndarray) -> None:
        """Runtime::write (runtime.rs:1020): host numbers into a device value."""
        values = np.ascontiguousarray(values)
        if values.nbytes != tensor.nbytes:
            raise ValueError(f"writing {values.nbytes} bytes into a value of {tensor.nbytes}")
        _check(self._lib.neura_cuda_write(self._ctx, self.stream, ctypes.c_void_p(tensor.ptr),
                                          ctypes.c_void_p(values.ctypes.data), values.nbytes))
        self.sync()  # `values` may be pageable and short-lived

    def read(self, tensor: DeviceTensor, dtype=np.float32) -> np.ndarray:
        """Runtime::read (runtime.rs:1064): blocking readback."""
        out = np.empty(tensor.nbytes // np.dtype(dtype).itemsize, dtype=dtype)
        _check(self._lib.neura_cuda_read(self._ctx, self.stream, ctypes.c_void_p(out.ctypes.data),
                                         ctypes.c_void_p(tensor.ptr), tensor.nbytes))
        self.sync()
        return out.reshape(tensor.shape) if dtype == np.float32 else out

    def sync(self) -> None:
        _check(self._lib.neura_cuda_sync(self._ctx, self.stream))

    def set_wait_limit(self, nanoseconds: int) -> None:
        """How long a kernel waits for another party (a peer's flag, the grid barrier) before it gives up."""
        _check(self._lib.neura_cuda_set_wait_limit(self._ctx, nanoseconds))

    def memory(self) -> tuple:
        """(free, total) bytes of the GPU."""
        free, total = ctypes.c_uint64(), ctypes.c_uint64()
        _check(self._lib.neura_cuda_memory(self._ctx, ctypes.byref(free), ctypes.byref(total)))
        return free.value, total.value

    def reserve(self, rows: int, n: int, k: int) -> None:
        _check(self._lib.neura_cuda_reserve(self._ctx, rows, n, k))

    def reserve_bf16(self, rows: int, k: int) -> None:
        """Sizes what ``linear_bf16`` keeps between its kernels for up to ``rows`` rows of ``k`` activations."""
        _check(self._lib.neura_cuda_reserve_bf16(self._ctx, rows, k))

    def reserve_decoder(self, rows: int, heads: int, key_heads: int, width: int, capacity: int) -> None:
        _check(self._lib.neura_cuda_reserve_decoder(self._ctx, rows, heads, key_heads, width, capacity))

    @property
    def launches(self) -> int:
        return int(self._lib.neura_cuda_launches(self._ctx))

    # -- weights ----------------------------------------------------------------
    def upload(self, data: np.ndarray) -> DeviceTensor:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        t = DeviceTensor(self.alloc(max(16, data.nbytes)), data.nbytes, (data.nbytes,))
        _check(self._lib.neura_cuda_write(self._ctx, self.stream, ctypes.c_void_p(t.ptr),
                                          ctypes.c_void_p(data.ctypes.data), data.nbytes))
        self.sync()
        return t

    def load(self, element: int, n: int, k: int, gguf_bytes: np.ndarray, seal: bool = True) -> Weight:
        """Runtime::load for one tensor: pours the GGUF payload verbatim (store.rs:131-135)
        and seals it into the tiled layout.  The GGUF shape contract is decoder::matrix's:
        ne[0] = k (columns), ne[1] = n (rows) (crates/neura-decoder/src/parameter.rs:7-13)."""
        if element not in _BLOCK:
            raise NeuraCudaError(-1, f"element {element} is not a block format this path loads")
        per, _ = _BLOCK[element]
        if k % per:
            raise NeuraCudaError(-1, f"rows of {k} numbers do not fill whole blocks of {per}")
        need = payload_bytes(element, n * k)
        data = np.ascontiguousarray(gguf_bytes).view(np.uint8).reshape(-1)
        if data.size < need:
            raise NeuraCudaError(-1, f"a [{n}, {k}] tensor packs {need} bytes and the source holds {data.size}")
        raw = self.upload(data[:need])
        if not seal or element in GGUF_ONLY:   # these weights are multiplied where the GGUF left them
            return Weight(raw.ptr, element, LAYOUT_GGUF, n, k, need)
        sealed = self.seal_device(element, n, k, raw.ptr)
        self.sync()
        self.free(raw.ptr)
        return sealed

    def sealed_bytes(self, element: int, n: int, k: int) -> int:
        return int(self._lib.neura_cuda_sealed_bytes(element, n, k))

    def seal_device(self, element: int, n: int, k: int, gguf_ptr: int, dst: Optional[int] = None) -> Weight:
        """Seals a GGUF tensor already on the device; into ``dst`` if given (a caller that lays
        several tensors of the same ``k`` end to end, each a multiple of 32 rows, gets one
        weight of their rows stacked, e.g. q, k and v)."""
        nbytes = self.sealed_bytes(element, n, k)
        if dst is None:
            dst = self.alloc(nbytes)
        _check(self._lib.neura_cuda_weight_seal(self._ctx, self.stream, element, n, k,
                                                ctypes.c_void_p(gguf_ptr), ctypes.c_void_p(dst)))
        return Weight(dst, element, LAYOUT_TILED, n, k, nbytes)

    def seal_pair_device(self, element: int, n: int, k: int, gate_ptr: int, up_ptr: int) -> Weight:
        """Seals the gate and up tensors of an MLP (both GGUF [n, k], on the device) as one paired weight."""
        nbytes = int(self._lib.neura_cuda_sealed_pair_bytes(element, n, k))
        dst = self.alloc(nbytes)
        _check(self._lib.neura_cuda_weight_seal_pair(self._ctx, self.stream, element, n, k, ctypes.c_void_p(gate_ptr),
                                                     ctypes.c_void_p(up_ptr), ctypes.c_void_p(dst)))
        return Weight(dst, element, LAYOUT_TILED_PAIR, n, k, nbytes)

    def load_pair(self, element: int, n: int, k: int, gate_bytes: np.ndarray, up_bytes: np.ndarray) -> Weight:
        """``load`` for the gate and up projections of an MLP: a product with the result is silu(gate x) * (up x)."""
        gate = self.load(element, n, k, gate_bytes, seal=False)
        up = self.load(element, n, k, up_bytes, seal=False)
        weight = self.seal_pair_device(element, n, k, gate.ptr, up.ptr)
        self.sync()
        self.free(gate.ptr)
        self.free(up.ptr)
        return weight

    def quantize_device(self, element: int, src_ptr: int, elements: int, dst_ptr: int) -> None:
        _check(self._lib.neura_cuda_quantize(self._ctx, self.stream, element, ctypes.c_void_p(src_ptr), elements,
                                             ctypes.c_void_p(dst_ptr)))

    def dequant(self, weight: Weight) -> np.ndarray:
        """unpack (crates/neura-precision/src/lib.rs:25) run on the device: [n, k] f32."""
        out = self.tensor(weight.n, weight.k)
        rec = weight.record()
        _check(self._lib.neura_cuda_dequant(self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(out.ptr)))
        values = self.read(out)
        self.free(out.ptr)
        return values

    def quantize(self, element: int, values: np.ndarray) -> np.ndarray:
        """pack (crates/neura-precision/src/lib.rs:5) run on the device: GGUF block bytes."""
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        src = self.tensor(values.size)
        self.write(src, values)
        nbytes = payload_bytes(element, values.size)
        dst = DeviceTensor(self.alloc(nbytes), nbytes, (nbytes,))
        _check(self._lib.neura_cuda_quantize(self._ctx, self.stream, element, ctypes.c_void_p(src.ptr),
                                             values.size, ctypes.c_void_p(dst.ptr)))
        out = self.read(dst, dtype=np.uint8)
        self.free(src.ptr)
        self.free(dst.ptr)
        return out

    # -- the product ------------------------------------------------------------
    @staticmethod
    def _steps(chain: Optional[Sequence[Step]], n: int):
        chain = list(chain or [])
        arr = (NcStep * max(1, len(chain)))()
        for i, step in enumerate(chain):
            arr[i].op = step.op
            arr[i].swapped = int(step.swapped)
            if step.operand is None:
                arr[i].operand_dev, arr[i].row_stride, arr[i].col_stride = None, 0, 0
                continue
            shape = step.operand.shape
            rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
            cols = shape[-1]
            if cols not in (1, n):
                raise NeuraCudaError(-1, f"an operand of {cols} columns does not broadcast over {n}")
            arr[i].operand_dev = step.operand.ptr
            arr[i].row_stride = step.row_stride if step.row_stride is not None else (cols if rows > 1 else 0)
            arr[i].col_stride = step.col_stride if step.col_stride is not None else (1 if cols > 1 else 0)
        return arr, len(chain)

    def linear(self, weight: Weight, x: DeviceTensor, out: DeviceTensor, chain: Optional[Sequence[Step]] = None,
               rows: Optional[int] = None) -> None:
        """graph.matmul(x, permute(W)) plus the fused chain, on device values (asynchronous)."""
        rows = rows if rows is not None else x.rows
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear(self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(x.ptr), rows,
                                           x.shape[-1], ctypes.c_void_p(out.ptr), out.shape[-1], arr, count))

    def linear_bf16(self, weight: Weight, x: DeviceTensor, out: DeviceTensor,
                    chain: Optional[Sequence[Step]] = None, rows: Optional[int] = None) -> None:
        """The prefill product on the tensor cores: bf16 operands, f32 accumulation (asynchronous)."""
        rows = rows if rows is not None else x.rows
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear_bf16(self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(x.ptr), rows,
                                                x.shape[-1], ctypes.c_void_p(out.ptr), out.shape[-1], arr, count))

    def linear_static(self, weight: Weight, x: DeviceTensor, out: DeviceTensor,
                      chain: Optional[Sequence[Step]] = None, rows: Optional[int] = None) -> None:
        """``linear`` for callers that may not allocate on the device (a frame-budgeted game
        loop, a host engine that owns the device heap): up to 4 rows, scratch from a fixed
        array inside the library instead of the context's growable regions."""
        rows = rows if rows is not None else x.rows
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear_static(self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(x.ptr),
                                                  rows, x.shape[-1], ctypes.c_void_p(out.ptr), out.shape[-1], arr,
                                                  count))

    def stage(self, x: DeviceTensor, element: int, rows: Optional[int] = None, k: Optional[int] = None) -> None:
        """First half of ``linear``: rewrites up to 16 activation rows for the MMA kernels."""
        rows = rows if rows is not None else x.rows
        k = k if k is not None else x.shape[-1]
        _check(self._lib.neura_cuda_stage(self._ctx, self.stream, ctypes.c_void_p(x.ptr), rows, x.shape[-1], k, element))

    def stage_window(self, x: DeviceTensor, element: int, k: int, lo: int, hi: int, rows: Optional[int] = None) -> None:
        """``stage`` for a row-parallel shard: ``x`` holds elements [lo, hi) of a K axis of ``k``."""
        rows = rows if rows is not None else x.rows
        _check(self._lib.neura_cuda_stage_window(self._ctx, self.stream, ctypes.c_void_p(x.ptr), rows, x.shape[-1], k,
                                                 element, lo, hi))

    def linear_staged(self, weight: Weight, out: DeviceTensor, chain: Optional[Sequence[Step]] = None,
                      out_ptr: Optional[int] = None, out_stride: Optional[int] = None) -> None:
        """Second half of ``linear``: the staged rows times ``weight``."""
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear_staged(
            self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(out_ptr if out_ptr is not None else out.ptr),
            out_stride if out_stride is not None else out.shape[-1], arr, count))

    def staging_select(self, slot: int) -> None:
        """Which of the context's three staged forms ``stage`` writes and the staged products read."""
        _check(self._lib.neura_cuda_staging_select(self._ctx, slot))

    def linear_staged_then(self, weight: Weight, out: DeviceTensor, chain: Optional[Sequence[Step]] = None,
                           normed: bool = False, floor: float = 0.0, then_slot: Optional[int] = None,
                           gain: Optional[DeviceTensor] = None, squares: bool = False) -> None:
        """``linear_staged`` (1 or 2 rows) that applies the rms_norm scalar of its input when the input was staged
        with a norm's gain (``normed``), and whose epilogue stages its output rows into ``then_slot`` for the next
        product, multiplied by ``gain`` and leaving their sums of squares (``squares``)."""
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear_staged_then(
            self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(out.ptr), out.shape[-1], arr, count,
            1 if normed else 0, floor, NO_SLOT if then_slot is None else then_slot,
            ctypes.c_void_p(gain.ptr) if gain is not None else None, 1 if squares else 0))

    def linear_staged_fused(self, weight: Weight, out: DeviceTensor, chain: Optional[Sequence[Step]] = None,
                            normed: bool = False, floor: float = 0.0, reduce=None, then_slot: Optional[int] = None,
                            window: Optional[tuple] = None, gain: Optional[DeviceTensor] = None,
                            squares: bool = False) -> None:
        """``linear_staged_then`` for a tensor-parallel rank: ``window`` = (k, lo, hi) places the output rows on the K
        axis of the row-parallel product that reads them, ``reduce`` (a communicator handle) makes the rows the sum
        over the ranks, exchanged chunk by chunk in the product's epilogue before they are staged."""
        from ._lib import NcThen

        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        k, lo, hi = window if window is not None else (0, 0, 0)
        then = NcThen(NO_SLOT if then_slot is None else then_slot, k, lo, hi, gain.ptr if gain is not None else None,
                      1 if squares else 0)
        _check(self._lib.neura_cuda_linear_staged_fused(
            self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(out.ptr), out.shape[-1], arr, count,
            1 if normed else 0, floor, reduce, ctypes.byref(then)))

    # -- the steps either side of the products ---------------------------------------
    def tensor_u32(self, count: int) -> DeviceTensor:
        return DeviceTensor(self.alloc(count * 4), count * 4, (count,))

    def rms_norm_stage(self, x: DeviceTensor, weight: Optional[DeviceTensor], floor: float, element: int,
                       normed: Optional[DeviceTensor] = None, rows: Optional[int] = None,
                       k: Optional[int] = None) -> None:
        """decoder::rms (crates/neura-decoder/src/op.rs:3-5) fused with ``stage`` of its result."""
        rows = rows if rows is not None else x.rows
        k = k if k is not None else x.shape[-1]
        _check(self._lib.neura_cuda_rms_norm_stage(
            self._ctx, self.stream, ctypes.c_void_p(x.ptr), rows, x.shape[-1], k,
            ctypes.c_void_p(weight.ptr) if weight is not None else None, floor, element,
            ctypes.c_void_p(normed.ptr) if normed is not None else None,
            normed.shape[-1] if normed is not None else 0))

    def rms_norm(self, x: DeviceTensor, weight: Optional[DeviceTensor], floor: float, out: DeviceTensor,
                 rows: Optional[int] = None, k: Optional[int] = None) -> None:
        """decoder::rms (crates/neura-decoder/src/op.rs:3-5) alone: f32 rows out, any number of rows."""
        rows = rows if rows is not None else x.rows
        k = k if k is not None else x.shape[-1]
        _check(self._lib.neura_cuda_rms_norm(self._ctx, self.stream, ctypes.c_void_p(x.ptr), rows, x.shape[-1], k,
                                             ctypes.c_void_p(weight.ptr) if weight is not None else None, floor,
                                             ctypes.c_void_p(out.ptr), out.shape[-1]))

    def rope_cache(self, qkv: DeviceTensor, position: DeviceTensor, base: float, heads: int, key_heads: int,
                   width: int, capacity: int, keys: DeviceTensor, values: DeviceTensor,
                   batch: Optional[int] = None) -> None:
        """decoder::partial over the full width + Cache::write (crates/neura-decoder/src/rope.rs:3-12, cache.rs:267-310)."""
        batch = batch if batch is not None else qkv.rows
        _check(self._lib.neura_cuda_rope_cache(self._ctx, self.stream, ctypes.c_void_p(qkv.ptr), qkv.shape[-1],
                                               ctypes.c_void_p(position.ptr), base, batch, heads, key_heads, width,
                                               capacity, ctypes.c_void_p(keys.ptr), ctypes.c_void_p(values.ptr)))

    def attend(self, q: DeviceTensor, keys: DeviceTensor, values: DeviceTensor, position: DeviceTensor, scale: float,
               heads: int, key_heads: int, width: int, capacity: int, out: DeviceTensor,
               batch: Optional[int] = None) -> None:
        """Cache::attend (crates/neura-decoder/src/cache.rs:311-406) for one new row per sequence."""
        batch = batch if batch is not None else q.rows
        _check(self._lib.neura_cuda_attend(self._ctx, self.stream, ctypes.c_void_p(q.ptr), q.shape[-1],
                                           ctypes.c_void_p(keys.ptr), ctypes.c_void_p(values.ptr),
                                           ctypes.c_void_p(position.ptr), scale, batch, heads, key_heads, width,
                                           capacity, ctypes.c_void_p(out.ptr), out.shape[-1]))

    def rope_cache_rows(self, qkv: DeviceTensor, position: DeviceTensor, base: float, rows: int, heads: int,
                        key_heads: int, width: int, capacity: int, keys_ptr: int, values_ptr: int) -> None:
        """``rope_cache`` for a chunk of one sequence's prompt: ``keys_ptr`` / ``values_ptr`` are that sequence's cache."""
        _check(self._lib.neura_cuda_rope_cache_rows(self._ctx, self.stream, ctypes.c_void_p(qkv.ptr), qkv.shape[-1],
                                                    ctypes.c_void_p(position.ptr), base, rows, heads, key_heads, width,
                                                    capacity, ctypes.c_void_p(keys_ptr), ctypes.c_void_p(values_ptr)))

    def attend_rows(self, q: DeviceTensor, keys_ptr: int, values_ptr: int, position: DeviceTensor, scale: float,
                    rows: int, heads: int, key_heads: int, width: int, capacity: int, out: DeviceTensor) -> None:
        """``attend`` for a chunk of one sequence's prompt: row i attends to slots 0..position[i] of that sequence."""
        _check(self._lib.neura_cuda_attend_rows(self._ctx, self.stream, ctypes.c_void_p(q.ptr), q.shape[-1],
                                                ctypes.c_void_p(keys_ptr), ctypes.c_void_p(values_ptr),
                                                ctypes.c_void_p(position.ptr), scale, rows, heads, key_heads, width,
                                                capacity, ctypes.c_void_p(out.ptr), out.shape[-1]))

    def rope_table(self, position: DeviceTensor, base: float, width: int, table: DeviceTensor,
                   batch: Optional[int] = None) -> None:
        """The step's RoPE angles: table [batch, width / 2, 2] = (cosine, sine) of every sequence's position."""
        batch = batch if batch is not None else position.shape[0]
        _check(self._lib.neura_cuda_rope_table(self._ctx, self.stream, ctypes.c_void_p(position.ptr), base, batch, width,
                                               ctypes.c_void_p(table.ptr)))

    def rope_attend(self, qkv: DeviceTensor, position: DeviceTensor, table: DeviceTensor, scale: float, heads: int,
                    key_heads: int, width: int, capacity: int, keys: DeviceTensor, values: DeviceTensor,
                    out: DeviceTensor, batch: Optional[int] = None) -> None:
        """``rope_cache`` and ``attend`` as one launch: ``qkv`` holds the un-turned rows and stays as it is;
        ``table`` holds the step's angles (``rope_table``)."""
        batch = batch if batch is not None else qkv.rows
        _check(self._lib.neura_cuda_rope_attend(self._ctx, self.stream, ctypes.c_void_p(qkv.ptr), qkv.shape[-1],
                                                ctypes.c_void_p(position.ptr), ctypes.c_void_p(table.ptr), scale, batch, heads, key_heads,
                                                width, capacity, ctypes.c_void_p(keys.ptr), ctypes.c_void_p(values.ptr),
                                                ctypes.c_void_p(out.ptr), out.shape[-1]))

    def argmax(self, x: DeviceTensor, out: DeviceTensor, rows: Optional[int] = None) -> None:
        rows = rows if rows is not None else x.rows
        _check(self._lib.neura_cuda_argmax(self._ctx, self.stream, ctypes.c_void_p(x.ptr), rows, x.shape[-1],
                                           x.shape[-1], ctypes.c_void_p(out.ptr)))

    def argmax_segments(self, x_ptr: int, rows: int, width: int, stride: int, segment: int, segment_stride: int,
                        out: DeviceTensor) -> None:
        """argmax over rows gathered in segments from the ranks of a tensor-parallel group."""
        _check(self._lib.neura_cuda_argmax_segments(self._ctx, self.stream, ctypes.c_void_p(x_ptr), rows, width, stride,
                                                    segment, segment_stride, ctypes.c_void_p(out.ptr)))

    def embed(self, table: Weight, tokens: DeviceTensor, out: DeviceTensor, rows: Optional[int] = None) -> None:
        rows = rows if rows is not None else out.rows
        rec = table.record()
        _check(self._lib.neura_cuda_embed(self._ctx, self.stream, ctypes.byref(rec), ctypes.c_void_p(tokens.ptr), rows,
                                          ctypes.c_void_p(out.ptr), out.shape[-1]))

    def advance(self, position: DeviceTensor, by: int = 1) -> None:
        _check(self._lib.neura_cuda_advance(self._ctx, self.stream, ctypes.c_void_p(position.ptr), position.shape[0], by))

    def load_stacked(self, element: int, k: int, parts: Sequence[tuple]) -> Weight:
        """Several GGUF tensors of the same ``k`` sealed end to end as one weight of their rows
        stacked (q, k and v share their activations, so one product serves all three).
        ``parts`` = [(n, gguf_bytes), ...], every n a multiple of 32."""
        total = sum(n for n, _ in parts)
        base = self.alloc(self.sealed_bytes(element, total, k))
        at = base
        for n, data in parts:
            if n % 32:
                raise NeuraCudaError(-1, f"a stacked part of {n} rows does not fill tiles of 32")
            raw = self.load(element, n, k, data, seal=False)
            self.seal_device(element, n, k, raw.ptr, at)
            self.sync()
            self.free(raw.ptr)
            at += self.sealed_bytes(element, n, k)
        return Weight(base, element, LAYOUT_TILED, total, k, at - base)

    # -- recorded programs --------------------------------------------------------
    def new_stream(self) -> int:
        out = ctypes.c_void_p()
        _check(self._lib.neura_cuda_stream_create(self._ctx, ctypes.byref(out)))
        return out.value

    def use_stream(self, stream: int) -> None:
        self.stream = ctypes.c_void_p(stream)

    def capture_begin(self) -> None:
        """Runtime::compile (runtime.rs:528): start recording the calls that follow."""
        _check(self._lib.neura_cuda_capture_begin(self._ctx, self.stream))

    def capture_end(self) -> int:
        out = ctypes.c_void_p()
        _check(self._lib.neura_cuda_capture_end(self._ctx, self.stream, ctypes.byref(out)))
        return out.value

    def run(self, program: int) -> None:
        """Runtime::run (runtime.rs:833): replay a recorded program (asynchronous)."""
        _check(self._lib.neura_cuda_program_run(self._ctx, self.stream, ctypes.c_void_p(program)))

    def program_free(self, program: int) -> None:
        _check(self._lib.neura_cuda_program_free(self._ctx, ctypes.c_void_p(program)))

    def linear_host(self, weight: Weight, x: np.ndarray, chain: Optional[Sequence[Step]] = None,
                    out: Optional[np.ndarray] = None) -> np.ndarray:
        """write + run + read in one call: host activations in, host results out."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, weight.k)
        if out is None:
            out = np.empty((x.shape[0], weight.n), dtype=np.float32)
        arr, count = self._steps(chain, weight.n)
        rec = weight.record()
        _check(self._lib.neura_cuda_linear_host(self._ctx, self.stream, ctypes.byref(rec),
                                                ctypes.c_void_p(x.ctypes.data), x.shape[0],
                                                ctypes.c_void_p(out.ctypes.data), arr, count))
        return out
