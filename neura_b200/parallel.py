"""Tensor-parallel sharding of the decoder's projections over the GPUs of one box.

The reference runs on one device; this split has no counterpart there and is checked against
the single-device result.  Column-parallel projections (q/k/v, gate, up, the head) split their
rows (output features): a rank's share is a contiguous run of GGUF rows, so no block is cut.
Row-parallel projections (attention output, down) split K; a rank keeps the whole Q4_K
super-blocks (or Q8_0 blocks) that cover its K range, stages its activations at their offset
inside them (the rest of K staged as zero, ``Runtime.stage_window``) and the ranks' partial
products are summed by one all-reduce per projection.  The weights are quantised as whole
rows first, so every rank dequantises exactly the values the single-device model does.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np

from .qwen import Config
from .runtime import Q4K, Q8_0, payload_bytes

_BLOCK = {Q8_0: (32, 34), Q4K: (256, 144)}


@dataclass(frozen=True)
class Window:
    """A rank's share of a K axis: elements [lo, hi) of the padded local axis of ``k`` columns,
    which are blocks [first_block, first_block + k / block) of the full axis."""
    k: int
    lo: int
    hi: int
    first_block: int


@dataclass(frozen=True)
class Shard:
    """``attention``: "split" shards the attention block by heads (q/k/v rows, attention output by K, one exchange);
    "whole" keeps it on every rank (each rank computes all heads; only the MLP and the head are split, one exchange a
    layer).  At batch 1 the whole attention block streams 35 MB a layer, which takes a rank less time than its share
    of it plus the exchange, so "whole" is the faster split at every group size measured."""
    config: Config
    world: int
    rank: int
    attention: str = "split"

    def __post_init__(self):
        c, w = self.config, self.world
        if self.attention not in ("split", "whole"):
            raise ValueError(f"the attention block is split or whole, not {self.attention!r}")
        if c.feed_forward % w or c.vocab % w or (not self.whole and (c.heads % w or c.key_heads % w)):
            raise ValueError(f"{c.name} does not split evenly over {w} ranks "
                             f"({c.heads}/{c.key_heads} heads, ff {c.feed_forward}, vocab {c.vocab})")
        for width in (c.feed_forward // w, c.vocab // w) + (() if self.whole else (c.key_width // w,)):
            if width % 32:
                raise ValueError(f"a share of {width} rows does not fill tiles of 32")
        if (not self.whole and (c.query_width // w) % 32) or (c.feed_forward // w) % 32:
            raise ValueError("a share of a K axis starts on a multiple of 32")

    @property
    def whole(self) -> bool:
        return self.attention == "whole"

    # -- shapes of the local model ---------------------------------------------------
    @property
    def heads(self) -> int:
        return self.config.heads if self.whole else self.config.heads // self.world

    @property
    def key_heads(self) -> int:
        return self.config.key_heads if self.whole else self.config.key_heads // self.world

    @property
    def query_width(self) -> int:
        return self.heads * self.config.head_width

    @property
    def key_width(self) -> int:
        return self.key_heads * self.config.head_width

    @property
    def feed_forward(self) -> int:
        return self.config.feed_forward // self.world

    @property
    def vocab(self) -> int:
        return self.config.vocab // self.world

    def rows(self, n: int, whole: bool = False) -> Tuple[int, int]:
        """The run of rows [n0, n1) of a column-parallel projection of ``n`` rows (all of them for a projection the
        ranks keep whole)."""
        if whole:
            return 0, n
        share = n // self.world
        return self.rank * share, (self.rank + 1) * share

    def window(self, k: int, whole: bool = False) -> Window:
        """The share of a row-parallel projection's K axis of ``k`` columns (the whole axis for a projection the ranks
        keep whole)."""
        per = _BLOCK[self.config.element][0]
        if whole:
            return Window(k, 0, k, 0)
        share = k // self.world
        k0, k1 = self.rank * share, (self.rank + 1) * share
        b0, b1 = k0 // per, (k1 + per - 1) // per
        return Window((b1 - b0) * per, k0 - b0 * per, k1 - b0 * per, b0)

    # -- slicing GGUF tensors ------------------------------------------------------------
    def slice_rows(self, packed: np.ndarray, n: int, k: int, whole: bool = False) -> np.ndarray:
        """Rows [n0, n1) of a GGUF [n, k] tensor (a contiguous run of its bytes)."""
        n0, n1 = self.rows(n, whole)
        row = payload_bytes(self.config.element, k)
        return np.ascontiguousarray(packed, dtype=np.uint8)[n0 * row: n1 * row]

    def slice_columns(self, packed: np.ndarray, n: int, k: int, whole: bool = False) -> np.ndarray:
        """The whole blocks that cover this rank's share of K, for every row of a GGUF [n, k] tensor."""
        per, size = _BLOCK[self.config.element]
        window = self.window(k, whole)
        blocks = np.ascontiguousarray(packed, dtype=np.uint8)[: n * (k // per) * size].reshape(n, k // per, size)
        return np.ascontiguousarray(blocks[:, window.first_block: window.first_block + window.k // per]).reshape(-1)

    def local_bytes_per_token(self) -> int:
        """GGUF bytes this rank streams per decoded token (projections and its share of the head)."""
        c = self.config
        e = c.element
        per_layer = (payload_bytes(e, (self.query_width + 2 * self.key_width) * c.hidden)
                     + payload_bytes(e, c.hidden * self.window(c.query_width, self.whole).k)
                     + 2 * payload_bytes(e, self.feed_forward * c.hidden)
                     + payload_bytes(e, c.hidden * self.window(c.feed_forward).k))
        return c.layers * per_layer + payload_bytes(e, self.vocab * c.hidden)


class TorchComm:
    """The two exchanges of a tensor-parallel decode step over torch.distributed (NCCL on the
    GPUs, gloo in the CPU tests), enqueued on the runtime's stream."""

    def __init__(self, world: int, rank: int, device=None, stream=None):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world, self.rank, self.device, self.stream = world, rank, device, stream
        self.views: Dict[int, object] = {}

    def view(self, ptr: int, count: int):
        """A torch view of ``count`` f32 at a device pointer this process owns."""
        key = (ptr, count)
        if key not in self.views:
            torch = self.torch

            class _Span:
                __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3}

            self.views[key] = torch.as_tensor(_Span(), device=self.device)
        return self.views[key]

    def all_reduce(self, ptr: int, count: int) -> None:
        tensor = self.view(ptr, count)
        with self.torch.cuda.stream(self.stream):
            self.dist.all_reduce(tensor)

    def all_reduce_norm_stage(self, ptr: int, rows: int, k: int, weight_ptr: int, floor: float, element: int) -> bool:
        """The all-reduce fused with the rms_norm and staging that follow it; False when this transport has no
        such launch (the caller then issues the three separately)."""
        return False

    def all_gather(self, dst_ptr: int, src_ptr: int, count: int) -> None:
        """dst [world][count] <- every rank's src [count]."""
        dst, src = self.view(dst_ptr, count * self.world), self.view(src_ptr, count)
        with self.torch.cuda.stream(self.stream):
            self.dist.all_gather_into_tensor(dst, src)


class NullComm(TorchComm):
    """No exchange at all: one rank's share of a tensor-parallel step on one GPU, for timing the rank's own chain
    of launches without its peers (the sums it leaves are partial, so the tokens mean nothing)."""

    def __init__(self, world: int, rank: int):
        self.world, self.rank = world, rank

    def all_reduce(self, ptr: int, count: int) -> None:
        pass

    def all_gather(self, dst_ptr: int, src_ptr: int, count: int) -> None:
        pass

    def reduce_handle(self):
        """No communicator: a product that would exchange in its epilogue keeps its own partial sums."""
        return None


def load_decoder_weights(rt, config: Config, packed: Dict[str, np.ndarray], norms: Dict[str, np.ndarray],
                         shard: Shard = None, pair_mlp: bool = True):
    """Runtime::load for a whole decoder: pours the GGUF tensors of ``packed`` (named as a Qwen GGUF
    names them: token_embd.weight, output.weight, blk.N.attn_q/k/v/output.weight, blk.N.ffn_gate/up/
    down.weight) into sealed device weights, the rank's shares only when ``shard`` is given.
    Returns (weights, norms) as ``qwen.Decoder`` takes them."""
    c = config
    e = c.element
    weights, device_norms = {}, {}

    whole_attention = shard is not None and shard.whole

    def rows_of(name: str, n: int, k: int, whole: bool = False):
        data = packed[name]
        if shard is None or whole:
            return n, data
        return n // shard.world, shard.slice_rows(data, n, k)

    def columns_of(name: str, n: int, k: int, whole: bool = False):
        data = packed[name]
        if shard is None or whole:
            return k, data
        return shard.window(k).k, shard.slice_columns(data, n, k)

    for layer in range(c.layers):
        name = lambda part: f"blk.{layer}.{part}.weight"  # noqa: E731
        parts = [rows_of(name("attn_q"), c.query_width, c.hidden, whole_attention),
                 rows_of(name("attn_k"), c.key_width, c.hidden, whole_attention),
                 rows_of(name("attn_v"), c.key_width, c.hidden, whole_attention)]
        weights[name("attn_qkv")] = rt.load_stacked(e, c.hidden, parts)
        k, data = columns_of(name("attn_output"), c.hidden, c.query_width, whole_attention)
        weights[name("attn_output")] = rt.load(e, c.hidden, k, data)
        n, gate = rows_of(name("ffn_gate"), c.feed_forward, c.hidden)
        n, up = rows_of(name("ffn_up"), c.feed_forward, c.hidden)
        if pair_mlp:
            weights[name("ffn_gate_up")] = rt.load_pair(e, n, c.hidden, gate, up)
        else:
            weights[name("ffn_gate")] = rt.load(e, n, c.hidden, gate)
            weights[name("ffn_up")] = rt.load(e, n, c.hidden, up)
        k, data = columns_of(name("ffn_down"), c.hidden, c.feed_forward)
        weights[name("ffn_down")] = rt.load(e, c.hidden, k, data)
    n, data = rows_of("output.weight", c.vocab, c.hidden)
    weights["output.weight"] = rt.load(e, n, c.hidden, data)
    if c.tied_head and shard is None:
        weights["token_embd.weight"] = weights["output.weight"]
    else:  # every rank gathers from the whole table, kept in GGUF order
        weights["token_embd.weight"] = rt.load(e, c.vocab, c.hidden, packed["token_embd.weight"], seal=False)
    for key, value in norms.items():
        device_norms[key] = rt.tensor(value.size)
        rt.write(device_norms[key], value)
    return weights, device_norms


class PeerComm(TorchComm):
    """The same exchanges with the all-reduce done by the library's own one-shot kernel over NVLink
    peer memory (``neura_cuda_allreduce``); torch.distributed only carries the IPC handles at set-up
    and the (rare) logits gather."""

    def __init__(self, rt, world: int, rank: int, max_count: int, device=None, stream=None):
        import ctypes

        from .runtime import _check

        super().__init__(world, rank, device=device, stream=stream)
        self.rt = rt
        handle = (ctypes.c_ubyte * 64)()
        comm = ctypes.c_void_p()
        _check(rt._lib.neura_cuda_comm_create(rt._ctx, max_count, ctypes.byref(comm), handle))
        self.comm = comm
        gathered = [None] * world
        self.dist.all_gather_object(gathered, bytes(handle))
        blob = (ctypes.c_ubyte * (64 * world)).from_buffer_copy(b"".join(gathered))
        _check(rt._lib.neura_cuda_comm_connect(rt._ctx, comm, rank, world, blob))
        self.dist.barrier()

    def all_reduce(self, ptr: int, count: int) -> None:
        import ctypes

        from .runtime import _check

        _check(self.rt._lib.neura_cuda_allreduce(self.rt._ctx, self.rt.stream, self.comm, ctypes.c_void_p(ptr), count))

    def reduce_handle(self):
        """The communicator as ``Runtime.linear_staged_fused`` takes it: the product then adds the ranks' partial
        sums up in its own epilogue."""
        return self.comm

    def all_reduce_norm_stage(self, ptr: int, rows: int, k: int, weight_ptr: int, floor: float, element: int) -> bool:
        import ctypes

        from .runtime import _check

        _check(self.rt._lib.neura_cuda_allreduce_norm_stage(self.rt._ctx, self.rt.stream, self.comm, ctypes.c_void_p(ptr),
                                                            rows, k, ctypes.c_void_p(weight_ptr), floor, element))
        return True
