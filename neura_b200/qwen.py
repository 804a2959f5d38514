"""Qwen2.5-shaped decoders over the quantized-linear path.

The wiring follows the reference's example model (examples/qwen/mlp.rs:29-36,
attention.rs:98-153, model.rs:77-103): every projection is
``graph.matmul(x, permute(W))`` over a ``decoder::matrix`` parameter, the MLP is
``down(silu(gate(x)) * up(x))`` and residual adds ride the products as fused
chain steps.  The shapes are the Qwen2.5 ones the benchmark configurations name
(no delta-net layers, no attention gate).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .runtime import ADD, MUL, SILU, Q4K, Q8_0, DeviceTensor, Runtime, Step, Weight, payload_bytes


@dataclass(frozen=True)
class Config:
    name: str
    layers: int
    hidden: int
    heads: int
    key_heads: int
    head_width: int
    feed_forward: int
    vocab: int
    element: int
    floor: float = 1e-6          # RMSNorm epsilon
    rope_base: float = 1e6
    tied_head: bool = False      # logits against the token embedding (examples/qwen/model.rs:83)

    @property
    def query_width(self) -> int:
        return self.heads * self.head_width

    @property
    def key_width(self) -> int:
        return self.key_heads * self.head_width

    def linears(self) -> List[tuple]:
        """(name, n, k) of the projections of one layer, in call order."""
        return [
            ("attn_q", self.query_width, self.hidden),
            ("attn_k", self.key_width, self.hidden),
            ("attn_v", self.key_width, self.hidden),
            ("attn_output", self.hidden, self.query_width),
            ("ffn_gate", self.feed_forward, self.hidden),
            ("ffn_up", self.feed_forward, self.hidden),
            ("ffn_down", self.hidden, self.feed_forward),
        ]

    def weight_elements(self) -> int:
        per_layer = sum(n * k for _, n, k in self.linears())
        return self.layers * per_layer + self.vocab * self.hidden

    def weight_bytes(self) -> int:
        """GGUF payload bytes one decoded token streams (projections and the head)."""
        return payload_bytes(self.element, self.weight_elements())


QWEN25_05B_Q8 = Config("qwen2.5-0.5b-q8_0", 24, 896, 14, 2, 64, 4864, 151936, Q8_0, tied_head=True)
QWEN25_7B_MLP_Q4K = Config("qwen2.5-7b-q4_k", 28, 3584, 28, 4, 128, 18944, 152064, Q4K)
QWEN25_32B_Q4K = Config("qwen2.5-32b-q4_k", 64, 5120, 40, 8, 128, 27648, 152064, Q4K)

PRESETS: Dict[str, Config] = {c.name: c for c in (QWEN25_05B_Q8, QWEN25_7B_MLP_Q4K, QWEN25_32B_Q4K)}


def scaled(config: Config, layers: int, vocab: Optional[int] = None) -> Config:
    """The same layer shapes with fewer layers (and a smaller vocabulary) for tests."""
    return Config(f"{config.name}-{layers}l", layers, config.hidden, config.heads, config.key_heads,
                  config.head_width, config.feed_forward, vocab or config.vocab, config.element, config.floor,
                  config.rope_base, config.tied_head)


class Decoder:
    """A Qwen2.5-shaped decoder stepping one token per sequence (greedy), on the device.

    Layer wiring after examples/qwen/attention.rs:98-153 and mlp.rs:29-36 without the
    Qwen3.5 extras (no q/k norms, no attention gate, RoPE over the full head width);
    the step is Batch::answer (crates/neura-generate/src/batch.rs:1646-1725): token ids and
    cursors stay on the device, so one recorded program replays per token.

    ``weights``: "token_embd.weight" (any layout; the sealed head when tied), "output.weight",
    per layer "blk.N.attn_qkv.weight" (q, k, v rows stacked), "blk.N.attn_output.weight",
    "blk.N.ffn_gate.weight", "blk.N.ffn_up.weight", "blk.N.ffn_down.weight".
    ``norms``: "blk.N.attn_norm.weight", "blk.N.ffn_norm.weight", "output_norm.weight" (f32 [hidden]).
    """

    def __init__(self, rt: Runtime, config: Config, weights: Dict[str, Weight], norms: Dict[str, DeviceTensor],
                 batch: int = 1, capacity: int = 640, shard=None, comm=None):
        """``shard`` (parallel.Shard) and ``comm`` (parallel.TorchComm) make this one rank of a
        tensor-parallel group: ``weights`` then hold the rank's shares (q/k/v, gate, up and head
        rows; the K blocks of attention output and down that cover its window)."""
        if batch > 16:
            raise ValueError("one decode step carries at most 16 sequences")
        if (shard is None) != (comm is None):
            raise ValueError("a tensor-parallel rank needs both its shard and its communicator")
        self.rt, self.config, self.weights, self.norms = rt, config, weights, norms
        self.batch, self.capacity, self.shard, self.comm = batch, capacity, shard, comm
        c = config
        world = shard.world if shard else 1
        self.heads, self.key_heads = c.heads // world, c.key_heads // world
        self.query_width, self.key_width = self.heads * c.head_width, self.key_heads * c.head_width
        self.feed_forward, self.vocab = c.feed_forward // world, c.vocab // world
        self.tokens = rt.tensor_u32(batch)
        self.position = rt.tensor_u32(batch)
        self.hidden = rt.tensor(batch, c.hidden)
        self.qkv = rt.tensor(batch, self.query_width + 2 * self.key_width)
        self.attended = rt.tensor(batch, self.query_width)
        self.gate = rt.tensor(batch, self.feed_forward)
        self.held = rt.tensor(batch, self.feed_forward)
        self.logits = rt.tensor(batch, self.vocab)
        self.gathered = rt.tensor(world, batch, self.vocab) if shard else None
        cache = batch * self.key_heads * capacity * c.head_width
        self.keys = [rt.tensor(cache) for _ in range(c.layers)]
        self.values = [rt.tensor(cache) for _ in range(c.layers)]
        widest_k = max(c.hidden, self.window(c.feed_forward)[0], self.window(c.query_width)[0])
        rt.reserve(batch, max(self.vocab, 2 * self.feed_forward, c.hidden), widest_k)   # 2x: a sealed gate|up pair
        rt.reserve_decoder(batch, self.heads, self.key_heads, c.head_width, capacity)
        self.program: Optional[int] = None
        self.compiled = None   # the step as one persistent kernel (compile())
        self.fold = False      # True: fold norms and stagings into the products' epilogues (fewer, longer launches)
        self.scale = 1.0 / float(c.head_width) ** 0.5

    def window(self, k: int):
        """(local K, lo, hi) of a row-parallel projection over a K axis of ``k``."""
        if self.shard is None:
            return k, 0, k
        w = self.shard.window(k)
        return w.k, w.lo, w.hi

    def _row_parallel(self, x: DeviceTensor, weight: Weight, k: int, next_norm: DeviceTensor) -> None:
        """hidden += W x over this rank's share of K, summed over the ranks; then the rms_norm that follows
        every such projection (with ``next_norm``) and the staging of its result for the next product."""
        rt, c = self.rt, self.config
        local, lo, hi = self.window(k)
        if self.shard is None:
            rt.stage(x, c.element)
            rt.linear_staged(weight, self.hidden, [Step(ADD, self.hidden)])
            rt.rms_norm_stage(self.hidden, next_norm, c.floor, c.element)
            return
        rt.stage_window(x, c.element, local, lo, hi)
        # rank 0 carries the residual, so the sum over the ranks is hidden + W x on every rank
        rt.linear_staged(weight, self.hidden, [Step(ADD, self.hidden)] if self.shard.rank == 0 else None)
        if not self.comm.all_reduce_norm_stage(self.hidden.ptr, self.batch, c.hidden, next_norm.ptr, c.floor, c.element):
            self.comm.all_reduce(self.hidden.ptr, self.batch * c.hidden)
            rt.rms_norm_stage(self.hidden, next_norm, c.floor, c.element)

    def folded(self) -> bool:
        """Whether the step may fold the norms and stagings into the products' epilogues (``linear_staged_then``):
        one GPU, 1 or 2 sequences, the MLP sealed as a pair."""
        return self.shard is None and self.batch <= 2 and "blk.0.ffn_gate_up.weight" in self.weights and self.fold

    def _step_folded(self) -> None:
        """The step with seven launches a layer instead of ten: the output and down products stage the hidden row
        for the next norm (gain and sums of squares in their epilogues, the scalar applied by the consumer), the
        gate|up product stages its own output for the down product.  Slots: 0 hidden, 1 attended, 2 held."""
        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        rt.staging_select(0)
        rt.embed(w["token_embd.weight"], self.tokens, self.hidden)
        rt.rms_norm_stage(self.hidden, n["blk.0.attn_norm.weight"], c.floor, c.element)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            after = n[f"blk.{layer + 1}.attn_norm.weight"] if layer + 1 < c.layers else n["output_norm.weight"]
            rt.staging_select(0)
            rt.linear_staged_then(w[at("attn_qkv")], self.qkv, normed=layer > 0, floor=c.floor)
            rt.rope_cache(self.qkv, self.position, c.rope_base, self.heads, self.key_heads, c.head_width,
                          self.capacity, self.keys[layer], self.values[layer])
            rt.attend(self.qkv, self.keys[layer], self.values[layer], self.position, self.scale, self.heads,
                      self.key_heads, c.head_width, self.capacity, self.attended)
            rt.staging_select(1)
            rt.stage(self.attended, c.element)
            rt.linear_staged_then(w[at("attn_output")], self.hidden, [Step(ADD, self.hidden)], then_slot=0,
                                  gain=n[at("ffn_norm")], squares=True)
            rt.staging_select(0)
            rt.linear_staged_then(w[at("ffn_gate_up")], self.held, normed=True, floor=c.floor, then_slot=2)
            rt.staging_select(2)
            rt.linear_staged_then(w[at("ffn_down")], self.hidden, [Step(ADD, self.hidden)], then_slot=0, gain=after,
                                  squares=True)
        rt.staging_select(0)
        rt.linear_staged_then(w["output.weight"], self.logits, normed=True, floor=c.floor)
        rt.argmax(self.logits, self.tokens)
        rt.advance(self.position, 1)

    def step(self) -> None:
        if self.folded():
            return self._step_folded()
        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        rt.embed(w["token_embd.weight"], self.tokens, self.hidden)
        rt.rms_norm_stage(self.hidden, n["blk.0.attn_norm.weight"], c.floor, c.element)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            after = n[f"blk.{layer + 1}.attn_norm.weight"] if layer + 1 < c.layers else n["output_norm.weight"]
            rt.linear_staged(w[at("attn_qkv")], self.qkv)
            # (two launches on purpose: the small RoPE launch gives the attention's clusters time to become resident
            # while the product before them drains)
            rt.rope_cache(self.qkv, self.position, c.rope_base, self.heads, self.key_heads, c.head_width,
                          self.capacity, self.keys[layer], self.values[layer])
            rt.attend(self.qkv, self.keys[layer], self.values[layer], self.position, self.scale, self.heads,
                      self.key_heads, c.head_width, self.capacity, self.attended)
            self._row_parallel(self.attended, w[at("attn_output")], c.query_width, n[at("ffn_norm")])
            if at("ffn_gate_up") in w:   # gate and up sealed as a pair: one product, SwiGLU in its epilogue
                rt.linear_staged(w[at("ffn_gate_up")], self.held)
            else:
                rt.linear_staged(w[at("ffn_gate")], self.gate, [Step(SILU)])
                rt.linear_staged(w[at("ffn_up")], self.held, [Step(MUL, self.gate)])
            self._row_parallel(self.held, w[at("ffn_down")], c.feed_forward, after)
        rt.linear_staged(w["output.weight"], self.logits)
        if self.shard is None:
            rt.argmax(self.logits, self.tokens)
        else:
            self.comm.all_gather(self.gathered.ptr, self.logits.ptr, self.batch * self.vocab)
            rt.argmax_segments(self.gathered.ptr, self.batch, c.vocab, self.vocab, self.vocab,
                               self.batch * self.vocab, self.tokens)
        rt.advance(self.position, 1)

    def compile(self) -> None:
        """Runtime::compile for the whole step (crates/neura-runtime/src/runtime.rs:528): lays the step out
        as the phase table of one persistent kernel (``neura_cuda_decoder_compile``); ``run_token`` then
        launches that kernel instead of one kernel per operation.  Single GPU, 1 or 2 sequences, the MLP
        sealed as a gate|up pair."""
        import ctypes

        from ._lib import NcDecoderDesc, NcDecoderLayer
        from .runtime import _check

        if self.shard is not None:
            raise ValueError("the persistent step runs on one GPU")
        c, w, n = self.config, self.weights, self.norms
        layers = (NcDecoderLayer * c.layers)()
        for index in range(c.layers):
            at = lambda name: f"blk.{index}.{name}.weight"  # noqa: E731
            if at("ffn_gate_up") not in w:
                raise ValueError("the persistent step wants the MLP sealed as a gate|up pair")
            layer = layers[index]
            layer.qkv, layer.attn_output = w[at("attn_qkv")].record(), w[at("attn_output")].record()
            layer.gate_up, layer.down = w[at("ffn_gate_up")].record(), w[at("ffn_down")].record()
            layer.attn_norm_dev, layer.ffn_norm_dev = n[at("attn_norm")].ptr, n[at("ffn_norm")].ptr
            layer.keys_dev, layer.values_dev = self.keys[index].ptr, self.values[index].ptr
        desc = NcDecoderDesc(c.layers, c.hidden, c.heads, c.key_heads, c.head_width, c.feed_forward, c.vocab,
                             self.batch, self.capacity, c.floor, c.rope_base, self.scale,
                             w["token_embd.weight"].record(), w["output.weight"].record(), n["output_norm.weight"].ptr,
                             layers, self.tokens.ptr, self.position.ptr, self.logits.ptr)
        handle = ctypes.c_void_p()
        _check(self.rt._lib.neura_cuda_decoder_compile(self.rt._ctx, ctypes.byref(desc), ctypes.byref(handle)))
        self.compiled = handle

    def trace(self):
        """(kinds, nanoseconds) per phase of the last completed persistent step."""
        import ctypes

        import numpy as np

        from .runtime import _check

        self.rt.sync()
        count = ctypes.c_uint32()
        _check(self.rt._lib.neura_cuda_decoder_trace(self.rt._ctx, self.compiled, 0, None, None, ctypes.byref(count)))
        kinds, nanos = np.zeros(count.value, np.uint32), np.zeros(count.value, np.uint64)
        _check(self.rt._lib.neura_cuda_decoder_trace(self.rt._ctx, self.compiled, count.value, kinds.ctypes.data,
                                                     nanos.ctypes.data, ctypes.byref(count)))
        return kinds, nanos

    def release(self) -> None:
        if self.compiled is not None:
            self.rt._lib.neura_cuda_decoder_free(self.rt._ctx, self.compiled)
            self.compiled = None

    def launches_per_token(self) -> int:
        if self.compiled is not None:
            return 1
        if self.folded():
            return self.config.layers * 7 + 5
        paired = "blk.0.ffn_gate_up.weight" in self.weights
        return self.config.layers * (10 if paired else 11) + 5

    def record(self) -> int:
        self.rt.capture_begin()
        try:
            self.step()
        except Exception:
            try:   # leave no capture open behind a refused launch
                self.rt.program_free(self.rt.capture_end())
            except Exception:
                pass
            raise
        self.program = self.rt.capture_end()
        return self.program

    def reset(self) -> None:
        import numpy as np

        self.rt.write(self.position, np.zeros(self.batch, dtype=np.uint32))

    def run_token(self) -> None:
        if self.compiled is not None:
            from .runtime import _check

            _check(self.rt._lib.neura_cuda_decoder_step(self.rt._ctx, self.rt.stream, self.compiled))
        elif self.program is None:
            self.step()
        else:
            self.rt.run(self.program)

    def answer(self, tokens, cursors):
        """One step with the planes' tokens and cursors given by the host, as Batch::answer writes
        them (crates/neura-generate/src/batch.rs:1716-1725); returns the chosen ids [batch]."""
        import numpy as np

        self.rt.write(self.tokens, np.ascontiguousarray(tokens, dtype=np.uint32))
        self.rt.write(self.position, np.ascontiguousarray(cursors, dtype=np.uint32))
        self.run_token()
        return self.rt.read(self.tokens, dtype=np.uint32)

    @classmethod
    def from_gguf(cls, rt: Runtime, source, batch: int = 1, capacity: int = 640, shard=None, comm=None,
                  name: str = None) -> "Decoder":
        """A decoder over the tensors of a GGUF (a path or a parsed ``gguf.Gguf``): the shapes from its
        metadata (examples/qwen/config.rs:22-60), every projection poured and sealed
        (Runtime::load, crates/neura-runtime/src/runtime.rs:356)."""
        from . import gguf as gguf_reader
        from .parallel import load_decoder_weights

        held = gguf_reader.Gguf.open(source) if isinstance(source, str) else source
        config = gguf_reader.read_config(held, name)
        packed, norms = gguf_reader.decoder_tensors(held, config)
        weights, device_norms = load_decoder_weights(rt, config, packed, norms, shard=shard)
        return cls(rt, config, weights, device_norms, batch=batch, capacity=capacity, shard=shard, comm=comm)

    def generate(self, prompts, steps: int):
        """Feeds ``prompts`` [batch, length] one token at a time (every step attends to all the
        tokens before it), then decodes ``steps`` tokens greedily.  Returns [batch, steps] ids."""
        import numpy as np

        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.batch, -1)
        self.reset()
        out = np.zeros((self.batch, steps), dtype=np.uint32)
        for at in range(prompts.shape[1]):
            self.rt.write(self.tokens, prompts[:, at].copy())
            self.run_token()
        out[:, 0] = self.rt.read(self.tokens, dtype=np.uint32)
        for at in range(1, steps):
            self.run_token()
            out[:, at] = self.rt.read(self.tokens, dtype=np.uint32)
        return out
