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
                 batch: int = 1, capacity: int = 640, shard=None, comm=None, wide: int = 0):
        """``shard`` (parallel.Shard) and ``comm`` (parallel.TorchComm) make this one rank of a
        tensor-parallel group: ``weights`` then hold the rank's shares (q/k/v, gate, up and head
        rows; the K blocks of attention output and down that cover its window).
        ``wide`` > 0 asks for the tensor-core prompt path: the head of a long prompt is fed in chunks of up to ``wide``
        rows through the bf16 product (``fill_wide``); the caller asks because that product rounds both operands."""
        if batch > 16:
            raise ValueError("one decode step carries at most 16 sequences")
        if (shard is None) != (comm is None):
            raise ValueError("a tensor-parallel rank needs both its shard and its communicator")
        self.rt, self.config, self.weights, self.norms = rt, config, weights, norms
        self.batch, self.capacity, self.shard, self.comm = batch, capacity, shard, comm
        c = config
        world = shard.world if shard else 1
        # (a group may keep the attention block whole on every rank and split the MLP and the head only)
        self.whole_attention = bool(shard is not None and shard.whole)
        self.heads, self.key_heads = (shard.heads, shard.key_heads) if shard else (c.heads, c.key_heads)
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
        widest_k = max(c.hidden, self.window(c.feed_forward)[0], self.window(c.query_width, self.whole_attention)[0])
        # scratch for the decode step and for the largest prompt chunk, all of it now: a recorded step holds the
        # scratch's addresses, so nothing may grow it later
        most = max([batch, *self.chunks])
        if wide and (shard is not None or c.element != Q4K):
            raise ValueError("the tensor-core prompt path takes sealed Q4_K weights on one GPU")
        self.wide = min(int(wide), capacity) if wide else 0
        rt.reserve(most, max(self.vocab, 2 * self.feed_forward, c.hidden), widest_k)   # 2x: a sealed gate|up pair
        rt.reserve_decoder(max(most, self.wide), self.heads, self.key_heads, c.head_width, capacity)
        if self.wide:
            rt.reserve_bf16(self.wide, widest_k)
        self._wide_rows = None   # the activation rows of a wide chunk, made at its first use
        self.program: Optional[int] = None
        self._fill_programs: dict = {}   # (plane, rows of a chunk) -> "seen" once, then the chunk's recorded program
        self.compiled = None   # the step as one persistent kernel (compile())
        self.fold = False      # True: fold norms and stagings into the products' epilogues (fewer, longer launches)
        self.scale = 1.0 / float(c.head_width) ** 0.5

    def window(self, k: int, whole: bool = False):
        """(local K, lo, hi) of a row-parallel projection over a K axis of ``k`` (all of it for a projection the ranks
        keep whole)."""
        if self.shard is None or whole:
            return k, 0, k
        w = self.shard.window(k)
        return w.k, w.lo, w.hi

    def _row_parallel(self, x: DeviceTensor, weight: Weight, k: int, next_norm: DeviceTensor, whole: bool = False) -> None:
        """hidden += W x over this rank's share of K, summed over the ranks; then the rms_norm that follows
        every such projection (with ``next_norm``) and the staging of its result for the next product.  ``whole``: every
        rank holds all of K and of x (the attention output where the group keeps the attention block whole), so there
        is nothing to exchange."""
        rt, c = self.rt, self.config
        local, lo, hi = self.window(k, whole)
        if self.shard is None or whole:
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
        1 or 2 sequences, the MLP sealed as a pair, and, for a tensor-parallel rank, a communicator whose exchange a
        product can do in its own epilogue."""
        if self.batch > 2 or "blk.0.ffn_gate_up.weight" not in self.weights or not self.fold or self.whole_attention:
            return False
        return self.shard is None or hasattr(self.comm, "reduce_handle")

    def _step_folded(self) -> None:
        """The step with seven launches a layer instead of ten: the output and down products stage the hidden row
        for the next norm (gain and sums of squares in their epilogues, the scalar applied by the consumer), the
        gate|up product stages its own output for the down product.  On a tensor-parallel rank the output and down
        products also add the ranks' partial sums up in their epilogues (no launch of its own for the exchange), and
        the attended and held rows are staged at their window of the row-parallel weights' K axes.
        Slots: 0 hidden, 1 attended, 2 held."""
        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        reduce = self.comm.reduce_handle() if self.shard is not None else None
        carries = self.shard is None or self.shard.rank == 0   # rank 0 carries the residual into the sum
        attended_k, attended_lo, attended_hi = self.window(c.query_width)
        held_window = self.window(c.feed_forward)
        rt.staging_select(0)
        rt.embed(w["token_embd.weight"], self.tokens, self.hidden)
        rt.rms_norm_stage(self.hidden, n["blk.0.attn_norm.weight"], c.floor, c.element)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            after = n[f"blk.{layer + 1}.attn_norm.weight"] if layer + 1 < c.layers else n["output_norm.weight"]
            residual = [Step(ADD, self.hidden)] if carries else None
            rt.staging_select(0)
            rt.linear_staged_then(w[at("attn_qkv")], self.qkv, normed=layer > 0, floor=c.floor)
            rt.rope_cache(self.qkv, self.position, c.rope_base, self.heads, self.key_heads, c.head_width,
                          self.capacity, self.keys[layer], self.values[layer])
            rt.attend(self.qkv, self.keys[layer], self.values[layer], self.position, self.scale, self.heads,
                      self.key_heads, c.head_width, self.capacity, self.attended)
            rt.staging_select(1)
            rt.stage_window(self.attended, c.element, attended_k, attended_lo, attended_hi)
            rt.linear_staged_fused(w[at("attn_output")], self.hidden, residual, reduce=reduce, then_slot=0,
                                   gain=n[at("ffn_norm")], squares=True)
            rt.staging_select(0)
            rt.linear_staged_fused(w[at("ffn_gate_up")], self.held, normed=True, floor=c.floor, then_slot=2,
                                   window=held_window if self.shard is not None else None)
            rt.staging_select(2)
            rt.linear_staged_fused(w[at("ffn_down")], self.hidden, residual, reduce=reduce, then_slot=0, gain=after,
                                   squares=True)
        rt.staging_select(0)
        rt.linear_staged_then(w["output.weight"], self.logits, normed=True, floor=c.floor)
        if self.shard is None:
            rt.argmax(self.logits, self.tokens)
        else:
            self.comm.all_gather(self.gathered.ptr, self.logits.ptr, self.batch * self.vocab)
            rt.argmax_segments(self.gathered.ptr, self.batch, c.vocab, self.vocab, self.vocab,
                               self.batch * self.vocab, self.tokens)
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
            self._row_parallel(self.attended, w[at("attn_output")], c.query_width, n[at("ffn_norm")], self.whole_attention)
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

    @property
    def chunks(self) -> tuple:
        """The prompt chunk sizes ``fill`` takes, largest first (the reference fills in chunks of 32 and 8,
        examples/qwen/main.rs:21); empty where a prompt goes through the decode step token by token."""
        if self.shard is not None:
            return ()
        return (32, 8) if self.config.element == Q4K else (16, 8)

    def fill(self, sequence: int, tokens, start: int) -> None:
        """Batch::prefill for one chunk (crates/neura-generate/src/batch.rs:1595-1599, :298-325): feeds ``tokens``, consecutive
        prompt tokens of plane ``sequence`` at cursors start, start + 1, ..., through every layer at once.  The
        projections see all the rows of the chunk in one product (a Q4_K chunk of more than eight rows streams each
        weight once for all of them), the rows' keys and values go to the plane's cache, and row i attends to the
        cache up to its own cursor.  Nothing is chosen: a prompt's last token goes through ``answer``."""
        import numpy as np

        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        rows = int(tokens.size)
        if self.shard is not None:
            raise ValueError("a tensor-parallel rank feeds its prompt through the decode step")
        if not 1 <= rows <= self.chunks[0]:
            raise ValueError(f"a chunk holds 1 to {self.chunks[0]} tokens, not {rows}")
        if not 0 <= sequence < self.batch or start + rows > self.capacity:
            raise ValueError(f"plane {sequence} has no room for cursors {start}..{start + rows - 1}")
        held = self._fill_buffers(rows)
        rt.write(held["tokens"], tokens)
        rt.write(held["position"], np.arange(start, start + rows, dtype=np.uint32))
        self._replayed((sequence, rows), lambda: self._fill_launches(sequence, rows, held))

    def _fill_launches(self, sequence: int, rows: int, held: dict) -> None:
        """The launches of one prompt chunk of ``rows`` tokens of plane ``sequence`` (tokens and cursors in ``held``)."""
        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        hidden, qkv, attended, mlp = held["hidden"], held["qkv"], held["attended"], held["held"]
        per_plane = self.key_heads * self.capacity * c.head_width * 4
        rt.staging_select(0)
        rt.embed(w["token_embd.weight"], held["tokens"], hidden)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            keys_ptr = self.keys[layer].ptr + sequence * per_plane
            values_ptr = self.values[layer].ptr + sequence * per_plane
            rt.rms_norm_stage(hidden, n[at("attn_norm")], c.floor, c.element)
            rt.linear_staged(w[at("attn_qkv")], qkv)
            rt.rope_cache_rows(qkv, held["position"], c.rope_base, rows, self.heads, self.key_heads, c.head_width,
                               self.capacity, keys_ptr, values_ptr)
            rt.attend_rows(qkv, keys_ptr, values_ptr, held["position"], self.scale, rows, self.heads, self.key_heads,
                           c.head_width, self.capacity, attended)
            rt.stage(attended, c.element)
            rt.linear_staged(w[at("attn_output")], hidden, [Step(ADD, hidden)])
            rt.rms_norm_stage(hidden, n[at("ffn_norm")], c.floor, c.element)
            if at("ffn_gate_up") in w:
                rt.linear_staged(w[at("ffn_gate_up")], mlp)
            else:
                rt.linear_staged(w[at("ffn_gate")], held["gate"], [Step(SILU)])
                rt.linear_staged(w[at("ffn_up")], mlp, [Step(MUL, held["gate"])])
            rt.stage(mlp, c.element)
            rt.linear_staged(w[at("ffn_down")], hidden, [Step(ADD, hidden)])

    WIDE_FROM = 64   # fewer prompt tokens than this go through the ordinary chunks

    def wide_tokens(self, length: int) -> int:
        """How many leading tokens of a prompt of ``length`` ``prefill`` feeds through ``fill_wide``."""
        fed = length - 1
        return 0 if not self.wide or fed < self.WIDE_FROM else fed - (fed % self.wide if fed % self.wide < self.WIDE_FROM else 0)

    def fill_wide(self, sequence: int, tokens, start: int) -> None:
        """A prompt chunk of up to ``wide`` rows on the tensor cores: as ``fill``, but every projection is the prefill
        product (template_run_matmul_cooperative, crates/neura-kernel/src/task/matmul.rs:1344-1565: weights dequantised
        to bf16 tile by tile, activations rounded to bf16, f32 accumulation), so a 512-token prompt streams each weight
        once or twice instead of sixteen times.  Norms, RoPE, the cache and attention stay f32."""
        import numpy as np

        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        rows = int(tokens.size)
        if not self.wide:
            raise ValueError("this decoder was built without the tensor-core prompt path (wide=0)")
        if not 1 <= rows <= self.wide:
            raise ValueError(f"a wide chunk holds 1 to {self.wide} tokens, not {rows}")
        if not 0 <= sequence < self.batch or start + rows > self.capacity:
            raise ValueError(f"plane {sequence} has no room for cursors {start}..{start + rows - 1}")
        if self._wide_rows is None:
            most = self.wide
            self._wide_rows = {
                "tokens": rt.tensor_u32(most), "position": rt.tensor_u32(most), "hidden": rt.tensor(most, c.hidden),
                "normed": rt.tensor(most, c.hidden), "qkv": rt.tensor(most, self.query_width + 2 * self.key_width),
                "attended": rt.tensor(most, self.query_width), "held": rt.tensor(most, self.feed_forward),
                "gate": rt.tensor(most, self.feed_forward),
            }
        held = self._wide_rows
        padded = np.zeros(self.wide, dtype=np.uint32)
        padded[:rows] = tokens
        rt.write(held["tokens"], padded)
        padded[:rows] = np.arange(start, start + rows, dtype=np.uint32)
        padded[rows:] = 0
        rt.write(held["position"], padded)
        self._replayed(("wide", sequence, rows), lambda: self._wide_launches(sequence, rows, held))

    def _replayed(self, key, launches) -> None:
        """Runs ``launches`` (a chunk's kernels: tokens and cursors are read from device buffers, so they depend on the
        key only) as issued the first time (it may still size scratch), records them into a program the second time and
        replays that from then on: several hundred launches a chunk cost more on the host than on the device."""
        rt = self.rt
        state = self._fill_programs.get(key)
        if isinstance(state, int):
            rt.run(state)
            return
        if state == "seen":
            rt.capture_begin()
            try:
                launches()
            except Exception:
                try:   # leave no capture open behind a refused launch
                    rt.program_free(rt.capture_end())
                except Exception:
                    pass
                raise
            self._fill_programs[key] = rt.capture_end()
            rt.run(self._fill_programs[key])
            return
        self._fill_programs[key] = "seen"
        launches()

    def _wide_launches(self, sequence: int, rows: int, held: dict) -> None:
        """The launches of one wide prompt chunk of ``rows`` tokens of plane ``sequence``."""
        rt, c, w, n = self.rt, self.config, self.weights, self.norms
        hidden, normed, qkv, attended, mlp = held["hidden"], held["normed"], held["qkv"], held["attended"], held["held"]
        per_plane = self.key_heads * self.capacity * c.head_width * 4
        rt.embed(w["token_embd.weight"], held["tokens"], hidden, rows=rows)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            keys_ptr = self.keys[layer].ptr + sequence * per_plane
            values_ptr = self.values[layer].ptr + sequence * per_plane
            rt.rms_norm(hidden, n[at("attn_norm")], c.floor, normed, rows=rows)
            rt.linear_bf16(w[at("attn_qkv")], normed, qkv, rows=rows)
            rt.rope_cache_rows(qkv, held["position"], c.rope_base, rows, self.heads, self.key_heads, c.head_width,
                               self.capacity, keys_ptr, values_ptr)
            rt.attend_rows(qkv, keys_ptr, values_ptr, held["position"], self.scale, rows, self.heads, self.key_heads,
                           c.head_width, self.capacity, attended)
            rt.linear_bf16(w[at("attn_output")], attended, hidden, [Step(ADD, hidden)], rows=rows)
            rt.rms_norm(hidden, n[at("ffn_norm")], c.floor, normed, rows=rows)
            if at("ffn_gate_up") in w:
                rt.linear_bf16(w[at("ffn_gate_up")], normed, mlp, rows=rows)
            else:
                rt.linear_bf16(w[at("ffn_gate")], normed, held["gate"], [Step(SILU)], rows=rows)
                rt.linear_bf16(w[at("ffn_up")], normed, mlp, [Step(MUL, held["gate"])], rows=rows)
            rt.linear_bf16(w[at("ffn_down")], mlp, hidden, [Step(ADD, hidden)], rows=rows)

    def _fill_buffers(self, rows: int) -> dict:
        """The activation rows of a chunk of ``rows`` tokens (kept per row count: shapes carry the row strides)."""
        if not hasattr(self, "_fills"):
            self._fills = {}
        if rows not in self._fills:
            rt, c = self.rt, self.config
            self._fills[rows] = {
                "tokens": rt.tensor_u32(rows), "position": rt.tensor_u32(rows), "hidden": rt.tensor(rows, c.hidden),
                "qkv": rt.tensor(rows, self.query_width + 2 * self.key_width), "attended": rt.tensor(rows, self.query_width),
                "held": rt.tensor(rows, self.feed_forward), "gate": rt.tensor(rows, self.feed_forward),
            }
        return self._fills[rows]

    def prefill(self, prompts, wide: bool = True) -> None:
        """Feeds all but the last token of every plane's prompt in chunks (``fill``; where the decoder was built with
        ``wide`` rows and ``wide`` is left on, the head of a long prompt through ``fill_wide``), then leaves tokens and
        cursors so that the next ``run_token`` feeds the last prompt token of every plane."""
        import numpy as np

        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.batch, -1)
        length = prompts.shape[1]
        for sequence in range(self.batch):
            at, wide_end = 0, self.wide_tokens(length) if wide else 0
            while at < wide_end:   # the head of a long prompt on the tensor cores, where the decoder was built for it
                take = min(self.wide, wide_end - at)
                self.fill_wide(sequence, prompts[sequence, at: at + take], at)
                at += take
            while at < length - 1:
                left = length - 1 - at
                take = next((size for size in self.chunks if size <= left), left)
                self.fill(sequence, prompts[sequence, at: at + take], at)
                at += take
        self.rt.write(self.tokens, prompts[:, -1].copy())
        self.rt.write(self.position, np.full(self.batch, length - 1, dtype=np.uint32))

    def compile(self) -> None:
        """Runtime::compile for the whole step (crates/neura-runtime/src/runtime.rs:528): lays the step out
        as the phase table of one persistent kernel (``neura_cuda_decoder_compile``); ``run_token`` then
        launches that kernel instead of one kernel per operation.  1 or 2 sequences, the MLP sealed as a gate|up
        pair; a tensor-parallel rank needs a communicator whose exchange a kernel can do itself (``PeerComm``): the
        ranks' sums and the choice among their argmax winners then happen inside the step."""
        import ctypes

        from ._lib import NcDecoderDesc, NcDecoderLayer
        from .runtime import _check

        if self.shard is not None and not hasattr(self.comm, "reduce_handle"):
            raise ValueError("the persistent step of a tensor-parallel rank exchanges over peer memory: give it a PeerComm")
        if self.whole_attention:
            raise ValueError("the persistent step of a rank splits the attention block: make the Shard with attention=\"split\"")
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
        desc = NcDecoderDesc(c.layers, c.hidden, self.heads, self.key_heads, c.head_width, self.feed_forward, self.vocab,
                             self.batch, self.capacity, c.floor, c.rope_base, self.scale,
                             w["token_embd.weight"].record(), w["output.weight"].record(), n["output_norm.weight"].ptr,
                             layers, self.tokens.ptr, self.position.ptr, self.logits.ptr)
        handle = ctypes.c_void_p()
        if self.shard is None:
            _check(self.rt._lib.neura_cuda_decoder_compile(self.rt._ctx, ctypes.byref(desc), ctypes.byref(handle)))
        else:
            _check(self.rt._lib.neura_cuda_decoder_compile_rank(self.rt._ctx, ctypes.byref(desc), self.comm.reduce_handle(),
                                                                self.shard.world, self.shard.rank, ctypes.byref(handle)))
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
        """Gives back what the decoder recorded or compiled (the step's program, the prompt chunks' programs, the
        persistent step); the decoder steps eagerly afterwards."""
        if self.compiled is not None:
            self.rt._lib.neura_cuda_decoder_free(self.rt._ctx, self.compiled)
            self.compiled = None
        self.rt.sync()   # (a program may still be running)
        for program in [self.program, *self._fill_programs.values()]:
            if isinstance(program, int):
                self.rt.program_free(program)
        self.program = None
        self._fill_programs = {}

    def launches_per_token(self) -> int:
        if self.compiled is not None:
            return 1
        if self.folded():
            return self.config.layers * 7 + (5 if self.shard is None else 6)
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

        cursors = np.ascontiguousarray(cursors, dtype=np.uint32)
        if cursors.size and int(cursors.max()) >= self.capacity:
            raise ValueError(f"cursor {int(cursors.max())} lies past a cache of {self.capacity} rows")
        self.rt.write(self.tokens, np.ascontiguousarray(tokens, dtype=np.uint32))
        self.rt.write(self.position, cursors)
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

    def generate(self, prompts, steps: int, chunked: bool = False):
        """Feeds ``prompts`` [batch, length] (one token at a time, every step attending to all the tokens before
        it; or, ``chunked``, in chunks through ``prefill``), then decodes ``steps`` tokens greedily.
        Returns [batch, steps] ids."""
        import numpy as np

        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.batch, -1)
        if prompts.shape[1] + steps > self.capacity:
            raise ValueError(f"{prompts.shape[1]} prompt tokens and {steps} steps do not fit a cache of {self.capacity} rows")
        self.reset()
        out = np.zeros((self.batch, steps), dtype=np.uint32)
        if chunked and self.chunks:
            self.prefill(prompts)
            self.run_token()
        else:
            for at in range(prompts.shape[1]):
                self.rt.write(self.tokens, prompts[:, at].copy())
                self.run_token()
        out[:, 0] = self.rt.read(self.tokens, dtype=np.uint32)
        for at in range(1, steps):
            self.run_token()
            out[:, at] = self.rt.read(self.tokens, dtype=np.uint32)
        return out
