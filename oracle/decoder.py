"""CPU oracle of a Qwen2.5-shaped decoder step (test infrastructure).

The same wiring as ``neura_b200.qwen.Decoder`` stated with the oracle's primitives: products
in the reference tests' order over unpack(pack(w)) (crates/neura-runtime/tests/runtime.rs:72-83),
rms_norm (crates/neura-kernel/src/task/norm.rs:55-131), half-rotation RoPE
(crates/neura-kernel/src/task/rope.rs:48-122), causal grouped-query attention
(crates/neura-runtime/tests/support/attention.rs:71-109) and argmax with the lowest index on ties
(crates/neura-kernel/src/task/choice.rs:46-52).
"""
from __future__ import annotations

import numpy as np

import oracle


def bf16_round(values: np.ndarray) -> np.ndarray:
    """f32 -> bf16 -> f32, round to nearest even (crates/neura-precision/src/lib.rs:325-329); finite inputs."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = (bits + (((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


class OracleDecoder:
    def __init__(self, config, packed: dict, norms: dict, batch: int = 1, capacity: int = 640, threads: int = 8):
        """``packed``: name -> GGUF bytes of "token_embd.weight", "output.weight" and per layer
        attn_q/attn_k/attn_v/attn_output/ffn_gate/ffn_up/ffn_down; ``norms``: name -> f32 [hidden]."""
        self.c, self.batch, self.capacity, self.threads = config, batch, capacity, threads
        self.norms = norms
        self.embedding = packed["token_embd.weight"]
        c = config
        self.w = {}
        shapes = {name: (n, k) for name, n, k in c.linears()}
        for layer in range(c.layers):
            for name, (n, k) in shapes.items():
                key = f"blk.{layer}.{name}.weight"
                self.w[key] = oracle.unpack(c.element, n * k, packed[key]).reshape(n, k)
        self.w["output.weight"] = oracle.unpack(c.element, c.vocab * c.hidden, packed["output.weight"]).reshape(c.vocab, c.hidden)
        self.keys = np.zeros((c.layers, batch, c.key_heads, capacity, c.head_width), dtype=np.float32)
        self.values = np.zeros_like(self.keys)
        self.position = np.zeros(batch, dtype=np.uint32)
        self.logits = None
        self.bf16 = False     # True while a step stands for a row of a tensor-core prompt chunk
        self.w_bf16 = {}

    def _mm(self, name: str, x: np.ndarray) -> np.ndarray:
        if self.bf16:   # the tensor path: both operands rounded to bf16, f32 accumulation
            if name not in self.w_bf16:
                self.w_bf16[name] = bf16_round(self.w[name])
            return oracle.matmul_f32(self.w_bf16[name], bf16_round(x), threads=self.threads)
        return oracle.matmul_f32(self.w[name], x, threads=self.threads)

    def step(self, tokens: np.ndarray) -> np.ndarray:
        c = self.c
        hidden = oracle.embed(c.element, self.embedding, c.hidden, tokens)
        scale = np.float32(1.0 / float(c.head_width) ** 0.5)
        for layer in range(c.layers):
            at = lambda name: f"blk.{layer}.{name}.weight"  # noqa: E731
            normed = oracle.rms_norm(hidden, self.norms[at("attn_norm")], c.floor)
            q = self._mm(at("attn_q"), normed).reshape(self.batch, c.heads, c.head_width)
            k = self._mm(at("attn_k"), normed).reshape(self.batch, c.key_heads, c.head_width)
            v = self._mm(at("attn_v"), normed).reshape(self.batch, c.key_heads, c.head_width)
            q = oracle.rope(q, self.position, c.rope_base)
            k = oracle.rope(k, self.position, c.rope_base)
            for b in range(self.batch):
                self.keys[layer, b, :, self.position[b]] = k[b]
                self.values[layer, b, :, self.position[b]] = v[b]
            attended = oracle.attend(q, self.keys[layer], self.values[layer], self.position + 1, float(scale))
            hidden = hidden + self._mm(at("attn_output"), attended.reshape(self.batch, -1))
            normed = oracle.rms_norm(hidden, self.norms[at("ffn_norm")], c.floor)
            gate = self._mm(at("ffn_gate"), normed)
            gate = gate * (np.float32(1.0) / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)))   # silu
            held = self._mm(at("ffn_up"), normed) * gate
            hidden = hidden + self._mm(at("ffn_down"), held)
        normed = oracle.rms_norm(hidden, self.norms["output_norm.weight"], c.floor)
        self.logits = self._mm("output.weight", normed)
        self.position += 1
        return oracle.argmax(self.logits)

    def answer(self, tokens: np.ndarray, cursors: np.ndarray) -> np.ndarray:
        """One step with every plane's token and cursor given (the stepper ``generate.Batch`` drives)."""
        self.position[:] = np.asarray(cursors, dtype=np.uint32)
        return self.step(np.ascontiguousarray(tokens, dtype=np.uint32))

    chunks = (4, 2)   # the chunk sizes ``fill`` offers a ``generate.Batch`` (small, for the bookkeeping tests)
    wide = 0          # rows of a tensor-path chunk (``fill_wide``); 0: the stepper offers none
    WIDE_FROM = 64    # fewer prompt tokens than this go through the ordinary chunks

    def wide_tokens(self, length: int) -> int:
        """How many leading tokens of a prompt of ``length`` go through ``fill_wide`` (the rule of ``qwen.Decoder``)."""
        fed = length - 1
        if not self.wide or fed < self.WIDE_FROM:
            return 0
        return fed - (fed % self.wide if fed % self.wide < self.WIDE_FROM else 0)

    def fill_wide(self, sequence: int, tokens, start: int) -> None:
        """A prompt chunk through the tensor path: ``fill`` with both operands of every product rounded to bf16."""
        self.bf16 = True
        try:
            self.fill(sequence, tokens, start)
        finally:
            self.bf16 = False

    def fill(self, sequence: int, tokens, start: int) -> None:
        """A prompt chunk of one plane: the same cache rows the decode step writes token by token (the other
        planes ride along at their own cursors and are put back afterwards)."""
        keep = self.position.copy()
        for offset, token in enumerate(tokens):
            feed = np.zeros(self.batch, dtype=np.uint32)
            feed[sequence] = token
            cursors = keep.copy()
            cursors[sequence] = start + offset
            saved = (self.keys[:, :, :, :].copy(), self.values[:, :, :, :].copy())
            self.answer(feed, cursors)
            for b in range(self.batch):   # only the fed plane keeps what the step wrote
                if b != sequence:
                    self.keys[:, b] = saved[0][:, b]
                    self.values[:, b] = saved[1][:, b]
        self.position[:] = keep

    def generate(self, prompts: np.ndarray, steps: int, bf16_tokens: int = 0):
        """Returns (tokens [batch, steps], margins [batch, steps]): the gap between the two largest
        logits at every decoded step, which says how decisive each greedy choice was.  The first ``bf16_tokens``
        prompt tokens go through products with bf16 operands (a prompt fed through the tensor path)."""
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.batch, -1)
        self.position[:] = 0
        out = np.zeros((self.batch, steps), dtype=np.uint32)
        margins = np.zeros((self.batch, steps), dtype=np.float32)
        chosen = None
        for at in range(prompts.shape[1]):
            self.bf16 = at < bf16_tokens
            chosen = self.step(prompts[:, at].copy())
        self.bf16 = False
        for at in range(steps):
            if at:
                chosen = self.step(chosen)
            out[:, at] = chosen
            top = np.partition(self.logits, -2, axis=1)[:, -2:]
            margins[:, at] = top[:, 1] - top[:, 0]
        return out, margins


def synthetic_model(config, seed: int = 23, deviation: float = 0.02):
    """Random-init weights drawn in layer order from one stream of the reference's PRNG
    (Init::Normal{0, deviation}), packed by the oracle's quantiser; norm weights are 1."""
    stream = oracle.Stream(seed)
    c = config
    packed, norms = {}, {}
    table = stream.normal(c.vocab * c.hidden, 0.0, deviation).reshape(c.vocab, c.hidden)
    packed["token_embd.weight"] = oracle.pack_rows(c.element, table)
    for layer in range(c.layers):
        for name, n, k in c.linears():
            w = stream.normal(n * k, 0.0, deviation).reshape(n, k)
            packed[f"blk.{layer}.{name}.weight"] = oracle.pack_rows(c.element, w)
        norms[f"blk.{layer}.attn_norm.weight"] = np.ones(c.hidden, dtype=np.float32)
        norms[f"blk.{layer}.ffn_norm.weight"] = np.ones(c.hidden, dtype=np.float32)
    norms["output_norm.weight"] = np.ones(c.hidden, dtype=np.float32)
    if c.tied_head:
        packed["output.weight"] = packed["token_embd.weight"]
    else:
        head = stream.normal(c.vocab * c.hidden, 0.0, deviation).reshape(c.vocab, c.hidden)
        packed["output.weight"] = oracle.pack_rows(c.element, head)
    return packed, norms
