"""GGUF reader (and a small writer for fixtures): the wire format of the weights on this path.

Mirrors the reference's ``neura-gguf`` (crates/neura-gguf/src/header.rs:43-148): versions 2 and 3,
the metadata table, the tensor table (name, rank 1-4, ggml type, offset aligned to
``general.alignment``, default 32), the ggml-type -> element map (header.rs:150-162) and the
refusals of malformed files (crates/neura-gguf/tests/gguf.rs:173-243).  A tensor's payload is
handed out verbatim: ``Runtime.load`` pours those bytes and seals them.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple, Union

import numpy as np

MAGIC = b"GGUF"
VERSIONS = (2, 3)
DEFAULT_ALIGNMENT = 32

# ggml type -> (element code of neura_abi::Element, block elements, block bytes)
SINGLE, HALF, BFLOAT16, Q8_0, Q4K, Q5K, Q6K, Q3K = 0, 1, 2, 8, 9, 10, 11, 12
TYPES = {
    0: (SINGLE, 1, 4), 1: (HALF, 1, 2), 8: (Q8_0, 32, 34), 11: (Q3K, 256, 110), 12: (Q4K, 256, 144),
    13: (Q5K, 256, 176), 14: (Q6K, 256, 210), 30: (BFLOAT16, 1, 2),
}
GGML_OF = {SINGLE: 0, HALF: 1, Q8_0: 8, Q4K: 12, BFLOAT16: 30}


class GgufError(ValueError):
    """A malformed or truncated file (the reference panics with a sentence; this raises it)."""


@dataclass(frozen=True)
class Tensor:
    element: int
    elements: int
    shape: Tuple[int, ...]   # ne[0] first: for a weight matrix (k, n)
    at: int                  # offset inside the tensor data
    nbytes: int


class _Reader:
    def __init__(self, data):
        self.data, self.at = data, 0

    def take(self, count: int) -> bytes:
        if count < 0 or self.at + count > len(self.data):
            raise GgufError("a gguf header runs past the bytes this file holds")
        out = bytes(self.data[self.at: self.at + count])
        self.at += count
        return out

    def number(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))[0]

    def text(self) -> str:
        length = self.number("Q")
        if length > (1 << 24):
            raise GgufError(f"a gguf string of {length} bytes is longer than a header holds")
        return self.take(length).decode("utf-8", "replace")

    _SCALARS = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}

    def value(self, depth: int = 0):
        kind = self.number("I")
        return self.typed(kind, depth)

    def typed(self, kind: int, depth: int):
        if kind in self._SCALARS:
            return self.number(self._SCALARS[kind])
        if kind == 8:
            return self.text()
        if kind == 9:
            if depth > 4:
                raise GgufError("a gguf nests arrays deeper than this reader follows")
            inner, count = self.number("I"), self.number("Q")
            if count > (1 << 28):
                raise GgufError(f"a gguf array of {count} entries is longer than a header holds")
            return [self.typed(inner, depth + 1) for _ in range(count)]
        raise GgufError(f"a gguf metadata value of type {kind} is not one this reader knows")


class Gguf:
    """A parsed GGUF over bytes, a numpy array or a memory-mapped file."""

    def __init__(self, data):
        self.data = data
        reader = _Reader(data)
        magic = reader.take(4)
        if magic != MAGIC:
            raise GgufError(f"this file opens with {magic!r} where a gguf opens with GGUF")
        version = reader.number("I")
        if version not in VERSIONS:
            raise GgufError(f"this gguf declares version {version}, and this reader holds the versions {VERSIONS}")
        tensors, pairs = reader.number("Q"), reader.number("Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(pairs):
            key = reader.text()
            if key in self.metadata:
                raise GgufError(f"two entries of this gguf carry the metadata key {key}")
            self.metadata[key] = reader.value()
        alignment = self.metadata.get("general.alignment", DEFAULT_ALIGNMENT)
        if not isinstance(alignment, int) or isinstance(alignment, bool):
            raise GgufError("this gguf measures its alignment by a value that is not an integer")
        if alignment == 0 or alignment % 8:
            raise GgufError(f"this gguf aligns its tensors by {alignment}, and a gguf aligns them by a multiple of eight")
        self.alignment = alignment
        self.tensors: Dict[str, Tensor] = {}
        for _ in range(tensors):
            name = reader.text()
            rank = reader.number("I")
            if rank == 0 or rank > 4:
                raise GgufError(f"the tensor {name} declares {rank} dimensions, and a gguf tensor carries one to four")
            shape = tuple(reader.number("Q") for _ in range(rank))
            elements = 1
            for dim in shape:
                elements *= dim
            if elements >= 1 << 63:
                raise GgufError(f"the tensor {name} spans more numbers than a gguf counts")
            kind, at = reader.number("I"), reader.number("Q")
            if at % alignment:
                raise GgufError(f"the tensor {name} begins at byte {at} of the tensor data, and a gguf aligns it by {alignment}")
            if kind not in TYPES:
                raise GgufError(f"the tensor {name} holds numbers of ggml type {kind}, which this framework does not read")
            element, per, size = TYPES[kind]
            if elements % per:
                raise GgufError(f"the tensor {name} holds {elements} numbers, and a block packs {per} of them")
            self.tensors[name] = Tensor(element, elements, shape, at, elements // per * size)
        self.data_start = (reader.at + alignment - 1) // alignment * alignment
        for name, tensor in self.tensors.items():
            if self.data_start + tensor.at + tensor.nbytes > len(data):
                raise GgufError(f"the tensor {name} runs past the bytes this file holds")

    @classmethod
    def open(cls, path: str) -> "Gguf":
        """GgufFile::open (crates/neura-gguf/src/lib.rs:102): the file is mapped, not read."""
        with open(path, "rb") as fh:
            mapped = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        return cls(mapped)

    def payload(self, name: str) -> np.ndarray:
        """The tensor's bytes, verbatim (Source::payload, crates/neura-source/src/lib.rs:16-22)."""
        if name not in self.tensors:
            raise GgufError(f"this gguf holds no tensor {name}")
        t = self.tensors[name]
        start = self.data_start + t.at
        return np.frombuffer(self.data, dtype=np.uint8, count=t.nbytes, offset=start)

    def matrix(self, name: str, rows: int, columns: int) -> Tuple[int, np.ndarray]:
        """decoder::matrix's contract (crates/neura-decoder/src/parameter.rs:5-15): the GGUF shape of
        a [rows, columns] weight is (columns, rows).  Returns (element, payload)."""
        if name not in self.tensors:
            raise GgufError(f"this gguf holds no tensor {name}")
        t = self.tensors[name]
        if len(t.shape) < 2 or (t.shape[0], t.shape[1]) != (columns, rows) or t.elements != rows * columns:
            raise GgufError(f"the tensor {name} is shaped {t.shape} where a [{rows}, {columns}] matrix stores ({columns}, {rows})")
        return t.element, self.payload(name)

    def vector(self, name: str, width: int) -> np.ndarray:
        """decoder::vector (parameter.rs:17-33): an f32 (or f16) vector of ``width``."""
        if name not in self.tensors:
            raise GgufError(f"this gguf holds no tensor {name}")
        t = self.tensors[name]
        if t.elements != width:
            raise GgufError(f"the tensor {name} holds {t.elements} numbers where {width} are declared")
        raw = self.payload(name)
        if t.element == SINGLE:
            return raw.view(np.float32).copy()
        if t.element == HALF:
            return raw.view(np.float16).astype(np.float32)
        raise GgufError(f"the tensor {name} is not stored as plain floats")


Scalar = Union[int, float, bool, str]


def write(tensors: List[Tuple[str, int, Tuple[int, ...], np.ndarray]], metadata: Dict[str, Scalar] = None,
          alignment: int = 32, version: int = 3) -> bytes:
    """Builds a GGUF image: ``tensors`` = [(name, element, shape (ne[0] first), payload bytes)].
    The counterpart of the reference tests' fixture writer (crates/neura-runtime/tests/support/mod.rs:84-124)."""
    out = bytearray()
    out += MAGIC + struct.pack("<I", version) + struct.pack("<Q", len(tensors))
    pairs = dict(metadata or {})
    pairs.setdefault("general.alignment", alignment)
    out += struct.pack("<Q", len(pairs))

    def text(s: str) -> bytes:
        raw = s.encode("utf-8")
        return struct.pack("<Q", len(raw)) + raw

    for key, value in pairs.items():
        out += text(key)
        if isinstance(value, bool):
            out += struct.pack("<I?", 7, value)
        elif isinstance(value, int):
            out += struct.pack("<II", 4, value) if 0 <= value < (1 << 32) else struct.pack("<Iq", 11, value)
        elif isinstance(value, float):
            out += struct.pack("<If", 6, value)
        else:
            out += struct.pack("<I", 8) + text(str(value))
    tensors = [(name, element, shape, np.ascontiguousarray(payload).view(np.uint8).tobytes())
               for name, element, shape, payload in tensors]
    at = 0
    for name, element, shape, payload in tensors:
        out += text(name) + struct.pack("<I", len(shape))
        for dim in shape:
            out += struct.pack("<Q", dim)
        out += struct.pack("<I", GGML_OF[element]) + struct.pack("<Q", at)
        at = (at + len(payload) + alignment - 1) // alignment * alignment
    while len(out) % alignment:
        out.append(0)
    for _, _, _, payload in tensors:
        out += payload
        while len(out) % alignment:
            out.append(0)
    return bytes(out)


# -- a decoder out of a GGUF ---------------------------------------------------------------

def read_config(gguf: Gguf, name: str = None):
    """Config::read (examples/qwen/config.rs:22-60): the decoder's shapes from the metadata keyed by
    ``general.architecture``; the vocabulary is the token table's row count and the element is the
    one the layer projections are stored in."""
    from .qwen import Config

    meta = gguf.metadata
    arch = meta.get("general.architecture")
    if not isinstance(arch, str):
        raise GgufError("this gguf names no general.architecture")

    def word(key: str) -> int:
        value = meta.get(f"{arch}.{key}")
        if not isinstance(value, int) or isinstance(value, bool) or value < 0:
            raise GgufError(f"this gguf holds no count under {arch}.{key}")
        return value

    def single(key: str, default: float) -> float:
        value = meta.get(f"{arch}.{key}", default)
        if not isinstance(value, float):
            raise GgufError(f"this gguf holds no number under {arch}.{key}")
        return value

    hidden, heads = word("embedding_length"), word("attention.head_count")
    head_width = meta.get(f"{arch}.attention.key_length", hidden // max(heads, 1))
    table = gguf.tensors.get("token_embd.weight")
    if table is None or len(table.shape) != 2 or table.shape[0] != hidden:
        raise GgufError("this gguf holds no token_embd.weight of the declared width")
    first = gguf.tensors.get("blk.0.attn_q.weight")
    if first is None:
        raise GgufError("this gguf holds no blk.0.attn_q.weight")
    return Config(name or str(meta.get("general.name", arch)), word("block_count"), hidden, heads,
                  word("attention.head_count_kv"), head_width, word("feed_forward_length"), table.shape[1],
                  first.element, floor=single("attention.layer_norm_rms_epsilon", 1e-6),
                  rope_base=single("rope.freq_base", 1e6), tied_head="output.weight" not in gguf.tensors)


def decoder_tensors(gguf: Gguf, config):
    """(packed, norms) as ``parallel.load_decoder_weights`` takes them: every projection checked
    against its declared shape and element (parameter.rs:5-33), payloads still in the file's bytes."""
    c = config
    packed, norms = {}, {}

    def matrix(name: str, rows: int, columns: int):
        element, payload = gguf.matrix(name, rows, columns)
        if element != c.element:
            raise GgufError(f"the tensor {name} is stored as element {element} where this decoder runs element {c.element}")
        packed[name] = payload

    matrix("token_embd.weight", c.vocab, c.hidden)
    if c.tied_head:
        packed["output.weight"] = packed["token_embd.weight"]
    else:
        matrix("output.weight", c.vocab, c.hidden)
    norms["output_norm.weight"] = gguf.vector("output_norm.weight", c.hidden)
    for layer in range(c.layers):
        at = lambda part: f"blk.{layer}.{part}"  # noqa: E731
        for part, n, k in c.linears():
            matrix(at(part + ".weight"), n, k)
        norms[at("attn_norm.weight")] = gguf.vector(at("attn_norm.weight"), c.hidden)
        mlp_norm = at("ffn_norm.weight") if at("ffn_norm.weight") in gguf.tensors else at("post_attention_norm.weight")
        norms[at("ffn_norm.weight")] = gguf.vector(mlp_norm, c.hidden)
    return packed, norms


def write_decoder(config, packed, norms, arch: str = "qwen2") -> bytes:
    """A GGUF image of a decoder (fixtures and the synthetic benchmark model written out)."""
    c = config
    meta = {
        "general.architecture": arch, "general.name": c.name,
        f"{arch}.block_count": c.layers, f"{arch}.embedding_length": c.hidden,
        f"{arch}.feed_forward_length": c.feed_forward, f"{arch}.attention.head_count": c.heads,
        f"{arch}.attention.head_count_kv": c.key_heads, f"{arch}.attention.key_length": c.head_width,
        f"{arch}.rope.freq_base": float(c.rope_base), f"{arch}.attention.layer_norm_rms_epsilon": float(c.floor),
    }
    tensors = [("token_embd.weight", c.element, (c.hidden, c.vocab), packed["token_embd.weight"])]
    if not c.tied_head:
        tensors.append(("output.weight", c.element, (c.hidden, c.vocab), packed["output.weight"]))
    tensors.append(("output_norm.weight", SINGLE, (c.hidden,), np.asarray(norms["output_norm.weight"], np.float32)))
    for layer in range(c.layers):
        for part, n, k in c.linears():
            name = f"blk.{layer}.{part}.weight"
            tensors.append((name, c.element, (k, n), packed[name]))
        for part in ("attn_norm", "ffn_norm"):
            name = f"blk.{layer}.{part}.weight"
            tensors.append((name, SINGLE, (c.hidden,), np.asarray(norms[name], np.float32)))
    return write(tensors, meta)
