"""The GGUF reader against hand-built files: the cases of the reference's own reader tests
(crates/neura-gguf/tests/gguf.rs:29-275) restated over this reader, and a decoder read back
from a GGUF image of the oracle's synthetic model."""
import struct

import numpy as np
import pytest

import oracle
from neura_b200 import gguf
from neura_b200.qwen import Config
from oracle.decoder import synthetic_model


def text(s):
    raw = s.encode()
    return struct.pack("<Q", len(raw)) + raw


def build(alignment, pairs, tensors, version=3, spacing=None):
    """A GGUF image: pairs = [(key, kind, packed value)], tensors = [(name, ggml type, dims, bytes)].
    ``spacing`` places consecutive tensors by that step instead of the declared alignment."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(pairs)))
    for key, kind, value in pairs:
        out += text(key) + struct.pack("<I", kind) + value
    at, step = 0, spacing or alignment
    for name, kind, dims, payload in tensors:
        out += text(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", kind, at)
        at = (at + len(payload) + step - 1) // step * step
    while len(out) % alignment:
        out.append(0)
    start = len(out)
    at = 0
    for _, _, _, payload in tensors:
        out += b"\0" * (at - (len(out) - start)) + payload
        at = (at + len(payload) + step - 1) // step * step
    return bytes(out), start


ALIGN32 = [("general.alignment", 4, struct.pack("<I", 32))]


def test_metadata_of_every_kind_comes_back():
    pairs = ALIGN32 + [
        ("general.architecture", 8, text("qwen2")), ("a.u8", 0, struct.pack("<B", 200)), ("a.i8", 1, struct.pack("<b", -3)),
        ("a.u16", 2, struct.pack("<H", 60000)), ("a.i16", 3, struct.pack("<h", -300)), ("a.i32", 5, struct.pack("<i", -70000)),
        ("a.f32", 6, struct.pack("<f", 0.5)), ("a.flag", 7, struct.pack("<?", True)), ("a.u64", 10, struct.pack("<Q", 1 << 40)),
        ("a.i64", 11, struct.pack("<q", -(1 << 40))), ("a.f64", 12, struct.pack("<d", 0.25)),
        ("a.words", 9, struct.pack("<IQ", 4, 3) + struct.pack("<3I", 1, 2, 3)),
        ("a.names", 9, struct.pack("<IQ", 8, 2) + text("x") + text("yz")),
    ]
    image, _ = build(32, pairs, [])
    held = gguf.Gguf(image)
    m = held.metadata
    assert m["general.architecture"] == "qwen2" and m["a.u8"] == 200 and m["a.i8"] == -3
    assert m["a.u16"] == 60000 and m["a.i16"] == -300 and m["a.i32"] == -70000 and m["a.f32"] == 0.5
    assert m["a.flag"] is True and m["a.u64"] == 1 << 40 and m["a.i64"] == -(1 << 40) and m["a.f64"] == 0.25
    assert m["a.words"] == [1, 2, 3] and m["a.names"] == ["x", "yz"]
    assert held.alignment == 32 and not held.tensors


@pytest.mark.parametrize("version", [2, 3])
def test_every_readable_type_is_named_and_sized(version):
    cases = [(0, gguf.SINGLE, 64, 256), (1, gguf.HALF, 64, 128), (30, gguf.BFLOAT16, 64, 128), (8, gguf.Q8_0, 64, 68),
             (12, gguf.Q4K, 512, 288), (11, gguf.Q3K, 256, 110), (13, gguf.Q5K, 256, 176), (14, gguf.Q6K, 256, 210)]
    rng = np.random.default_rng(5)
    tensors = [(f"t{kind}", kind, [count], rng.integers(0, 256, size, dtype=np.uint8).tobytes())
               for kind, _, count, size in cases]
    image, start = build(32, ALIGN32, tensors, version=version)
    held = gguf.Gguf(image)
    assert held.data_start == start
    for (kind, element, count, size), (_, _, _, payload) in zip(cases, tensors):
        t = held.tensors[f"t{kind}"]
        assert (t.element, t.elements, t.nbytes, t.shape) == (element, count, size, (count,))
        assert held.payload(f"t{kind}").tobytes() == payload


def test_alignment_defaults_to_32_and_may_be_declared():
    image, start = build(32, [], [("w", 12, [256], b"\7" * 144)])
    assert gguf.Gguf(image).alignment == 32 and start % 32 == 0
    image, start = build(64, [("general.alignment", 4, struct.pack("<I", 64))], [("w", 12, [256], b"\7" * 144), ("v", 8, [32], b"\1" * 34)])
    held = gguf.Gguf(image)
    assert held.alignment == 64 and held.tensors["v"].at == 192 and held.payload("v").tobytes() == b"\1" * 34


def test_a_tensor_this_framework_cannot_read_is_refused_by_name():
    image, _ = build(32, ALIGN32, [("packed", 23, [256], b"\0" * 136)])
    with pytest.raises(gguf.GgufError, match="packed.*ggml type 23"):
        gguf.Gguf(image)


def test_files_that_do_not_follow_the_layout_are_refused():
    image, start = build(32, ALIGN32, [("weights", 12, [256], b"\0" * 144)])
    with pytest.raises(gguf.GgufError, match="opens with"):
        gguf.Gguf(b"GGFU" + image[4:])
    with pytest.raises(gguf.GgufError, match="version 9"):
        gguf.Gguf(image[:4] + struct.pack("<I", 9) + image[8:])
    with pytest.raises(gguf.GgufError, match="runs past"):
        gguf.Gguf(image[:8])
    with pytest.raises(gguf.GgufError, match="runs past"):
        gguf.Gguf(image[:start + 100])
    half, _ = build(32, ALIGN32, [("weights", 12, [128], b"\0" * 144)])
    with pytest.raises(gguf.GgufError, match="a block packs 256"):
        gguf.Gguf(half)
    off, _ = build(32, ALIGN32, [("first", 12, [256], b"\0" * 144), ("second", 12, [256], b"\0" * 144)], spacing=8)
    with pytest.raises(gguf.GgufError, match="second begins at byte 144"):
        gguf.Gguf(off)
    twice, _ = build(32, ALIGN32 + ALIGN32, [])
    with pytest.raises(gguf.GgufError, match="two entries"):
        gguf.Gguf(twice)
    odd, _ = build(32, [("general.alignment", 4, struct.pack("<I", 12))], [])
    with pytest.raises(gguf.GgufError, match="multiple of eight"):
        gguf.Gguf(odd)
    worded, _ = build(32, [("general.alignment", 8, text("32"))], [])
    with pytest.raises(gguf.GgufError, match="not an integer"):
        gguf.Gguf(worded)
    for rank in (0, 5):
        body = bytearray(b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + text("w") + struct.pack("<I", rank))
        body += b"".join(struct.pack("<Q", 1) for _ in range(rank)) + struct.pack("<IQ", 0, 0) + b"\0" * 64
        with pytest.raises(gguf.GgufError, match="one to four"):
            gguf.Gguf(bytes(body))


def test_a_mapped_file_hands_out_the_same_bytes_as_the_whole_image(tmp_path):
    image, _ = build(32, [("general.alignment", 4, struct.pack("<I", 16))], [("weights", 12, [256], b"\7" * 144)])
    path = tmp_path / "weights.gguf"
    path.write_bytes(image)
    file, held = gguf.Gguf.open(str(path)), gguf.Gguf(image)
    assert file.tensors == held.tensors and len(file.tensors) == 1
    assert file.payload("weights").tobytes() == held.payload("weights").tobytes() == b"\7" * 144


def test_matrix_and_vector_check_the_declared_shape():
    w = oracle.pack_rows(gguf.Q8_0, np.arange(4 * 64, dtype=np.float32).reshape(4, 64))
    image = gguf.write([("w", gguf.Q8_0, (64, 4), w), ("n", gguf.SINGLE, (64,), np.ones(64, np.float32)),
                        ("h", gguf.HALF, (8,), np.arange(8, dtype=np.float16))])
    held = gguf.Gguf(image)
    element, payload = held.matrix("w", 4, 64)
    assert element == gguf.Q8_0 and payload.tobytes() == w.tobytes()
    with pytest.raises(gguf.GgufError, match="shaped"):
        held.matrix("w", 64, 4)
    with pytest.raises(gguf.GgufError, match="no tensor"):
        held.matrix("missing", 4, 64)
    assert held.vector("n", 64).tolist() == [1.0] * 64
    assert held.vector("h", 8).tolist() == list(range(8))
    with pytest.raises(gguf.GgufError, match="where 32 are declared"):
        held.vector("n", 32)
    with pytest.raises(gguf.GgufError, match="plain floats"):
        held.vector("w", 256)


@pytest.mark.parametrize("element,tied", [(gguf.Q8_0, True), (gguf.Q4K, False)])
def test_a_decoder_comes_back_out_of_its_gguf(element, tied):
    config = Config("tiny", 2, 256, 4, 2, 64, 512, 96, element, floor=float(np.float32(1e-5)), rope_base=10000.0, tied_head=tied)
    packed, norms = synthetic_model(config, seed=3)
    norms["blk.1.ffn_norm.weight"] = np.linspace(0.5, 1.5, 256, dtype=np.float32)
    image = gguf.write_decoder(config, packed, norms)
    held = gguf.Gguf(image)
    read = gguf.read_config(held)
    assert read == config
    got_packed, got_norms = gguf.decoder_tensors(held, read)
    assert set(got_packed) == set(packed) and set(got_norms) == set(norms)
    for name in packed:
        assert got_packed[name].tobytes() == np.ascontiguousarray(packed[name]).tobytes(), name
    for name in norms:
        assert np.array_equal(got_norms[name], norms[name]), name
    wrong = Config("tiny", 2, 256, 4, 2, 64, 512, 96, gguf.Q8_0 if element == gguf.Q4K else gguf.Q4K, tied_head=tied)
    with pytest.raises(gguf.GgufError):
        gguf.decoder_tensors(held, wrong)
