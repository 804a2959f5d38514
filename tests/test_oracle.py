"""The CPU oracle against what the reference pins for this path (no GPU needed)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "blocks.npz")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_block_byte_counts_follow_the_abi(oracle):
    # crates/neura-abi/tests/layout.rs:148-158 pins 32 -> 34 bytes and 256 -> 144 bytes
    assert oracle.payload_bytes(oracle.Q8_0, 32) == 34
    assert oracle.payload_bytes(oracle.Q8_0, 33) == 68
    assert oracle.payload_bytes(oracle.Q4K, 256) == 144
    assert oracle.payload_bytes(oracle.Q4K, 257) == 288
    assert oracle.payload_bytes(oracle.Q8_0, 4864 * 896) == 4630528       # config 1
    assert oracle.payload_bytes(oracle.Q4K, 18944 * 3584) == 38191104     # config 2
    # pack() pads its bytes to whole 4-byte words (ggml.rs:17-18)
    assert oracle.pack(oracle.Q8_0, np.ones(32, np.float32)).size == 36


def test_half_conversion_is_ieee_round_to_nearest_even(oracle):
    lib = oracle.lib()
    halves = np.arange(65536, dtype=np.uint16)
    expected = halves.view(np.float16).astype(np.float32)
    got = np.array([lib.nro_f16_to_f32(int(h)) for h in halves], dtype=np.float32)
    same = (bits(got) == bits(expected)) | (np.isnan(got) & np.isnan(expected))
    assert same.all()
    rng = np.random.default_rng(0)
    values = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000)).astype(np.float32)
    values = np.concatenate([values, np.array([0.0, -0.0, 65504, 65519.99, 65520, 5.96e-8, 2.98e-8, 2.9802322e-8,
                                               6.1e-5, 6.0975552e-05, np.inf, -np.inf], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = values.astype(np.float16).view(np.uint16)
    have = np.array([lib.nro_f32_to_f16(float(v)) for v in values], dtype=np.uint16)
    assert np.array_equal(want, have)
    # the one half the reference's own tests name: f16(0.25) (crates/neura-precision/tests/format.rs:232-234)
    assert lib.nro_f32_to_f16(0.25) == 0x3400


def test_bfloat16_rounds_to_nearest_even(oracle):
    lib = oracle.lib()
    # crates/neura-precision/src/lib.rs:325-329
    assert lib.nro_bf16_rne(1.0) == 0x3F80
    assert lib.nro_bf16_rne(float(np.float32(1.00390625))) == 0x3F80      # tie -> even (down)
    assert lib.nro_bf16_rne(float(np.float32(1.01171875))) == 0x3F82      # tie -> even (up)
    assert lib.nro_bf16_rne(float(np.float32(1.005))) == 0x3F81


def test_the_prng_is_xorshift32_13_17_5(oracle):
    # crates/neura-graph/src/init.rs:86-91, seeded seed|1 (tests/support/mod.rs:41-48)
    state = 23 | 1
    expected = []
    for _ in range(16):
        state ^= (state << 13) & 0xFFFFFFFF
        state ^= state >> 17
        state ^= (state << 5) & 0xFFFFFFFF
        expected.append(np.float32(-1.0) + np.float32(2.0) * (np.float32(state >> 8) / np.float32(1 << 24)))
    assert np.array_equal(bits(oracle.random(16, 23)), bits(np.array(expected, dtype=np.float32)))
    # an even seed and the odd seed above it draw the same stream
    assert np.array_equal(oracle.random(8, 22), oracle.random(8, 23))
    normal = oracle.Stream(23).normal(20000)
    assert abs(float(normal.mean())) < 0.03 and abs(float(normal.std()) - 1.0) < 0.03


def ggml_q4k_reference(field: np.ndarray) -> np.ndarray:
    """The published GGML Q4_K walk (dequantize_row_q4_K), written independently of the oracle."""
    d = np.frombuffer(field[0:2].tobytes(), dtype=np.float16)[0].astype(np.float32)
    dmin = np.frombuffer(field[2:4].tobytes(), dtype=np.float16)[0].astype(np.float32)
    scales = field[4:16].astype(np.uint32)
    qs = field[16:144]
    out = []

    def scale_min(j):
        if j < 4:
            return scales[j] & 63, scales[j + 4] & 63
        return (scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4), (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4)

    for group in range(4):
        chunk = qs[32 * group: 32 * group + 32]
        sc1, m1 = scale_min(2 * group)
        sc2, m2 = scale_min(2 * group + 1)
        d1, min1 = np.float32(d * np.float32(sc1)), np.float32(dmin * np.float32(m1))
        d2, min2 = np.float32(d * np.float32(sc2)), np.float32(dmin * np.float32(m2))
        out.extend(np.float32(d1 * np.float32(q & 0xF)) - min1 for q in chunk)
        out.extend(np.float32(d2 * np.float32(q >> 4)) - min2 for q in chunk)
    return np.array(out, dtype=np.float32)


def test_the_q4k_walk_agrees_across_three_restatements(oracle):
    # ggml.rs:336-350 (unpack), fetch.rs:256-267 (device scalar fetch), and the published GGML layout
    rng = np.random.default_rng(7)
    for _ in range(8):
        field = rng.integers(0, 256, 144, dtype=np.uint8)
        field[0:2] = np.frombuffer(np.float16(rng.uniform(0.001, 0.1)).tobytes(), dtype=np.uint8)
        field[2:4] = np.frombuffer(np.float16(rng.uniform(0.001, 0.1)).tobytes(), dtype=np.uint8)
        walked = oracle.unpack(oracle.Q4K, 256, field)
        fetched = np.array([oracle.fetch(oracle.Q4K, field, i) for i in range(256)], dtype=np.float32)
        assert np.array_equal(bits(walked), bits(fetched))
        assert np.array_equal(bits(walked), bits(ggml_q4k_reference(field)))


def test_the_q8_0_walk_agrees_across_restatements(oracle):
    rng = np.random.default_rng(8)
    field = rng.integers(0, 256, 34 * 3, dtype=np.uint8)
    for b in range(3):
        field[34 * b: 34 * b + 2] = np.frombuffer(np.float16(rng.uniform(0.001, 0.1)).tobytes(), dtype=np.uint8)
    walked = oracle.unpack(oracle.Q8_0, 96, field)
    fetched = np.array([oracle.fetch(oracle.Q8_0, field, i) for i in range(96)], dtype=np.float32)
    assert np.array_equal(bits(walked), bits(fetched))
    for b in range(3):
        d = np.frombuffer(field[34 * b: 34 * b + 2].tobytes(), dtype=np.float16)[0].astype(np.float32)
        q = field[34 * b + 2: 34 * b + 34].view(np.int8).astype(np.float32)
        assert np.array_equal(bits(walked[32 * b: 32 * b + 32]), bits(q * d))


def test_six_bit_scales_survive_their_packing(oracle):
    # put_scale_min_k4 / scale_min_k4 (ggml.rs:127-147): every sub-block keeps its own pair
    w = np.zeros(256, dtype=np.float32)
    for sub in range(8):
        w[32 * sub: 32 * sub + 32] = np.linspace(-(sub + 1) * 0.01, (8 - sub) * 0.02, 32)
    field = oracle.pack(oracle.Q4K, w)[:144]
    back = oracle.unpack(oracle.Q4K, 256, field)
    for sub in range(8):
        span = w[32 * sub: 32 * sub + 32]
        step = (span.max() - min(0.0, span.min())) / 15.0
        assert np.abs(back[32 * sub: 32 * sub + 32] - span).max() <= step * 0.75 + 2e-3


def test_round_trips_stay_within_half_a_step(oracle):
    w = oracle.Stream(23).normal(64 * 256, 0.0, 0.02)
    back = oracle.unpack(oracle.Q8_0, w.size, oracle.pack(oracle.Q8_0, w))
    for b in range(w.size // 32):
        block = w[32 * b: 32 * b + 32]
        quantum = np.abs(block).max() / 127.0
        # codes are taken with the f32 quantum and decoded with its fp16 rounding: 0.5 + 127 * 2^-11 steps
        assert np.abs(back[32 * b: 32 * b + 32] - block).max() <= quantum * 0.57 + 1e-7
    back = oracle.unpack(oracle.Q4K, w.size, oracle.pack(oracle.Q4K, w))
    assert np.abs(back - w).max() < 0.02 * 0.35


def test_zero_blocks_and_short_tails(oracle):
    zeros = np.zeros(256, dtype=np.float32)
    for element in (oracle.Q8_0, oracle.Q4K):
        packed = oracle.pack(element, zeros)
        assert np.array_equal(oracle.unpack(element, 256, packed), zeros)
    # the last block is padded with zeros (ggml.rs:12-15) and unpack truncates (ggml.rs:36)
    w = oracle.random(40, 5)
    packed = oracle.pack(oracle.Q8_0, w)
    assert packed.size == 68
    assert oracle.unpack(oracle.Q8_0, 40, packed).size == 40
    assert np.all(packed[34 + 2 + 8: 68] == 0)
    with pytest.raises(ValueError):
        oracle.unpack(oracle.Q8_0, 80, packed)   # fewer bytes than the shape packs (ggml.rs:25-30)


def test_the_product_is_the_reference_tests_loop(oracle):
    n, k, rows = 24, 512, 3
    w = oracle.random(n * k, 23).reshape(n, k)
    x = oracle.random(rows * k, 29).reshape(rows, k)
    for element in (oracle.Q8_0, oracle.Q4K):
        packed = oracle.pack_rows(element, w)
        weight = oracle.unpack(element, n * k, packed).reshape(n, k)
        expected = np.zeros((rows, n), dtype=np.float32)
        for r in range(rows):          # crates/neura-runtime/tests/runtime.rs:72-83
            for c in range(n):
                total = np.float32(0.0)
                for s in range(k):
                    total = np.float32(total + np.float32(weight[c, s] * x[r, s]))
                expected[r, c] = total
        got = oracle.linear(element, packed, n, k, x)
        assert np.array_equal(bits(got), bits(expected))
        assert np.array_equal(bits(oracle.linear(element, packed, n, k, x, threads=4)), bits(expected))
        assert np.array_equal(bits(oracle.matmul_f32(weight, x)), bits(expected))
        assert np.abs(got - (weight.astype(np.float64) @ x.astype(np.float64).T).T).max() < 1e-3


def test_the_chain_applies_ops_in_order_with_broadcast_operands(oracle):
    n, k, rows = 16, 256, 2
    w = oracle.random(n * k, 3).reshape(n, k)
    x = oracle.random(rows * k, 4).reshape(rows, k)
    packed = oracle.pack_rows(oracle.Q4K, w)
    plain = oracle.linear(oracle.Q4K, packed, n, k, x)
    bias = oracle.random(n, 5)
    gate = oracle.random(rows * n, 6).reshape(rows, n)
    got = oracle.linear(oracle.Q4K, packed, n, k, x, chain=[(oracle.ADD, bias), (oracle.SILU, None),
                                                            (oracle.MUL, gate), (oracle.SUB, gate, True)])
    y = plain + bias
    y = y * (np.float32(1.0) / (np.float32(1.0) + np.exp(-y, dtype=np.float32)))
    y = gate - y * gate
    assert np.abs(got - y).max() < 1e-5
    assert oracle.op_apply(oracle.SIGMOID, 0.0) == 0.5
    assert oracle.op_apply(oracle.MAXIMUM, 1.0, 2.0) == 2.0


def test_bf16_product_rounds_both_operands_first(oracle):
    n, k = 8, 256
    w = oracle.Stream(1).normal(n * k, 0.0, 0.02).reshape(n, k)
    x = oracle.Stream(2).normal(k).reshape(1, k)
    packed = oracle.pack_rows(oracle.Q4K, w)
    weight = oracle.unpack(oracle.Q4K, n * k, packed).reshape(n, k)

    def bf16(a):
        b = bits(a).astype(np.uint64)
        return (((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)

    expected = (bf16(weight).astype(np.float64) @ bf16(x).astype(np.float64).T).T
    got = oracle.linear(oracle.Q4K, packed, n, k, x, bf16=True)
    assert np.abs(got - expected).max() < 1e-4


def test_golden_vectors_still_hold(oracle):
    golden = np.load(GOLDEN)
    assert np.array_equal(bits(oracle.random(64, 23)), bits(golden["uniform_seed23"]))
    assert np.allclose(oracle.Stream(23).normal(64, 0.0, 0.02), golden["normal_seed23"], rtol=0, atol=1e-8)
    for name, element in (("q8_0", oracle.Q8_0), ("q4k", oracle.Q4K)):
        w, packed = golden[f"{name}_weight"], golden[f"{name}_packed"]
        n, k = w.shape
        assert np.array_equal(oracle.pack_rows(element, w), packed)
        assert np.array_equal(bits(oracle.unpack(element, n * k, packed)), bits(golden[f"{name}_unpacked"].reshape(-1)))
        x = golden[f"{name}_x"]
        assert np.array_equal(bits(oracle.linear(element, packed, n, k, x)), bits(golden[f"{name}_product"]))
        chain = [(oracle.ADD, golden[f"{name}_bias"]), (oracle.SILU, None)]
        assert np.allclose(oracle.linear(element, packed, n, k, x, chain=chain), golden[f"{name}_chain"], rtol=0, atol=1e-6)
    assert np.array_equal(oracle.pack_rows(oracle.Q8_0, golden["edge_weight"]), golden["edge_q8_0"])
    assert np.array_equal(oracle.pack_rows(oracle.Q4K, golden["edge_weight"]), golden["edge_q4k"])


def q6k_numpy(blocks):
    """An independent restatement of the published GGML Q6_K layout for [count, 210] bytes: ql 128, qh 64, int8 scales
    16, d; numbers 128 half + 32 group + lane."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 210)
    ql, qh = blocks[:, :128].astype(np.int32), blocks[:, 128:192].astype(np.int32)
    scales = blocks[:, 192:208].view(np.int8).astype(np.float32)
    d = blocks[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    out = np.zeros((blocks.shape[0], 256), dtype=np.float32)
    for half in range(2):
        for group in range(4):
            low = ql[:, half * 64 + (group % 2) * 32: half * 64 + (group % 2) * 32 + 32]
            low = (low >> 4) if group >= 2 else (low & 15)
            high = (qh[:, half * 32: half * 32 + 32] >> (2 * group)) & 3
            code = (low | (high << 4)).astype(np.float32) - np.float32(32.0)
            scale = np.repeat(scales[:, half * 8 + group * 2: half * 8 + group * 2 + 2], 16, axis=1)
            out[:, half * 128 + group * 32: half * 128 + group * 32 + 32] = (d[:, None] * scale) * code
    return out


def test_the_q6k_walk_agrees_across_restatements(oracle):
    # crates/neura-abi/tests/layout.rs:150 pins 256 -> 210 bytes; the walk is stated in ggml.rs:395-407 and fetch.rs:284-301
    assert oracle.payload_bytes(oracle.Q6K, 256) == 210 and oracle.payload_bytes(oracle.Q6K, 257) == 420
    rng = np.random.default_rng(7)
    blocks = rng.integers(0, 256, (64, 210), dtype=np.uint8)
    blocks[:, 208:210] = rng.uniform(-0.01, 0.01, 64).astype(np.float16).view(np.uint8).reshape(64, 2)   # finite d
    packed = blocks.reshape(-1)
    unpacked = oracle.unpack(oracle.Q6K, 64 * 256, packed)
    assert np.array_equal(bits(unpacked), bits(q6k_numpy(blocks).reshape(-1)))
    lib = oracle.lib()
    fetched = np.array([lib.nro_fetch(oracle.Q6K, packed.ctypes.data, at) for at in range(0, 64 * 256, 5)], dtype=np.float32)
    assert np.array_equal(bits(fetched), bits(unpacked[::5]))


def test_the_q6k_packer_follows_the_reference_to_the_letter(oracle):
    # ggml.rs:352-393.  The sub-block scale comes from the largest magnitude; `quantized(..., -32, 31) as u32` saturates
    # at zero, so what the reference's packer keeps of a negative number is code 32, i.e. zero.
    w = oracle.Stream(5).normal(4 * 512, 0.0, 0.02).reshape(4, 512)
    packed = oracle.pack_rows(oracle.Q6K, w)
    assert packed.size == 4 * 2 * 210
    back = oracle.unpack(oracle.Q6K, w.size, packed).reshape(w.shape)
    assert np.all(back[w < 0] == 0.0)
    step = np.abs(w).reshape(4, 32, 16).max(axis=2, keepdims=True) / 32.0
    err = np.abs(back - w).reshape(4, 32, 16)
    keep = (w > 0).reshape(4, 32, 16)
    # half a step inside the range; a whole step at the run's own peak, whose quotient 32 is clamped to 31; and the
    # run's factor is itself rounded to an int8 multiple of the block's scale
    assert np.all(err[keep] <= (np.broadcast_to(step, err.shape)[keep] * 1.1 + 2e-4))
    # a block of zeros: every code is the bias 32 (high bits 10 in all four groups), scales and d are zero; 210 bytes
    # padded to whole words
    assert oracle.pack(oracle.Q6K, np.zeros(256, np.float32)).tolist() == [0] * 128 + [170] * 64 + [0] * 20


def q5k_numpy(blocks):
    """An independent restatement of the published GGML Q5_K layout for [count, 176] bytes: d, dmin, twelve bytes of
    six-bit scales and mins, qh 32, qs 128; numbers 64 group + 32 seat + lane."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 176)
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = blocks[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    sc = blocks[:, 4:16].astype(np.int32)
    qh, qs = blocks[:, 16:48].astype(np.int32), blocks[:, 48:176].astype(np.int32)
    out = np.zeros((blocks.shape[0], 256), dtype=np.float32)
    for sub in range(8):
        if sub < 4:
            scale, low = sc[:, sub] & 63, sc[:, sub + 4] & 63
        else:
            scale = (sc[:, sub + 4] & 15) | ((sc[:, sub - 4] >> 6) << 4)
            low = (sc[:, sub + 4] >> 4) | ((sc[:, sub] >> 6) << 4)
        group, seat = sub // 2, sub % 2
        nibble = qs[:, group * 32: group * 32 + 32]
        nibble = (nibble >> 4) if seat else (nibble & 15)
        code = (nibble | (((qh >> sub) & 1) << 4)).astype(np.float32)
        out[:, sub * 32: sub * 32 + 32] = (d * scale.astype(np.float32))[:, None] * code - (dmin * low.astype(np.float32))[:, None]
    return out


def q3k_numpy(blocks):
    """An independent restatement of the published GGML Q3_K layout for [count, 110] bytes: hmask 32, qs 64, twelve bytes
    of six-bit scales, d; numbers 128 half + 32 j + lane, run 8 half + 2 j + lane // 16."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 110)
    hmask, qs, sc = blocks[:, :32].astype(np.int32), blocks[:, 32:96].astype(np.int32), blocks[:, 96:108].astype(np.int32)
    d = blocks[:, 108:110].copy().view(np.float16).astype(np.float32)[:, 0]
    out = np.zeros((blocks.shape[0], 256), dtype=np.float32)
    for run in range(16):
        low = sc[:, run % 8]
        code = ((low >> 4) if run >= 8 else (low & 15)) | (((sc[:, 8 + run % 4] >> (2 * (run // 4))) & 3) << 4)
        half, j, upper = run // 8, (run % 8) // 2, run % 2
        lanes = slice(upper * 16, upper * 16 + 16)
        two = (qs[:, half * 32: half * 32 + 32][:, lanes] >> (2 * j)) & 3
        third = (hmask[:, lanes] >> (half * 4 + j)) & 1
        quant = (two - np.where(third == 1, 0, 4)).astype(np.float32)
        at = half * 128 + j * 32 + upper * 16
        out[:, at: at + 16] = (d * (code.astype(np.float32) - np.float32(32.0)))[:, None] * quant
    return out


def random_blocks(seed, count, size, halves):
    """Random bytes with finite half floats at the byte offsets ``halves`` (a real GGUF holds finite scales)."""
    rng = np.random.default_rng(seed)
    blocks = rng.integers(0, 256, (count, size), dtype=np.uint8)
    for at in halves:
        blocks[:, at: at + 2] = rng.uniform(-0.01, 0.01, count).astype(np.float16).view(np.uint8).reshape(count, 2)
    return blocks


@pytest.mark.parametrize("name,size,halves,restated", [("Q5K", 176, (0, 2), q5k_numpy), ("Q3K", 110, (108,), q3k_numpy)])
def test_the_q5k_and_q3k_walks_agree_across_restatements(oracle, name, size, halves, restated):
    # crates/neura-abi/tests/layout.rs pins the block sizes; each walk is stated in ggml.rs (q5_k_values :318-334,
    # q3_k_values :292-308) and again in fetch.rs (:269-282, :242-254)
    element = getattr(oracle, name)
    assert oracle.payload_bytes(element, 256) == size and oracle.payload_bytes(element, 257) == 2 * size
    blocks = random_blocks(17, 64, size, halves)
    packed = blocks.reshape(-1)
    unpacked = oracle.unpack(element, 64 * 256, packed)
    assert np.array_equal(bits(unpacked), bits(restated(blocks).reshape(-1)))
    lib = oracle.lib()
    fetched = np.array([lib.nro_fetch(element, packed.ctypes.data, at) for at in range(0, 64 * 256, 7)], dtype=np.float32)
    assert np.array_equal(bits(fetched), bits(unpacked[::7]))


def test_the_q5k_and_q3k_packers_follow_the_reference(oracle):
    w = oracle.Stream(5).normal(4 * 512, 0.0, 0.02).reshape(4, 512)
    # q5_k (ggml.rs:310-312): affine_block with 31 steps; half a step of the sub-block's own span, plus what the six-bit
    # scale and min and the half-float d and dmin lose
    back = oracle.unpack(oracle.Q5K, w.size, oracle.pack_rows(oracle.Q5K, w)).reshape(w.shape)
    runs = w.reshape(4, 16, 32)
    span = np.maximum(runs.max(axis=2), 0) - np.minimum(runs.min(axis=2), 0)
    assert np.all(np.abs(back - w).reshape(4, 16, 32) <= (span / 31.0)[:, :, None] * 1.6 + 1e-4)
    # q3_k (ggml.rs:243-290): codes -4..3 times a quarter of the run's peak (rounded to 1/31 of the block's widest):
    # half a step inside the range, a whole step at the positive peak whose quotient 4 is clamped to 3 (three steps, each
    # off by up to half of d = widest / 124)
    packed = oracle.pack_rows(oracle.Q3K, w)
    assert packed.size == 4 * 2 * 110
    back = oracle.unpack(oracle.Q3K, w.size, packed).reshape(w.shape)
    peak = np.abs(w).reshape(4, 32, 16).max(axis=2, keepdims=True)
    widest = np.abs(w).reshape(4, 2, 256).max(axis=2).repeat(16, axis=1)[:, :, None]
    assert np.all(np.abs(back - w).reshape(4, 32, 16) <= peak / 4.0 + 2.0 * widest / 124.0 + 1e-5)
    # a block of zeros: d is the smallest normal over 124 (a half-float zero), every scale code the bias 32, every code
    # zero with its third bit set
    zero = oracle.pack(oracle.Q3K, np.zeros(256, np.float32)).tolist()
    assert zero[:32] == [255] * 32 and zero[32:96] == [0] * 64 and zero[96:104] == [0] * 8 and zero[104:108] == [170] * 4
    assert zero[108:110] == [0, 0] and len(zero) == 112   # 110 bytes padded to whole words


def test_sixteen_bit_weights_round_as_the_reference_packs_them(oracle):
    # crates/neura-precision/src/lib.rs:8-9, :34-42: half::f16::from_f32 and the bfloat16 of :325-329, both to nearest even
    w = np.array([1.0, -2.5, 1.0009765625, 1.00048828125, 65504.0, 1e-8, 3.140625, 1.00390625, 1.001953125], dtype=np.float32)
    halves = oracle.unpack(oracle.HALF, w.size, oracle.pack(oracle.HALF, w))
    assert np.array_equal(bits(halves), bits(w.astype(np.float16).astype(np.float32)))
    brains = oracle.unpack(oracle.BFLOAT16, w.size, oracle.pack(oracle.BFLOAT16, w))
    rounded = ((w.view(np.uint32).astype(np.uint64) + 0x7fff + ((w.view(np.uint32) >> 16) & 1)) >> 16 << 16).astype(np.uint32)
    assert np.array_equal(bits(brains), rounded)
    assert oracle.payload_bytes(oracle.HALF, 7) == 14 and oracle.pack(oracle.HALF, w[:7]).size == 16


def test_the_decoder_oracle_rounds_to_bf16_as_the_c_oracle_does(oracle):
    from oracle.decoder import bf16_round

    x = oracle.Stream(5).normal(4096).astype(np.float32)
    x[:6] = [1.00390625, 1.01171875, -1.00390625, 0.0, 3.0e38, 1e-40]   # two ties, a negative tie, zero, near the top, a subnormal
    want = np.array([oracle.lib().nro_bf16_rne(float(v)) for v in x], dtype=np.uint16)
    got = (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal(got, want)
