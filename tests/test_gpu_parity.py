"""CUDA path against the CPU oracle, through the C ABI (needs a B200)."""
import os

import numpy as np
import pytest

import neura_b200 as nb

pytestmark = pytest.mark.gpu

ELEMENTS = [nb.Q8_0, nb.Q4K]
# the reference's own bar: |device - naive f32 loop| <= 1e-3 absolute on uniform(-1, 1) data
# (crates/neura-runtime/tests/runtime.rs:85, tests/support/mod.rs:50-67)
ABS_TOL = 1e-3
# the bar of this path: within 1e-3 relative (fp32 accumulation-order differences only)
REL_TOL = 1e-3


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def weights(oracle, element, n, k, seed=23, normal=False):
    stream = oracle.Stream(seed)
    w = stream.normal(n * k, 0.0, 0.02) if normal else stream.uniform(n * k)
    return w.reshape(n, k), oracle.pack_rows(element, w.reshape(n, k))


def assert_close(actual, expected, what=""):
    """max |diff| <= 1e-3 of the expected output's rms (the absolute 1e-3 of the reference's own tests is kept
    only by the two tests that restate them)."""
    err = np.abs(actual - expected)
    scale = np.sqrt(np.mean(expected.astype(np.float64) ** 2)) + 1e-30
    assert err.max() <= REL_TOL * scale, (
        f"{what}: max |diff| {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}, rms of expected {scale:.3e}")


@pytest.mark.parametrize("element", ELEMENTS)
@pytest.mark.parametrize("n,k", [(16, 256), (40, 512), (1024, 2048), (33, 1280)])
def test_dequant_is_bit_exact_in_both_layouts(runtime, oracle, element, n, k):
    _, packed = weights(oracle, element, n, k)
    expected = oracle.unpack(element, n * k, packed).reshape(n, k)
    raw = runtime.load(element, n, k, packed, seal=False)
    assert np.array_equal(bits(runtime.dequant(raw)), bits(expected))
    sealed = runtime.load(element, n, k, packed)
    assert sealed.layout == nb.LAYOUT_TILED
    assert np.array_equal(bits(runtime.dequant(sealed)), bits(expected))


@pytest.mark.parametrize("element", ELEMENTS)
@pytest.mark.parametrize("normal", [False, True])
def test_device_packer_matches_host_packer_bit_for_bit(runtime, oracle, element, normal):
    # a_quantized_tensor_reads_back_the_blocks_a_device_packs (runtime.rs:717-736)
    w, packed = weights(oracle, element, 64, 1024, seed=5, normal=normal)
    got = runtime.quantize(element, w)
    assert np.array_equal(got, packed[: got.size])


@pytest.mark.parametrize("element", ELEMENTS)
def test_device_packer_handles_zero_and_constant_blocks(runtime, oracle, element):
    w = np.zeros((4, 512), dtype=np.float32)
    w[1] = 0.75
    w[2, ::3] = -1e-3
    w[3] = np.linspace(-2, 5, 512, dtype=np.float32)
    packed = oracle.pack_rows(element, w)
    assert np.array_equal(runtime.quantize(element, w), packed)


@pytest.mark.parametrize("element", ELEMENTS)
@pytest.mark.parametrize("rows", [1, 2, 4])
def test_a_narrow_product_walks_the_quantized_weight(runtime, oracle, element, rows):
    # a_narrow_product_walks_the_quantized_weight_a_gguf_stores (runtime.rs:12-86)
    depth, columns = 2048, 1024
    _, packed = weights(oracle, element, columns, depth, seed=23)
    x = oracle.random(rows * depth, 29).reshape(rows, depth)
    expected = oracle.linear(element, packed, columns, depth, x, threads=8)
    w = runtime.load(element, columns, depth, packed)
    got = runtime.linear_host(w, x)
    assert np.abs(got - expected).max() <= ABS_TOL


@pytest.mark.parametrize("element", ELEMENTS)
def test_a_wide_product_walks_the_quantized_weight(runtime, oracle, element):
    # a_wide_product_walks_the_quantized_weight_a_gguf_stores (runtime.rs:88-144)
    rows, depth, columns = 8, 512, 4096
    _, packed = weights(oracle, element, columns, depth, seed=23)
    x = oracle.random(rows * depth, 29).reshape(rows, depth)
    expected = oracle.linear(element, packed, columns, depth, x, threads=8)
    w = runtime.load(element, columns, depth, packed)
    got = runtime.linear_host(w, x)
    assert np.abs(got - expected).max() <= ABS_TOL


@pytest.mark.parametrize("element,n,k", [
    (nb.Q8_0, 4864, 896),    # config 1: Qwen2.5-0.5B up projection
    (nb.Q8_0, 1, 32), (nb.Q8_0, 17, 96), (nb.Q8_0, 130, 4864),
    (nb.Q4K, 1, 256), (nb.Q4K, 31, 768), (nb.Q4K, 1000, 3584), (nb.Q4K, 48, 27648),
])
@pytest.mark.parametrize("rows", [1, 3, 5, 16, 19])
def test_products_over_ragged_shapes(runtime, oracle, element, n, k, rows):
    _, packed = weights(oracle, element, n, k, seed=101, normal=True)
    x = oracle.Stream(7).normal(rows * k).reshape(rows, k)
    expected = oracle.linear(element, packed, n, k, x, threads=8)
    w = runtime.load(element, n, k, packed)
    got = runtime.linear_host(w, x)
    assert_close(got, expected, f"element {element} [{n},{k}] rows {rows}")


@pytest.fixture(scope="module")
def mlp_7b(runtime, oracle):
    """Config 2's weight: Q4_K [18944 x 3584] ~ N(0, 0.02), packed by the oracle and sealed on the device."""
    n, k = 18944, 3584
    _, packed = weights(oracle, nb.Q4K, n, k, seed=23, normal=True)
    sealed = runtime.load(nb.Q4K, n, k, packed)
    yield n, k, packed, sealed
    runtime.free(sealed.ptr)


@pytest.mark.parametrize("rows", [1, 4, 16, 64])
def test_the_7b_mlp_product_at_its_own_size(runtime, oracle, mlp_7b, rows):
    # the sweep of config 2: K = 3584, N = 18944, batch 1 / 4 / 16 / 64
    n, k, packed, sealed = mlp_7b
    x = oracle.Stream(29).normal(rows * k).reshape(rows, k)
    expected = oracle.linear(nb.Q4K, packed, n, k, x, threads=os.cpu_count() or 8)
    got = runtime.linear_host(sealed, x)
    assert_close(got, expected, f"Q4_K [{n},{k}] rows {rows}")


@pytest.mark.parametrize("element", ELEMENTS)
@pytest.mark.parametrize("rows", [9, 24, 33, 64, 70])
def test_products_of_many_rows_over_ragged_shapes(runtime, oracle, element, rows):
    # the row counts the reference gives its staged-run tiles (crates/neura-plan/src/product.rs:118-131)
    for n, k in ((130, 768), (257, 1024)):
        _, packed = weights(oracle, element, n, k, seed=77, normal=True)
        x = oracle.Stream(79).normal(rows * k).reshape(rows, k)
        expected = oracle.linear(element, packed, n, k, x, threads=8)
        w = runtime.load(element, n, k, packed)
        assert_close(runtime.linear_host(w, x), expected, f"element {element} [{n},{k}] rows {rows}")
        runtime.free(w.ptr)


@pytest.mark.parametrize("element", ELEMENTS)
def test_the_fused_chain_applies_its_steps_in_order(runtime, oracle, element):
    n, k, rows = 96, 512, 3
    _, packed = weights(oracle, element, n, k, seed=3, normal=True)
    x = oracle.Stream(11).normal(rows * k).reshape(rows, k)
    gate = oracle.Stream(13).normal(rows * n).reshape(rows, n)
    bias = oracle.Stream(17).normal(n)
    chain_o = [(oracle.ADD, bias), (oracle.SILU, None), (oracle.MUL, gate), (oracle.SUB, gate, True)]
    expected = oracle.linear(element, packed, n, k, x, chain=chain_o)
    w = runtime.load(element, n, k, packed)
    xd, od = runtime.tensor(rows, k), runtime.tensor(rows, n)
    gd, bd = runtime.tensor(rows, n), runtime.tensor(n)
    runtime.write(xd, x); runtime.write(gd, gate); runtime.write(bd, bias)
    chain = [nb.Step(nb.ADD, bd), nb.Step(nb.SILU), nb.Step(nb.MUL, gd), nb.Step(nb.SUB, gd, swapped=True)]
    runtime.linear(w, xd, od, chain)
    got = runtime.read(od)
    assert_close(got, expected, "chain")


def test_activations_far_from_one_keep_their_precision(runtime, oracle):
    # block fixed point must follow the magnitude of each stretch of the activations
    n, k = 64, 1024
    _, packed = weights(oracle, nb.Q4K, n, k, seed=9, normal=True)
    x = oracle.Stream(21).normal(k).reshape(1, k)
    x[0, :256] *= 1e-6
    x[0, 256:512] *= 1e4
    x[0, 512:768] = 0.0
    expected = oracle.linear(nb.Q4K, packed, n, k, x)
    got = runtime.linear_host(runtime.load(nb.Q4K, n, k, packed), x)
    assert_close(got, expected, "mixed magnitudes")
    tiny = (x * 1e-30).astype(np.float32)
    expected = oracle.linear(nb.Q4K, packed, n, k, tiny)
    got = runtime.linear_host(runtime.load(nb.Q4K, n, k, packed), tiny)
    assert np.abs(got - expected).max() <= 1e-3 * np.abs(expected).max()


def test_the_library_refuses_what_the_reference_panics_on(runtime, oracle):
    _, packed = weights(oracle, nb.Q4K, 16, 256)
    with pytest.raises(nb.NeuraCudaError):
        runtime.load(nb.Q4K, 16, 200, packed)           # rows that do not fill blocks
    with pytest.raises(nb.NeuraCudaError):
        runtime.load(nb.Q4K, 64, 256, packed)           # a source shorter than its shape (store.rs:90-123)
    raw = runtime.load(nb.Q4K, 16, 256, packed, seal=False)
    with pytest.raises(nb.NeuraCudaError):
        runtime.linear_host(raw, np.zeros((1, 256), np.float32))  # the product wants a sealed weight


def test_device_packer_keeps_the_sign_of_a_zero_extreme(runtime, oracle):
    # least/greatest (ggml.rs:90-96) return their second argument on a tie, which decides
    # whether an all-positive or all-zero block stores +0 or -0 in its fp16 fields
    w = np.zeros((6, 256), dtype=np.float32)
    w[1, 5] = -0.0
    w[2] = np.abs(oracle.Stream(3).normal(256)) + 0.1
    w[3] = -np.abs(oracle.Stream(4).normal(256)) - 0.1
    w[4, 40:] = 1.0
    w[4, 7] = -0.0
    w[5, :200] = -1.0
    w[5, 255] = -0.0
    packed = oracle.pack_rows(nb.Q4K, w)
    assert np.array_equal(runtime.quantize(nb.Q4K, w), packed)


@pytest.mark.parametrize("element", ELEMENTS)
@pytest.mark.parametrize("n,k,rows", [(48, 512, 1), (1000, 1024, 3), (27, 256, 2)])
def test_a_sealed_gate_up_pair_is_the_swiglu_of_the_two_products(runtime, oracle, element, n, k, rows):
    # examples/qwen/mlp.rs:31-33: mul(silu(matmul(x, gate)), matmul(x, up))
    gate = oracle.Stream(51).normal(n * k, 0.0, 0.05).reshape(n, k)
    up = oracle.Stream(53).normal(n * k, 0.0, 0.05).reshape(n, k)
    pg, pu = oracle.pack_rows(element, gate), oracle.pack_rows(element, up)
    x = oracle.Stream(57).normal(rows * k).reshape(rows, k)
    silu = oracle.linear(element, pg, n, k, x, chain=[(oracle.SILU, None)])
    expected = oracle.linear(element, pu, n, k, x, chain=[(oracle.MUL, silu)])
    pair = runtime.load_pair(element, n, k, pg, pu)
    assert pair.layout == nb.LAYOUT_TILED_PAIR
    xd, od = runtime.tensor(rows, k), runtime.tensor(rows, n)
    runtime.write(xd, x)
    runtime.linear(pair, xd, od)
    assert_close(runtime.read(od), expected, f"pair element {element} [{n},{k}] rows {rows}")


def q6k_blocks(seed, n, k):
    """Random Q6_K blocks with every code in use (the reference's own packer never writes a negative code) and a
    finite d, as a real GGUF holds them."""
    rng = np.random.default_rng(seed)
    blocks = rng.integers(0, 256, (n * (k // 256), 210), dtype=np.uint8)
    blocks[:, 208:210] = rng.uniform(-2e-3, 2e-3, blocks.shape[0]).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return blocks.reshape(-1)


@pytest.mark.parametrize("n,k", [(16, 256), (40, 512), (33, 1280), (1000, 5120)])
def test_q6k_dequant_is_bit_exact(runtime, oracle, n, k):
    for packed in (q6k_blocks(3, n, k), oracle.pack_rows(nb.Q6K, weights(oracle, nb.Q8_0, n, k, seed=9)[0])):
        expected = oracle.unpack(nb.Q6K, n * k, packed).reshape(n, k)
        held = runtime.load(nb.Q6K, n, k, packed)
        assert held.layout == nb.LAYOUT_GGUF
        assert np.array_equal(bits(runtime.dequant(held)), bits(expected))
        runtime.free(held.ptr)


@pytest.mark.parametrize("n,k", [(1, 256), (31, 768), (1000, 3584), (4099, 5120)])
@pytest.mark.parametrize("rows", [1, 2, 3, 8, 19])
def test_q6k_products_over_ragged_shapes(runtime, oracle, n, k, rows):
    packed = q6k_blocks(11, n, k)
    x = oracle.Stream(7).normal(rows * k).reshape(rows, k)
    expected = oracle.linear(nb.Q6K, packed, n, k, x, threads=8)
    w = runtime.load(nb.Q6K, n, k, packed)
    assert_close(runtime.linear_host(w, x), expected, f"Q6_K [{n},{k}] rows {rows}")
    runtime.free(w.ptr)


def test_q6k_narrow_and_wide_products_of_the_reference_tests(runtime, oracle):
    # crates/neura-runtime/tests/runtime.rs:12-144 run every GGML format, Q6_K among them: uniform(-1, 1) weights through
    # the host packer, absolute 1e-3
    for rows, depth, columns in ((1, 2048, 1024), (4, 2048, 1024), (8, 512, 4096)):
        w, _ = weights(oracle, nb.Q8_0, columns, depth, seed=23)
        packed = oracle.pack_rows(nb.Q6K, w)
        x = oracle.random(rows * depth, 29).reshape(rows, depth)
        expected = oracle.linear(nb.Q6K, packed, columns, depth, x, threads=8)
        held = runtime.load(nb.Q6K, columns, depth, packed)
        assert np.abs(runtime.linear_host(held, x) - expected).max() <= ABS_TOL
        runtime.free(held.ptr)


def test_q6k_product_applies_the_fused_chain_and_gathers_rows(runtime, oracle):
    n, k, rows = 96, 512, 3
    packed = q6k_blocks(13, n, k)
    x = oracle.Stream(11).normal(rows * k).reshape(rows, k)
    bias = oracle.Stream(17).normal(n)
    expected = oracle.linear(nb.Q6K, packed, n, k, x, chain=[(oracle.ADD, bias), (oracle.SILU, None)])
    w = runtime.load(nb.Q6K, n, k, packed)
    xd, od, bd = runtime.tensor(rows, k), runtime.tensor(rows, n), runtime.tensor(n)
    runtime.write(xd, x)
    runtime.write(bd, bias)
    runtime.linear(w, xd, od, [nb.Step(nb.ADD, bd), nb.Step(nb.SILU)])
    assert_close(runtime.read(od), expected, "Q6_K chain")
    # the embedding gather of a Q6_K table (select.rs:29-49 over fetch_q6_k)
    tokens = runtime.tensor_u32(4)
    runtime.write(tokens, np.array([5, 0, 95, 5], dtype=np.uint32))
    rows_out = runtime.tensor(4, k)
    runtime.embed(w, tokens, rows_out)
    table = oracle.unpack(nb.Q6K, n * k, packed).reshape(n, k)
    assert np.array_equal(bits(runtime.read(rows_out)), bits(table[[5, 0, 95, 5]]))


# ---- the other formats kept in GGUF order: Q5_K, Q3_K, half and bfloat16 numbers --------------------------------
def gguf_blocks(element, seed, n, k):
    """Random payload bytes of [n, k] numbers of ``element`` with finite scales, every code in use."""
    rng = np.random.default_rng(seed)
    if element in (nb.HALF, nb.BFLOAT16):
        numbers = rng.normal(0.0, 0.05, n * k).astype(np.float32)
        if element == nb.HALF:
            return numbers.astype(np.float16).view(np.uint8).reshape(-1).copy()
        return (numbers.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(-1).copy()
    size, halves = {nb.Q5K: (176, (0, 2)), nb.Q3K: (110, (108,)), nb.Q6K: (210, (208,))}[element]
    blocks = rng.integers(0, 256, (n * (k // 256), size), dtype=np.uint8)
    for at in halves:
        blocks[:, at: at + 2] = rng.uniform(-2e-3, 2e-3, blocks.shape[0]).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return blocks.reshape(-1)


GGUF_ORDER = [nb.Q5K, nb.Q3K, nb.HALF, nb.BFLOAT16]


@pytest.mark.parametrize("element", GGUF_ORDER)
@pytest.mark.parametrize("n,k", [(16, 256), (33, 1280), (1000, 5120)])
def test_dequant_of_the_formats_kept_in_gguf_order_is_bit_exact(runtime, oracle, element, n, k):
    sources = [gguf_blocks(element, 3, n, k), oracle.pack_rows(element, weights(oracle, nb.Q8_0, n, k, seed=9)[0])]
    for packed in sources:
        expected = oracle.unpack(element, n * k, packed).reshape(n, k)
        held = runtime.load(element, n, k, packed)
        assert held.layout == nb.LAYOUT_GGUF
        assert np.array_equal(bits(runtime.dequant(held)), bits(expected))
        runtime.free(held.ptr)


@pytest.mark.parametrize("element", GGUF_ORDER)
@pytest.mark.parametrize("n,k", [(1, 256), (31, 768), (1000, 3584)])
@pytest.mark.parametrize("rows", [1, 3, 8, 19])
def test_products_of_the_formats_kept_in_gguf_order(runtime, oracle, element, n, k, rows):
    packed = gguf_blocks(element, 11, n, k)
    x = oracle.Stream(7).normal(rows * k).reshape(rows, k)
    expected = oracle.linear(element, packed, n, k, x, threads=8)
    w = runtime.load(element, n, k, packed)
    assert_close(runtime.linear_host(w, x), expected, f"element {element} [{n},{k}] rows {rows}")
    runtime.free(w.ptr)


@pytest.mark.parametrize("element", GGUF_ORDER)
def test_the_reference_products_chain_and_gather_in_gguf_order(runtime, oracle, element):
    # crates/neura-runtime/tests/runtime.rs:12-144 run every GGML format: uniform(-1, 1) weights through the host packer,
    # absolute 1e-3
    for rows, depth, columns in ((1, 2048, 1024), (4, 2048, 1024)):
        w, _ = weights(oracle, nb.Q8_0, columns, depth, seed=23)
        packed = oracle.pack_rows(element, w)
        x = oracle.random(rows * depth, 29).reshape(rows, depth)
        expected = oracle.linear(element, packed, columns, depth, x, threads=8)
        held = runtime.load(element, columns, depth, packed)
        assert np.abs(runtime.linear_host(held, x) - expected).max() <= ABS_TOL
        runtime.free(held.ptr)
    n, k, rows = 96, 512, 3
    packed = gguf_blocks(element, 13, n, k)
    x = oracle.Stream(11).normal(rows * k).reshape(rows, k)
    bias = oracle.Stream(17).normal(n)
    expected = oracle.linear(element, packed, n, k, x, chain=[(oracle.ADD, bias), (oracle.SILU, None)])
    w = runtime.load(element, n, k, packed)
    xd, od, bd = runtime.tensor(rows, k), runtime.tensor(rows, n), runtime.tensor(n)
    runtime.write(xd, x)
    runtime.write(bd, bias)
    runtime.linear(w, xd, od, [nb.Step(nb.ADD, bd), nb.Step(nb.SILU)])
    assert_close(runtime.read(od), expected, f"element {element} chain")
    tokens = runtime.tensor_u32(4)
    runtime.write(tokens, np.array([5, 0, 95, 5], dtype=np.uint32))
    rows_out = runtime.tensor(4, k)
    runtime.embed(w, tokens, rows_out)   # the embedding gather (select.rs:29-49 over the format's fetch)
    table = oracle.unpack(element, n * k, packed).reshape(n, k)
    assert np.array_equal(bits(runtime.read(rows_out)), bits(table[[5, 0, 95, 5]]))
    # nothing seals these formats, and no staged product takes them
    with pytest.raises(nb.NeuraCudaError):
        runtime.seal_device(element, n, k, w.ptr)


@pytest.mark.parametrize("rows", [24, 32])
def test_a_product_whose_k_axis_is_split_gives_the_same_sums_every_time(runtime, oracle, rows):
    # [7168 x 5120] (the 32B q|k|v projection) has fewer 128-row tiles than the GPU has SMs, so the product splits the K
    # axis and adds the slices' partial sums up; run it often enough for a race between slices to show
    n, k = 7168, 5120
    w, packed = weights(oracle, nb.Q4K, n, k, seed=31)
    x = oracle.Stream(37).normal(rows * k).reshape(rows, k)
    expected = oracle.linear(nb.Q4K, packed, n, k, x, threads=16)
    held = runtime.load(nb.Q4K, n, k, packed)
    xd, od = runtime.tensor(rows, k), runtime.tensor(rows, n)
    runtime.write(xd, x)
    for turn in range(12):
        runtime.linear(held, xd, od)
        assert_close(runtime.read(od), expected, f"Q4_K [{n},{k}] rows {rows}, turn {turn}")
    runtime.free(held.ptr)
