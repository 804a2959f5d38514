"""The tensor-core prefill product against the CPU oracle (needs a B200)."""
import os

import numpy as np
import pytest

import neura_b200 as nb

pytestmark = pytest.mark.gpu

# both sides round the dequantised weights and the activations to bf16 the same way, so what is left
# is the order of the f32 accumulation: 1e-3 of the output's rms is the north star's bar
REL_TOL = 1e-3


def check(runtime, oracle, m, n, k, chain=False, seed=61, residual=False):
    w = oracle.Stream(seed).normal(n * k, 0.0, 0.02).reshape(n, k)
    packed = oracle.pack_rows(nb.Q4K, w)
    x = oracle.Stream(seed + 2).normal(m * k).reshape(m, k)
    weight = runtime.load(nb.Q4K, n, k, packed)
    xd, od = runtime.tensor(m, k), runtime.tensor(m, n)
    runtime.write(xd, x)
    steps, ochain = None, None
    if chain:
        bias = oracle.Stream(seed + 4).normal(n)
        bd = runtime.tensor(n)
        runtime.write(bd, bias)
        steps, ochain = [nb.Step(nb.ADD, bd), nb.Step(nb.SILU)], [(oracle.ADD, bias), (oracle.SILU, None)]
    if residual:   # an operand read at the output coordinate through a row stride
        carried = oracle.Stream(seed + 6).normal(m * n).reshape(m, n)
        rd = runtime.tensor(m, n)
        runtime.write(rd, carried)
        steps, ochain = steps + [nb.Step(nb.ADD, rd)], ochain + [(oracle.ADD, carried)]
    runtime.linear_bf16(weight, xd, od, steps)
    got = runtime.read(od)
    want = oracle.linear(nb.Q4K, packed, n, k, x, chain=ochain, threads=os.cpu_count() or 8, bf16=True)
    scale = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    worst = float(np.abs(got - want).max())
    assert worst <= REL_TOL * scale, f"[{m}x{k}] x [{n}x{k}]: |diff| {worst:.3e} against rms {scale:.3e}"
    for ptr in (xd.ptr, od.ptr, weight.ptr):
        runtime.free(ptr)


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 256, 1024), (256, 512, 512), (200, 300, 768), (1, 33, 256),
                                   (130, 5, 256)])
def test_prefill_product_matches_the_bf16_oracle(runtime, oracle, m, n, k):
    check(runtime, oracle, m, n, k)


@pytest.mark.parametrize("m,n,k", [(257, 300, 512), (512, 512, 512), (600, 300, 512), (700, 300, 512),
                                   (1024, 512, 256), (600, 512, 3584)])
def test_prefill_product_over_several_row_tiles(runtime, oracle, m, n, k):
    # more than 256 rows: the second and later row tiles of the grid, with a ragged last one
    check(runtime, oracle, m, n, k)


@pytest.mark.parametrize("m,n,k,chain", [(600, 6500, 256, False), (600, 6500, 256, True), (300, 9604, 512, True),
                                         (600, 6501, 256, True)])
def test_prefill_product_with_more_tiles_than_half_the_sms(runtime, oracle, m, n, k, chain):
    # 78 tiles and more: K is not split, the product writes the caller's rows itself, by bulk tensor stores of 32 x 32
    # blocks where the rows allow a tensor map (ragged last blocks in both directions), row by row where they do not
    # (rows of 6501 numbers are not a multiple of 16 bytes apart)
    check(runtime, oracle, m, n, k, chain=chain, residual=chain)


def test_prefill_product_applies_the_fused_chain(runtime, oracle):
    check(runtime, oracle, 96, 320, 512, chain=True)


def test_prefill_product_applies_a_row_strided_chain_over_several_row_tiles(runtime, oracle):
    check(runtime, oracle, 520, 300, 512, chain=True, residual=True)


def test_prefill_product_at_the_benchmark_depth_on_a_slice_of_its_width(runtime, oracle):
    # config 4 is [2048 x 3584] x [18944 x 3584]; the oracle takes a slice of that in seconds
    check(runtime, oracle, 64, 512, 3584)


def test_prefill_product_at_the_benchmark_rows_on_a_slice_of_its_width(runtime, oracle):
    # all 2048 rows of config 4 (eight row tiles) against one 256-row tile of its weight
    check(runtime, oracle, 2048, 256, 3584)


@pytest.mark.parametrize("m,n,k,residual", [(96, 320, 512, False), (300, 300, 768, True), (1, 16, 256, False),
                                            (300, 4872, 256, True), (520, 4864, 512, False)])
def test_prefill_product_of_a_sealed_gate_up_pair(runtime, oracle, m, n, k, residual):
    # the pair's tiles hold 16 gate rows and the 16 up rows of the same columns: out = chain(silu(gate . x) * (up . x)).
    # Few tiles: runs of K in scratch, joined by the finishing kernel; many tiles (the last two cases, 78 and 114 tiles,
    # a ragged last unit in the first): joined in the product's own epilogue
    gate = oracle.Stream(71).normal(n * k, 0.0, 0.02).reshape(n, k)
    up = oracle.Stream(73).normal(n * k, 0.0, 0.02).reshape(n, k)
    packed_gate, packed_up = oracle.pack_rows(nb.Q4K, gate), oracle.pack_rows(nb.Q4K, up)
    x = oracle.Stream(75).normal(m * k).reshape(m, k)
    weight = runtime.load_pair(nb.Q4K, n, k, packed_gate, packed_up)
    xd, od = runtime.tensor(m, k), runtime.tensor(m, n)
    runtime.write(xd, x)
    threads = os.cpu_count() or 8
    g = oracle.linear(nb.Q4K, packed_gate, n, k, x, threads=threads, bf16=True)
    u = oracle.linear(nb.Q4K, packed_up, n, k, x, threads=threads, bf16=True)
    want = g * (np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u
    steps = None
    if residual:
        carried = oracle.Stream(77).normal(m * n).reshape(m, n).astype(np.float32)
        runtime.write(od, carried)
        steps = [nb.Step(nb.ADD, od)]   # in place, as a decoder layer adds its residual
        want = want + carried
    runtime.linear_bf16(weight, xd, od, steps)
    got = runtime.read(od).reshape(m, n)
    scale = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    worst = float(np.abs(got - want).max())
    assert worst <= REL_TOL * scale, f"pair [{m}x{k}] x 2[{n}x{k}]: |diff| {worst:.3e} against rms {scale:.3e}"
    for ptr in (xd.ptr, od.ptr, weight.ptr):
        runtime.free(ptr)


def test_prefill_refuses_what_it_does_not_multiply(runtime, oracle):
    w = oracle.Stream(3).normal(32 * 256, 0.0, 0.02).reshape(32, 256)
    q8 = runtime.load(nb.Q8_0, 32, 256, oracle.pack_rows(nb.Q8_0, w))
    xd, od = runtime.tensor(4, 256), runtime.tensor(4, 32)
    with pytest.raises(nb.NeuraCudaError, match="Q4K"):
        runtime.linear_bf16(q8, xd, od)
