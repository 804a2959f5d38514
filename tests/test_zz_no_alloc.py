"""The allocation-free product against the ordinary one (needs a B200).

Some embedders cannot let a library allocate device memory while they run: a game loop
that steps generation inside a frame budget cannot absorb a cudaMalloc or the device-wide
wait behind a cudaFree, and an engine that owns the whole device heap forbids allocation
by anything it hosts.  ``neura_cuda_linear_static`` serves them from a fixed array inside
the library.  This file is named so that pytest collects it last.
"""
import numpy as np
import pytest

import neura_b200 as nb

pytestmark = pytest.mark.gpu

TOLERANCE = 1e-3  # the bar of the other product tests; both entry points run the same kernels


@pytest.mark.parametrize("element,n,k,rows", [
    (nb.Q4K, 1000, 3584, 1),
    (nb.Q4K, 96, 5120, 4),
    (nb.Q8_0, 4864, 896, 1),
    (nb.Q8_0, 130, 4864, 3),
])
def test_the_static_scratch_product_matches_the_allocating_one_twice_in_a_row(runtime, oracle, element, n, k, rows):
    w = oracle.Stream(31).normal(n * k, 0.0, 0.02).reshape(n, k)
    weight = runtime.load(element, n, k, oracle.pack_rows(element, w))
    bias = runtime.tensor(n)
    runtime.write(bias, oracle.Stream(37).normal(n))
    chain = [nb.Step(nb.ADD, bias)]
    x, expected, got = runtime.tensor(rows, k), runtime.tensor(rows, n), runtime.tensor(rows, n)
    for call in range(2):  # the second call meets whatever the first left in the shared array
        values = oracle.Stream(41 + call).normal(rows * k).reshape(rows, k)
        runtime.write(x, values)
        runtime.linear(weight, x, expected, chain)
        runtime.linear_static(weight, x, got, chain)
        a, b = runtime.read(expected), runtime.read(got)
        scale = float(np.sqrt(np.mean(a.astype(np.float64) ** 2)))
        assert np.abs(a - b).max() <= TOLERANCE * scale, f"call {call}: {np.abs(a - b).max()} against rms {scale}"
        reference = oracle.linear(element, oracle.pack_rows(element, w), n, k, values,
                                  chain=[(oracle.ADD, runtime.read(bias))])
        assert np.abs(b - reference).max() <= TOLERANCE * scale


def test_the_static_scratch_product_allocates_nothing_after_its_first_call(runtime, oracle):
    n, k, rows = 300, 1024, 2
    w = oracle.Stream(43).normal(n * k, 0.0, 0.02).reshape(n, k)
    weights = [runtime.load(element, n, k, oracle.pack_rows(element, w)) for element in (nb.Q4K, nb.Q8_0)]
    x, out = runtime.tensor(rows, k), runtime.tensor(rows, n)
    runtime.write(x, oracle.Stream(47).normal(rows * k).reshape(rows, k))
    runtime.linear_static(weights[0], x, out)   # the set-up call of this device (if no test before made it)
    runtime.sync()
    free_before, _ = runtime.memory()
    for _ in range(3):
        for weight in weights:                  # both block formats, one and two rows: all four kernel variants
            runtime.linear_static(weight, x, out)
            runtime.linear_static(weight, x, out, rows=1)
    runtime.sync()
    free_after, _ = runtime.memory()
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes across allocation-free calls"


def test_the_static_scratch_product_refuses_what_it_cannot_hold(runtime, oracle):
    n, k = 64, 512
    w = oracle.Stream(5).normal(n * k, 0.0, 0.02).reshape(n, k)
    weight = runtime.load(nb.Q4K, n, k, oracle.pack_rows(nb.Q4K, w))
    x, out = runtime.tensor(5, k), runtime.tensor(5, n)
    with pytest.raises(nb.NeuraCudaError, match="at most 4 rows"):
        runtime.linear_static(weight, x, out)
