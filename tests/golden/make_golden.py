"""Writes tests/golden/blocks.npz: frozen inputs and outputs of the CPU oracle.

The reference holds no known-answer vectors for Q8_0 / Q4_K bytes and cannot be run in
this environment, so these vectors do not pin the oracle to the reference; they freeze
the oracle (and, through the GPU tests, the CUDA path) against regressions.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def main() -> None:
    out = {}
    out["uniform_seed23"] = oracle.random(64, 23)
    out["normal_seed23"] = oracle.Stream(23).normal(64, 0.0, 0.02)
    for name, element, n, k in (("q8_0", oracle.Q8_0, 4, 96), ("q4k", oracle.Q4K, 3, 512)):
        w = oracle.Stream(23).normal(n * k, 0.0, 0.02).reshape(n, k)
        w[0, :8] = 0.0
        w[1, 5] = -0.0
        packed = oracle.pack_rows(element, w)
        x = oracle.random(2 * k, 29).reshape(2, k)
        out[f"{name}_weight"] = w
        out[f"{name}_packed"] = packed
        out[f"{name}_unpacked"] = oracle.unpack(element, n * k, packed).reshape(n, k)
        out[f"{name}_x"] = x
        out[f"{name}_product"] = oracle.linear(element, packed, n, k, x)
        bias = oracle.random(n, 31)
        out[f"{name}_bias"] = bias
        out[f"{name}_chain"] = oracle.linear(element, packed, n, k, x, chain=[(oracle.ADD, bias), (oracle.SILU, None)])
    # edge blocks: zeros, one constant, all positive, all negative, a huge outlier
    edge = np.zeros((5, 256), dtype=np.float32)
    edge[1] = 0.75
    edge[2] = np.abs(oracle.Stream(3).normal(256)) + 0.1
    edge[3] = -np.abs(oracle.Stream(4).normal(256)) - 0.1
    edge[4] = oracle.Stream(6).normal(256, 0.0, 0.02)
    edge[4, 17] = 1.0e4
    out["edge_weight"] = edge
    out["edge_q8_0"] = oracle.pack_rows(oracle.Q8_0, edge)
    out["edge_q4k"] = oracle.pack_rows(oracle.Q4K, edge)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "blocks.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
