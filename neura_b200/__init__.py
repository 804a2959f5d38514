"""neura_b200: the B200 (sm_100a) quantized-linear path of Neura behind a C ABI.

``libneura_cuda.so`` (csrc/, built by ``neura_b200.build``) is the product; this
package is the thin host side that loads it and mirrors the reference's runtime
calls for the path.  Nothing here computes on the CPU.
"""
from .runtime import (  # noqa: F401
    ADD, MUL, SUB, DIV, MAXIMUM, MINIMUM, RELU, SQRT, RECIP, EXP, LOG, TANH, SIGMOID, NEG, ABS, IDENTITY,
    SIN, COS, POW, FLOOR, GELU, SILU, SINGLE, HALF, BFLOAT16, Q8_0, Q4K, Q5K, Q6K, Q3K, LAYOUT_GGUF, LAYOUT_TILED, LAYOUT_TILED_PAIR,
    DeviceTensor, NeuraCudaError, Runtime, Step, Weight, payload_bytes,
)
