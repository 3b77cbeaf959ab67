"""joshua_b200: a B200 (sm_100a) implementation of the joshua engine's quantized-matmul path.

The product is the C-ABI shared library `libjoshua_b200.so` (declared in
`include/joshua_b200.h`, sources in `joshua_b200/csrc/`).  The Python modules are
the host-side mirror of the reference's operator interface, used by the tests
and the benchmark; they hold no arithmetic of their own.
"""
from .synth import IQ2_XXS, MXFP4, Q2_K, Q4_K, Q8_0  # noqa: F401

__all__ = ["Q8_0", "Q2_K", "Q4_K", "IQ2_XXS", "MXFP4"]
