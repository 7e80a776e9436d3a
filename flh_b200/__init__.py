"""flh_b200 — FLH's W4A4 inference hot path (online Hadamard + int4 activation quantiser + int4
GEMM with fused dequantisation) on hand-written sm_100a kernels behind a C ABI.

    import flh_b200
    flh_b200._CUDA.install()      # optional: make an existing `flh` checkout run on these kernels
    from flh_b200.nn import ActQuantizer, LinearFLH

Importing the package loads libflh_b200.so and fails if it is missing: there is no fallback.
"""
from . import _lib

_lib.load()

from . import _CUDA, functional, hadamard, nn  # noqa: E402

__all__ = ["_CUDA", "functional", "hadamard", "nn"]
