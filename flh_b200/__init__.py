"""flh_b200 — FLH's W4A4 inference hot path (online Hadamard + int4 activation quantiser + int4
GEMM with fused dequantisation) on hand-written sm_100a kernels behind a C ABI.

    import flh_b200
    flh_b200._CUDA.install()      # optional: make an existing `flh` checkout run on these kernels
    from flh_b200.nn import ActQuantizer, LinearFLH

Importing the package loads libflh_b200.so and fails if it is missing: there is no fallback.
"""
import sys

from . import _lib

# `python -m flh_b200.build` imports this package before the library exists (or while it is stale);
# every other import loads the library now and fails if that is impossible.
if "flh_b200.build" not in getattr(sys, "orig_argv", []):
    _lib.load()

from . import _CUDA, functional, hadamard, nn  # noqa: E402

__all__ = ["_CUDA", "functional", "hadamard", "nn"]
