"""ctypes binding of libflh_b200.so (the C ABI in include/flh_b200.h).

There is no fallback: if the library is missing or does not export a symbol the
import fails, and every call checks the returned status.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflh_b200.so")

c_void_p, c_long, c_int, c_size_t, c_float = ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_size_t, ctypes.c_float

# name -> (restype, argtypes); must list every symbol include/flh_b200.h declares
SIGNATURES = {
    "flh_b200_version": (c_int, []),
    "flh_b200_last_error": (ctypes.c_char_p, []),
    "flh_b200_device_check": (c_int, []),
    "flh_b200_quant_group_sym_i4": (c_int, [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "flh_b200_hadamard_f16_inplace": (c_int, [c_void_p, c_long, c_int, c_void_p]),
    "flh_b200_quant_token_asym_i4": (c_int, [c_void_p, c_int, c_long, c_long, c_long, c_int, c_int, c_void_p, c_float,
                                             c_void_p, c_void_p, c_void_p, c_void_p]),
    "flh_b200_quant_token_kernel": (ctypes.c_char_p, [c_long, c_long, c_int, c_int]),
    "flh_b200_silu_mul": (c_int, [c_void_p, c_int, c_long, c_long, c_long, c_void_p, c_void_p]),
    "flh_b200_silu_mul_quant_token_asym_i4": (c_int, [c_void_p, c_int, c_long, c_long, c_long, c_int, c_int, c_void_p, c_float,
                                                      c_void_p, c_void_p, c_void_p, c_void_p]),
    "flh_b200_rope_kv_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_void_p]),
    "flh_b200_gptq_block": (c_int, [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                    c_float, c_void_p, c_long, c_void_p, c_void_p]),
    "flh_b200_sign_table_bytes": (c_size_t, [c_int]),
    "flh_b200_pack_signs": (c_int, [c_void_p, c_int, c_void_p]),
    "flh_b200_weight_rowsum": (c_int, [c_void_p, c_long, c_long, c_long, c_void_p, c_void_p]),
    "flh_b200_gemm_i4_dequant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_long, c_long, c_long, c_long, c_long, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "flh_b200_gemm_i4_dequant_decode_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                        c_void_p, c_long, c_long, c_long, c_long, c_long, c_int, c_void_p]),
    "flh_b200_rmsnorm_quant_token_asym_i4": (c_int, [c_void_p, c_int, c_long, c_long, c_long, c_float, c_int, c_float, c_void_p,
                                                     c_void_p, c_void_p, c_void_p]),
    "flh_b200_rmsnorm_quant_group_sym_i4": (c_int, [c_void_p, c_long, c_long, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "flh_b200_expand_i4": (c_int, [c_void_p, c_long, c_long, c_void_p, c_void_p]),
    "flh_b200_gemm_i8w_dequant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_long, c_long, c_long, c_int, c_void_p, c_size_t, c_void_p]),
    "flh_b200_gemm_workspace_bytes": (c_size_t, [c_long, c_long, c_long, c_long, c_long, c_int]),
    "flh_b200_gemm_pick_algo": (c_int, [c_long, c_long, c_long, c_long, c_long]),
    "flh_b200_gemm_status": (c_int, [c_void_p]),
    "flh_b200_gemm_wait_profile": (c_int, [c_void_p]),
    "flh_b200_quant_token_wait_profile": (c_int, [c_void_p]),
    "flh_b200_ar_create": (c_int, [c_int, c_int, c_size_t, c_void_p]),
    "flh_b200_ar_export": (c_int, [c_void_p, c_void_p]),
    "flh_b200_ar_import": (c_int, [c_void_p, c_int, c_void_p]),
    "flh_b200_ar_attach": (c_int, [c_void_p, c_int, c_void_p]),
    "flh_b200_allreduce": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p]),
    "flh_b200_allreduce_ranks": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_void_p]),
    "flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_float, c_float,
                                                                   c_void_p, c_void_p, c_void_p, c_void_p]),
    "flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4_ranks": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_long, c_long, c_int, c_float,
                                                                         c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "flh_b200_ar_status": (c_int, [c_void_p, c_void_p]),
    "flh_b200_ar_destroy": (c_int, [c_void_p]),
    "flhDenseLayerGEMM_i4_o16": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m flh_b200.build` (nvcc, sm_100a). "
                "flh_b200 has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the build is stale
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().flh_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (status {rc}): {msg}")
