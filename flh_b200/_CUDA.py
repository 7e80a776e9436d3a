"""Drop-in for the `flh._CUDA` extension module (flh/cuda/flh_cuda_bindings.cpp:301-313).

Same nine function names, argument order, validation (RuntimeError, as TORCH_CHECK raises) and
return values; every call goes through the C ABI of libflh_b200.so on the tensor's device and the
current torch stream.  `install()` binds this module to `flh._CUDA`, which every FLH call site
resolves at call time (flh/nn/quantization.py:127,158,161; flh/nn/linear.py:128).

Extended entry points for the per-token asymmetric mode follow the same conventions.
PyTorch is used only for device memory, streams and the device guard.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import _lib
from .hadamard import get_hadK

F16, BF16 = 0, 1
GEMM_AUTO, GEMM_TCGEN05, GEMM_MMA_SYNC, GEMM_STREAM, GEMM_STREAM_SPLITK, GEMM_TCGEN05_DIRECT = 0, 1, 2, 3, 4, 5
GEMM_TCGEN05_I8, GEMM_TCGEN05_I8_PAIR, GEMM_DECODE_TC = 6, 7, 8


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _guard(device):
    """Device guard around a C-ABI call (the library launches on the current device)."""
    return torch.cuda.device(device)


# --------------------------------------------------------------------------- the nine pybind names
def gemm_i4_dequant_o16(A, B, A_scale, B_scale):
    """flh/cuda/flh_cuda_bindings.cpp:75-113.  u8[M,K/2], u8[N,K/2], f16[M,*], f16[N,*] -> f16[M,N]."""
    _check(A.is_cuda and B.is_cuda and A_scale.is_cuda and B_scale.is_cuda, "tensors must be CUDA")
    _check(A.dtype == torch.uint8, "A must be uint8 packed int4")
    _check(B.dtype == torch.uint8, "B must be uint8 packed int4")
    _check(A_scale.dtype == torch.float16, "A_scale must be float16")
    _check(B_scale.dtype == torch.float16, "B_scale must be float16")
    _check(A.is_contiguous() and B.is_contiguous() and A_scale.is_contiguous() and B_scale.is_contiguous(),
           "tensors must be contiguous")
    _check(A.dim() == 2 and B.dim() == 2, "A/B must be 2D")
    _check(A_scale.dim() == 2 and B_scale.dim() == 2, "scale must be 2D")
    M, Kp = A.shape
    N = B.shape[0]
    _check(B.shape[1] == Kp, "B.shape[1] must equal A.shape[1]")
    _check(A_scale.shape[0] == M, "A_scale.shape[0] must equal M")
    _check(B_scale.shape[0] == N, "B_scale.shape[0] must equal N")
    return gemm_i4_dequant(A, B, A_scale, B_scale)


def _fht(x, n):
    _check(x.is_cuda, "Input tensor must be on CUDA")
    _check(x.dtype == torch.float16, "Input tensor must be float16 (half)")
    _check(x.dim() == 2, "Input tensor must be 2D")
    _check(x.shape[1] == n, f"Last dimension must be {n}")
    _check(x.is_contiguous(), "Input tensor must be contiguous")
    with _guard(x.device):
        _lib.check(_lib.load().flh_b200_hadamard_f16_inplace(_ptr(x), x.shape[0], n, _stream(x)), "hadamard_transform")
    return x


def hadamard_transform_half(x):
    """In place, un-normalised, rows of 128 (flh/cuda/flh_cuda_bindings.cpp:115-126)."""
    return _fht(x, 128)


def hadamard_transform_64_half(x):
    return _fht(x, 64)


def hadamard_transform_32_half(x):
    return _fht(x, 32)


def _quant_group(x, gs, hadamard):
    _check(x.is_cuda, "Input tensor must be on CUDA")
    _check(x.dtype == torch.float16, "Input tensor must be float16 (half)")
    _check(x.dim() == 2, "Input tensor must be 2D")
    _check(gs in (32, 64, 128), "group_size must be 32, 64, or 128")
    _check(x.shape[1] == gs, "Last dimension must equal group_size" if gs != 128 else "Last dimension must be 128")
    _check(x.is_contiguous(), "Input tensor must be contiguous")
    rows = x.shape[0]
    q = torch.empty((rows, gs // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows,), dtype=torch.float16, device=x.device)
    with _guard(x.device):
        _lib.check(_lib.load().flh_b200_quant_group_sym_i4(_ptr(x), rows, gs, int(hadamard), _ptr(q), _ptr(s), _stream(x)),
                   "quant_group_sym_i4")
    return [q, s]


def hadamard_and_quantize_i4(x):
    """f16[R,128] -> [u8[R,64], f16[R]] (raw scale) — flh/cuda/flh_cuda_bindings.cpp:154-175."""
    return _quant_group(x, 128, True)


def quant_and_pack_i4(x):
    """flh/cuda/flh_cuda_bindings.cpp:177-198."""
    return _quant_group(x, 128, False)


def hadamard_and_quantize_i4_gs(x, group_size):
    """flh/cuda/flh_cuda_bindings.cpp:202-225."""
    return _quant_group(x, int(group_size), True)


def quant_and_pack_i4_gs(x, group_size):
    """flh/cuda/flh_cuda_bindings.cpp:227-251."""
    return _quant_group(x, int(group_size), False)


def gemm_i4_dequant_o16_gs(A, B, A_scale, B_scale, group_size):
    """flh/cuda/flh_cuda_bindings.cpp:253-299: u8[M,K/2], u8[N,K/2], f16[M,K/gs], f16[N,K/gs], gs in {32,64,128}
    -> f16[M,N].  Every K-group of gs elements is scaled with its own pair of scales (the reference kernel,
    flh/kernels/gemm_and_dequant_i4_gs.cu:408, applies the first scale of each 128-K block to the whole block,
    which is only right for gs = 128)."""
    _check(A.is_cuda and B.is_cuda and A_scale.is_cuda and B_scale.is_cuda, "tensors must be CUDA")
    _check(A.dtype == torch.uint8 and B.dtype == torch.uint8, "A and B must be uint8 packed int4")
    _check(A_scale.dtype == torch.float16 and B_scale.dtype == torch.float16, "scales must be float16")
    _check(A.is_contiguous() and B.is_contiguous() and A_scale.is_contiguous() and B_scale.is_contiguous(),
           "tensors must be contiguous")
    _check(group_size in (32, 64, 128), "group_size must be 32, 64, or 128")
    _check(A.dim() == 2 and B.dim() == 2, "A/B must be 2D")
    _check(A_scale.dim() == 2 and B_scale.dim() == 2, "scale must be 2D")
    _check(B.shape[1] == A.shape[1], "B.shape[1] must equal A.shape[1]")
    K = A.shape[1] * 2
    _check(K % group_size == 0, "K must be divisible by group_size")
    g = K // group_size
    _check(A_scale.shape[0] == A.shape[0], "A_scale.shape[0] must equal M")
    _check(A_scale.shape[1] == g, "A_scale.shape[1] must equal K/group_size")
    _check(B_scale.shape[0] == B.shape[0], "B_scale.shape[0] must equal N")
    _check(B_scale.shape[1] == g, "B_scale.shape[1] must equal K/group_size")
    return gemm_i4_dequant(A, B, A_scale, B_scale)


# --------------------------------------------------------------------------- extended entry points
_SIGN_CACHE: dict = {}


def _sign_bits(n: int, device):
    """(kfac, device uint32 bit rows or None) for width n, cached per (width, device)."""
    key = (n, str(device))
    hit = _SIGN_CACHE.get(key)
    if hit is not None:
        return hit
    signs, k = get_hadK(n)
    if k == 1:
        _SIGN_CACHE[key] = (1, None)
        return _SIGN_CACHE[key]
    tkey = ("table", k, str(device))
    if tkey not in _SIGN_CACHE:
        s8 = np.ascontiguousarray(signs, dtype=np.int8)
        out = np.zeros((_lib.load().flh_b200_sign_table_bytes(k) + 3) // 4, dtype=np.uint32)
        _lib.check(_lib.load().flh_b200_pack_signs(s8.ctypes.data_as(ctypes.c_void_p), k,
                                                   out.ctypes.data_as(ctypes.c_void_p)), "pack_signs")
        _SIGN_CACHE[tkey] = torch.from_numpy(out.view(np.int32)).to(device)
    _SIGN_CACHE[key] = (k, _SIGN_CACHE[tkey])
    return _SIGN_CACHE[key]


def quant_token_asym_i4(x, hadamard: bool = True, clip: float = 1.0, exact: bool = False, exact_factor=None, out=None):
    """x [M, K] f16/bf16 (row stride allowed) -> (q u8[M,K/2] codes 0..15, scale f16[M], zero f16[M]).
    hadamard=True applies the full-width transform of matmul_hadU (flh/functional/hadamard.py:92-113)
    before the per-token asymmetric quantiser of fake_quant/quant_utils.py:94-128.  By default the high part
    of the transform (the kfac x kfac factor and the butterfly bits above 64) is summed by the tensor cores
    (K = P * 64, P <= 512): same values up to the order of binary32 additions, the same order for every
    batch size.  exact=True keeps the sequential order of the reference (bit-exact with the CPU oracle,
    slower).  out=(q, scale, zero) writes into caller tensors instead of allocating."""
    if exact_factor is not None:        # earlier name of `exact`
        exact = bool(exact_factor)
    _check(x.is_cuda, "Input tensor must be on CUDA")
    _check(x.dtype in (torch.float16, torch.bfloat16), "Input tensor must be float16 or bfloat16")
    _check(x.dim() == 2 and x.stride(1) == 1, "Input tensor must be 2D with unit inner stride")
    M, K = x.shape
    kfac, bits = _sign_bits(K, x.device) if hadamard else (1, None)
    if out is not None:
        q, s, z = out
        _check(q.dtype == torch.uint8 and q.is_contiguous() and q.numel() == M * (K // 2) and q.device == x.device, "out[0] must be contiguous uint8 [M, K/2]")
        _check(s.dtype == torch.float16 and s.numel() == M and z.dtype == torch.float16 and z.numel() == M and s.is_contiguous() and z.is_contiguous(),
               "out[1], out[2] must be contiguous float16 [M]")
    else:
        q = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
        s = torch.empty((M,), dtype=torch.float16, device=x.device)
        z = torch.empty((M,), dtype=torch.float16, device=x.device)
    with _guard(x.device):
        _lib.check(_lib.load().flh_b200_quant_token_asym_i4(
            _ptr(x), BF16 if x.dtype == torch.bfloat16 else F16, M, K, x.stride(0) if M > 1 else K,
            (2 if exact else 1) if hadamard else 0, kfac,
            _ptr(bits), float(clip), _ptr(q), _ptr(s), _ptr(z), _stream(x)), "quant_token_asym_i4")
    return q, s, z


def silu_mul(gu):
    """SiLU(gate) * up of the merged gate/up GEMM output gu [M, 2F] (row stride allowed) -> [M, F] (include/flh_b200.h)."""
    _check(gu.is_cuda and gu.dtype in (torch.float16, torch.bfloat16), "gu must be a CUDA float16 or bfloat16 tensor")
    _check(gu.dim() == 2 and gu.stride(1) == 1 and gu.shape[1] % 2 == 0, "gu must be [M, 2F] with unit inner stride")
    M, F = gu.shape[0], gu.shape[1] // 2
    out = torch.empty((M, F), dtype=gu.dtype, device=gu.device)
    with _guard(gu.device):
        _lib.check(_lib.load().flh_b200_silu_mul(_ptr(gu), BF16 if gu.dtype == torch.bfloat16 else F16, M, F,
                                                 gu.stride(0) if M > 1 else 2 * F, _ptr(out), _stream(gu)), "silu_mul")
    return out


def silu_mul_quant_token_asym_i4(gu, hadamard: bool = True, clip: float = 1.0, exact: bool = False, fused: bool = False):
    """SiLU(gate) * up of gu [M, 2F], then (optionally the full-width transform and) the per-token asymmetric quantiser.
    -> (q u8[M, F/2], scale f16[M], zero f16[M]).

    Default: silu_mul followed by quant_token_asym_i4 (two launches).  `fused=True` runs the single-kernel form when the
    tensor-core quantiser takes the width (hadamard=True, exact=False, F = P * 64 with P <= 256): the same bits, but measured
    SLOWER than the pair at every batch size on B200 (F = 11008: 18.6 vs 11.1 us at 16 rows, 171 vs 113 us at 4096 rows) —
    its epilogue warps, already the limit of the quantiser, also have to make the SiLU rows — so nothing uses it by default."""
    _check(gu.is_cuda and gu.dtype in (torch.float16, torch.bfloat16), "gu must be a CUDA float16 or bfloat16 tensor")
    _check(gu.dim() == 2 and gu.stride(1) == 1 and gu.shape[1] % 2 == 0, "gu must be [M, 2F] with unit inner stride")
    M, F = gu.shape[0], gu.shape[1] // 2
    lib = _lib.load()
    if fused and hadamard and not exact and M > 0:
        kfac, bits = _sign_bits(F, gu.device)
        # the fused form makes whole rows in shared memory: widths up to P = 256 only (wider rows are read as two halves)
        if F // 64 <= 256 and lib.flh_b200_quant_token_kernel(M, F, 1, kfac) == b"quant_token_tc_kernel":
            q = torch.empty((M, F // 2), dtype=torch.uint8, device=gu.device)
            s = torch.empty((M,), dtype=torch.float16, device=gu.device)
            z = torch.empty((M,), dtype=torch.float16, device=gu.device)
            with _guard(gu.device):
                _lib.check(lib.flh_b200_silu_mul_quant_token_asym_i4(
                    _ptr(gu), BF16 if gu.dtype == torch.bfloat16 else F16, M, F, gu.stride(0) if M > 1 else 2 * F, 1, kfac,
                    _ptr(bits), float(clip), _ptr(q), _ptr(s), _ptr(z), _stream(gu)), "silu_mul_quant_token_asym_i4")
            return q, s, z
    return quant_token_asym_i4(silu_mul(gu), hadamard=hadamard, clip=clip, exact=exact)


def rope_kv(qkv, cos, sin, q_out, k_cache, v_cache, B, S, nh, nkv, cur):
    """Rotary embedding of q and k + KV-cache write from the merged QKV GEMM output (include/flh_b200.h: flh_b200_rope_kv_f16).
    qkv f16 [B*S, (nh + 2 nkv) * D] contiguous; cos, sin f32 [S, D/2]; q_out [B, nh, S, D]; caches [B, nkv, T, D] contiguous."""
    _check(qkv.is_cuda and qkv.dtype == torch.float16 and qkv.is_contiguous(), "qkv must be a contiguous CUDA float16 tensor")
    _check(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(), "cos / sin must be contiguous float32")
    _check(q_out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(), "outputs must be contiguous")
    D = q_out.shape[-1]
    with _guard(qkv.device):
        _lib.check(_lib.load().flh_b200_rope_kv_f16(_ptr(qkv), _ptr(cos), _ptr(sin), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                                    B, S, nh, nkv, D, k_cache.shape[2], cur, _stream(qkv)), "rope_kv")
    return q_out


def rmsnorm_quant_token_asym_i4(x, eps: float, hadamard: bool = False, clip: float = 1.0):
    """RMS-norm (weight 1) + per-token asymmetric int4 in one pass, K = 4096 or 8192 (include/flh_b200.h).
    x [M, K] f16/bf16 (row stride allowed) -> (q u8[M,K/2], scale f16[M], zero f16[M])."""
    _check(x.is_cuda, "Input tensor must be on CUDA")
    _check(x.dtype in (torch.float16, torch.bfloat16), "Input tensor must be float16 or bfloat16")
    _check(x.dim() == 2 and x.stride(1) == 1, "Input tensor must be 2D with unit inner stride")
    M, K = x.shape
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((M,), dtype=torch.float16, device=x.device)
    z = torch.empty((M,), dtype=torch.float16, device=x.device)
    with _guard(x.device):
        _lib.check(_lib.load().flh_b200_rmsnorm_quant_token_asym_i4(
            _ptr(x), BF16 if x.dtype == torch.bfloat16 else F16, M, K, x.stride(0), float(eps), int(hadamard), float(clip),
            _ptr(q), _ptr(s), _ptr(z), _stream(x)), "rmsnorm_quant_token_asym_i4")
    return q, s, z


def rmsnorm_quant_group_sym_i4(x, eps: float, hadamard: bool = False):
    """RMS-norm (weight 1) + group-128 symmetric int4 in one pass: x f16 [M, 4096] -> [q u8[M*32, 64], scale f16[M*32]]."""
    _check(x.is_cuda and x.dtype == torch.float16 and x.dim() == 2 and x.is_contiguous(), "x must be a contiguous CUDA float16 matrix")
    M, K = x.shape
    q = torch.empty((M * (K // 128), 64), dtype=torch.uint8, device=x.device)
    s = torch.empty((M * (K // 128),), dtype=torch.float16, device=x.device)
    with _guard(x.device):
        _lib.check(_lib.load().flh_b200_rmsnorm_quant_group_sym_i4(_ptr(x), M, K, float(eps), int(hadamard), _ptr(q), _ptr(s), _stream(x)),
                   "rmsnorm_quant_group_sym_i4")
    return [q, s]


def weight_rowsum(B, group: int):
    """int32 [N, K/group] sums of the signed weight codes (needed with zero-points)."""
    _check(B.is_cuda and B.dtype == torch.uint8 and B.dim() == 2 and B.is_contiguous(), "B must be a contiguous CUDA uint8 matrix")
    N, K = B.shape[0], B.shape[1] * 2
    rs = torch.empty((N, K // group), dtype=torch.int32, device=B.device)
    with _guard(B.device):
        _lib.check(_lib.load().flh_b200_weight_rowsum(_ptr(B), N, K, group, _ptr(rs), _stream(B)), "weight_rowsum")
    return rs


_WORKSPACES: dict = {}


def _workspace(device, stream: int, nbytes: int):
    """Zero-initialised scratch for the split-K decode kernel, one per (device, stream): launches on one
    stream run in order, so they may share it; the kernel leaves its counters zeroed."""
    key = (str(device), stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 8 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


_SCRATCH: dict = {}


def _scratch(device, stream: int, nbytes: int):
    """Uninitialised scratch for the int8-operand GEMM (the expanded operands), one per (device, stream); kept
    apart from the zeroed split-K workspace, whose counters it would overwrite."""
    key = (str(device), stream)
    ws = _SCRATCH.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _SCRATCH[key] = ws
    return ws


def gemm_i4_dequant(A, B, A_scale, B_scale, A_zero=None, B_rowsum=None, bias=None,
                    out_dtype=torch.float16, algo: int = GEMM_AUTO, out=None):
    """General form of the GEMM (include/flh_b200.h: flh_b200_gemm_i4_dequant).  Scale granularity
    is read off the scale shapes: a_group = K / A_scale.shape[1], b_group = K / B_scale.shape[1]."""
    M, Kp = A.shape
    N = B.shape[0]
    K = Kp * 2
    A_scale = A_scale.reshape(M, -1)
    B_scale = B_scale.reshape(N, -1)
    _check(A_scale.shape[1] > 0 and K % A_scale.shape[1] == 0, "A_scale columns must divide K")
    _check(B_scale.shape[1] > 0 and K % B_scale.shape[1] == 0, "B_scale columns must divide K")
    ag, bg = K // A_scale.shape[1], K // B_scale.shape[1]
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=A.device)
    lib = _lib.load()
    with _guard(A.device):
        stream = _stream(A)
        need = lib.flh_b200_gemm_workspace_bytes(M, N, K, ag, bg, algo)
        resolved = algo if algo != GEMM_AUTO else lib.flh_b200_gemm_pick_algo(M, N, K, ag, bg)
        if not need:
            ws = None
        elif resolved in (GEMM_TCGEN05_I8, GEMM_TCGEN05_I8_PAIR):
            ws = _scratch(A.device, stream, need)          # expanded operands: any contents
        else:
            ws = _workspace(A.device, stream, need)        # split-K: zeroed counters, left zeroed
        _lib.check(lib.flh_b200_gemm_i4_dequant(
            _ptr(A), _ptr(B), _ptr(A_scale), _ptr(A_zero), _ptr(B_scale), _ptr(B_rowsum), _ptr(bias), _ptr(D),
            M, N, K, ag, bg, BF16 if D.dtype == torch.bfloat16 else F16, algo, _ptr(ws), ws.numel() if ws is not None else 0,
            stream), "gemm_i4_dequant")
    return D


def expand_i4(B):
    """Packed int4 weights u8[N, K/2] -> the int8 copy u8[N, K] (16 * q) that gemm_i8w_dequant multiplies."""
    _check(B.is_cuda and B.dtype == torch.uint8 and B.dim() == 2 and B.is_contiguous(), "B must be a contiguous CUDA uint8 matrix")
    N, Kp = B.shape
    out = torch.empty((N, 2 * Kp), dtype=torch.uint8, device=B.device)
    with _guard(B.device):
        _lib.check(_lib.load().flh_b200_expand_i4(_ptr(B), N, 2 * Kp, _ptr(out), _stream(B)), "expand_i4")
    return out


def gemm_i8w_dequant(A, B8, A_scale, B_scale, A_zero=None, B_rowsum=None, bias=None, out_dtype=torch.float16, out=None):
    """The GEMM with per-token / per-channel scales on weights expanded ahead of time by expand_i4 (prefill batches)."""
    M, Kp = A.shape
    N, K = B8.shape
    _check(K == 2 * Kp, "B8 must be [N, K] for A [M, K/2]")
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=A.device)
    with _guard(A.device):
        stream = _stream(A)
        ws = _scratch(A.device, stream, M * K)
        _lib.check(_lib.load().flh_b200_gemm_i8w_dequant(
            _ptr(A), _ptr(B8), _ptr(A_scale), _ptr(A_zero), _ptr(B_scale), _ptr(B_rowsum), _ptr(bias), _ptr(D),
            M, N, K, BF16 if D.dtype == torch.bfloat16 else F16, _ptr(ws), ws.numel(), stream), "gemm_i8w_dequant")
    return D


def gemm_status():
    """[code, cta, 0, 0] of the tcgen05 GEMM's bounded waits; synchronises.  0 = clean."""
    out = (ctypes.c_int * 4)()
    _lib.check(_lib.load().flh_b200_gemm_status(out), "gemm_status")
    return list(out)


def gemm_wait_profile():
    """Nanoseconds the tcgen05 GEMM's roles waited on each other since the last call (see the header)."""
    out = (ctypes.c_ulonglong * 8)()
    _lib.check(_lib.load().flh_b200_gemm_wait_profile(out), "gemm_wait_profile")
    return list(out)


def quant_token_wait_profile():
    """Nanoseconds the roles of the tensor-core token quantiser waited on each other since the last call (see the header)."""
    out = (ctypes.c_ulonglong * 8)()
    _lib.check(_lib.load().flh_b200_quant_token_wait_profile(out), "quant_token_wait_profile")
    return list(out)


def install():
    """Bind this module as `flh._CUDA` so unmodified flh.nn / flh.quantized_model code runs on it."""
    import sys
    import flh  # the FLH package must be importable
    flh._CUDA = sys.modules[__name__]
    return flh
