"""numpy front end of the CPU oracle (oracle/flh_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke entry and by the
CPU-baseline leg of bench.py.  The shipped package never imports this module.

Each function cites the reference file it restates (paths relative to the FLH
repository root).  binary16 tensors are numpy float16 arrays; bfloat16 travels
as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i8p = ctypes.POINTER(ctypes.c_int8)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def build() -> str:
    """Compile oracle/flh_oracle.c with gcc (a few seconds) and return the .so path."""
    so = os.path.join(_HERE, "libflh_oracle.so")
    src = os.path.join(_HERE, "flh_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libflh_oracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
    return _LIB


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


def _threads() -> int:
    return max(1, os.cpu_count() or 1)


# ----------------------------------------------------------------------------- nibbles
def pack_i4(q: np.ndarray) -> np.ndarray:
    """Two's-complement nibbles, low nibble = even index.
    Restates pack_i4, flh/functional/quantization.py:42-49."""
    q = np.asarray(q).astype(np.int16)
    assert q.min() >= -8 and q.max() <= 15
    u = (q & 15).astype(np.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


def unpack_i4(p: np.ndarray, signed: bool = True) -> np.ndarray:
    """Inverse of pack_i4.  Restates unpack_i4, flh/functional/quantization.py:52-74
    (signed) and LinearFLH._unpack_activation_4bit, flh/nn/linear.py:287-324 (unsigned)."""
    p = np.asarray(p, dtype=np.uint8)
    lo = (p & 15).astype(np.int32)
    hi = (p >> 4).astype(np.int32)
    if signed:
        lo = np.where(lo >= 8, lo - 16, lo)
        hi = np.where(hi >= 8, hi - 16, hi)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.int32)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


# ----------------------------------------------------------------------------- Hadamard tables
_ORDER = (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)


def get_hadK(n: int):
    """(K x K int8 +-1 matrix or None, K): the factor get_hadK picks for width n,
    flh/functional/hadamard.py:39-89 (same precedence of the n % K tests)."""
    for k in _ORDER:
        if n % k == 0:
            p = n // k
            assert p & (p - 1) == 0, "n / K must be a power of two"
            z = np.load(os.path.join(_HERE, "..", "flh_b200", "data", "hadk_signs.npz"))
            bits = np.unpackbits(z[f"had{k}"])[: k * k].reshape(k, k)
            return (1 - 2 * bits.astype(np.int8)).astype(np.int8), k
    assert n & (n - 1) == 0 and n > 0
    return None, 1


# ----------------------------------------------------------------------------- transforms
def fht_f16(x: np.ndarray) -> np.ndarray:
    """Un-normalised binary16 WHT of every row (row length 32/64/128).
    Restates hadamard_transform_kernel_optimized, flh/kernels/cuda_had_kernel.cu:190-268."""
    x = np.ascontiguousarray(x, dtype=np.float16).copy()
    lib().flh_oracle_fht_f16(_p(x.view(np.uint16), _u16p), ctypes.c_long(x.shape[0]), ctypes.c_int(x.shape[1]))
    return x


def had_full_f32(x: np.ndarray) -> np.ndarray:
    """y = (hadK (x) H_p) x / sqrt(n) in binary32; restates matmul_hadU,
    flh/functional/hadamard.py:92-113."""
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    n = x.shape[-1]
    signs, k = get_hadK(n)
    x2 = x.reshape(-1, n)
    lib().flh_oracle_had_full_f32(_p(x2, _f32p), ctypes.c_long(x2.shape[0]), ctypes.c_long(n),
                                  ctypes.c_int(k), _p(signs, _i8p))
    return x2.reshape(x.shape)


# ----------------------------------------------------------------------------- quantisers
def quant_group_sym(x: np.ndarray, hadamard: bool):
    """x [R, gs] float16 -> (packed [R, gs/2] uint8, raw scale [R] float16).
    Restates had_and_quant_kernel, flh/kernels/had_and_quant.cu:61-155 (hadamard=True)
    and quant_and_pack_kernel, flh/kernels/quant_and_pack.cu:8-96 (hadamard=False)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    r, gs = x.shape
    q = np.empty((r, gs // 2), dtype=np.uint8)
    s = np.empty((r,), dtype=np.float16)
    lib().flh_oracle_quant_group_sym(_p(x.view(np.uint16), _u16p), ctypes.c_long(r), ctypes.c_int(gs),
                                     ctypes.c_int(int(hadamard)), _p(q, _u8p), _p(s.view(np.uint16), _u16p))
    return q, s


def quant_token_asym(x: np.ndarray, hadamard: bool, clip: float = 1.0, exact_norm: bool = False,
                     bf16: bool = False):
    """x [M, n] (float16, or uint16 bfloat16 bits when bf16) ->
    (packed [M, n/2] uint8 codes 0..15, scale [M] float16, zero [M] float16).
    Restates matmul_hadU (flh/functional/hadamard.py:92-113) followed by the
    per-token asymmetric quantiser of fake_quant/quant_utils.py:94-128, 17-21.
    exact_norm selects the reference's per-element normalisation; the default
    is the arithmetic of the B200 kernel (normalisation folded into the scale)."""
    xx = np.ascontiguousarray(x).view(np.uint16) if bf16 else np.ascontiguousarray(x, dtype=np.float16).view(np.uint16)
    m, n = xx.shape
    signs, k = get_hadK(n) if hadamard else (None, 1)
    q = np.empty((m, n // 2), dtype=np.uint8)
    s = np.empty((m,), dtype=np.float16)
    z = np.empty((m,), dtype=np.float16)
    lib().flh_oracle_quant_token_asym(_p(xx, _u16p), ctypes.c_int(int(bf16)), ctypes.c_long(m), ctypes.c_long(n),
                                      ctypes.c_long(n), ctypes.c_int(int(hadamard)), ctypes.c_int(k),
                                      _p(signs, _i8p), ctypes.c_float(clip), ctypes.c_int(int(exact_norm)),
                                      _p(q, _u8p), _p(s.view(np.uint16), _u16p), _p(z.view(np.uint16), _u16p))
    return q, s, z


def rmsnorm16(x: np.ndarray, eps: float, bf16: bool = False) -> np.ndarray:
    """RMS-norm (weight 1) of x [M, K] (float16, or uint16 bfloat16 bits) into the same 16-bit type, K = 4096 or
    8192, in the summation order of the fused B200 kernel.  Restates flh/nn/normalization.py up to that order."""
    xx = np.ascontiguousarray(x).view(np.uint16)
    m, k = xx.shape
    assert k % 4096 == 0
    y = np.empty((m, k), dtype=np.uint16)
    lib().flh_oracle_rmsnorm16(_p(xx, _u16p), ctypes.c_int(int(bf16)), ctypes.c_long(m), ctypes.c_long(k), ctypes.c_long(k),
                               ctypes.c_float(eps), _p(y, _u16p))
    return y if bf16 else y.view(np.float16)


# ----------------------------------------------------------------------------- weights (offline side)
def silu_mul16(gu: np.ndarray, bf16: bool = False) -> np.ndarray:
    """SiLU(gate) * up of a merged [M, 2F] gate/up matrix (float16, or uint16 bfloat16 bits) -> [M, F], with the
    arithmetic the fused kernels define (flh_oracle.c: flh_oracle_silu_mul16)."""
    xx = np.ascontiguousarray(gu)
    m, f2 = xx.shape
    out = np.empty((m, f2 // 2), dtype=np.uint16)
    lib().flh_oracle_silu_mul16(_p(xx.view(np.uint16), _u16p), ctypes.c_int(int(bf16)), ctypes.c_long(m), ctypes.c_long(f2 // 2),
                                ctypes.c_long(f2), _p(out, _u16p))
    return out if bf16 else out.view(np.float16)


def rtn_group_sym(w: np.ndarray, group: int = 128):
    """Symmetric RTN int4 with one scale per (row, group).
    Restates WeightQuantizer._calibrate_group_wise / _quantize_group_wise,
    flh/nn/quantization.py:374-406, 467-476: scale = max|w| / 7 clamped to >= 1e-8,
    q = clamp(round(w / scale), -8, 7), all in the dtype of w."""
    n, k = w.shape
    wg = w.reshape(n, k // group, group)
    scale = np.maximum(np.abs(wg).max(axis=2, keepdims=True) / w.dtype.type(7), w.dtype.type(1e-8))
    q = np.clip(np.rint(wg / scale), -8, 7).reshape(n, k).astype(np.int8)
    return q, scale.reshape(n, k // group)


def rtn_channel_sym(w: np.ndarray):
    """Symmetric RTN int4 with one scale per output row.
    Restates WeightQuantizer.find_params (perchannel, sym), fake_quant/quant_utils.py:244-256:
    xmax = max(|min(w,0)|, max(w,0)) clamped to >= 1e-5; scale = xmax / 7."""
    xmin = np.minimum(w.min(axis=1), 0)
    xmax = np.maximum(w.max(axis=1), 0)
    xmax = np.maximum(np.maximum(np.abs(xmin), xmax), w.dtype.type(1e-5))
    scale = (xmax / w.dtype.type(7)).reshape(-1, 1)
    q = np.clip(np.rint(w / scale), -8, 7).astype(np.int8)
    return q, scale


def weight_rowsum(b_packed: np.ndarray, group: int) -> np.ndarray:
    """rs[n, g] = sum of the signed weight codes of row n in K-group g (int32)."""
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    n, k = b.shape[0], b.shape[1] * 2
    rs = np.empty((n, k // group), dtype=np.int32)
    lib().flh_oracle_weight_rowsum(_p(b, _u8p), ctypes.c_long(n), ctypes.c_long(k), ctypes.c_long(group), _p(rs, _i32p))
    return rs


# ----------------------------------------------------------------------------- GEMM
def gemm_i4_int32(a_packed, b_packed, group: int, a_unsigned: bool = False) -> np.ndarray:
    """Exact int32 partial sums C[m, n, g]; the accumulators of
    flh_gemm_i4_dequant_o16_kernel, flh/kernels/gemm_and_dequant_i4.cu:199-240."""
    a = np.ascontiguousarray(a_packed, dtype=np.uint8)
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    m, k = a.shape[0], a.shape[1] * 2
    n = b.shape[0]
    c = np.empty((m, n, k // group), dtype=np.int32)
    lib().flh_oracle_gemm_i4_int32(_p(a, _u8p), _p(b, _u8p), ctypes.c_long(m), ctypes.c_long(n), ctypes.c_long(k),
                                   ctypes.c_long(group), ctypes.c_int(int(a_unsigned)), _p(c, _i32p))
    return c


def gemm_i4_dequant(a_packed, b_packed, a_scale, b_scale, a_zero=None, bias=None, bf16_out: bool = False):
    """D = dequantising int4 GEMM.  a_scale [M, Ga], b_scale [N, Gb] float16 (the
    granularity along K is K / columns), a_zero like a_scale (unsigned codes) or None.
    Restates flh_gemm_i4_dequant_o16_kernel, flh/kernels/gemm_and_dequant_i4.cu:287-313, 315-469.
    Output float16, or uint16 bfloat16 bits.  Rows of B are split over host threads."""
    a = np.ascontiguousarray(a_packed, dtype=np.uint8)
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    m, k = a.shape[0], a.shape[1] * 2
    n = b.shape[0]
    a_scale = np.ascontiguousarray(a_scale, dtype=np.float16).reshape(m, -1)
    b_scale = np.ascontiguousarray(b_scale, dtype=np.float16).reshape(n, -1)
    ag, bg = k // a_scale.shape[1], k // b_scale.shape[1]
    if a_zero is not None:
        a_zero = np.ascontiguousarray(a_zero, dtype=np.float16).reshape(m, -1)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float16)
    nt = min(_threads(), max(1, n // 16))
    bounds = np.linspace(0, n, nt + 1).astype(int)
    parts = [None] * nt

    def run(i):
        lo, hi = bounds[i], bounds[i + 1]
        d = np.empty((m, hi - lo), dtype=np.uint16)
        bb = np.ascontiguousarray(b[lo:hi])
        bs = np.ascontiguousarray(b_scale[lo:hi])
        bi = None if bias is None else np.ascontiguousarray(bias[lo:hi])
        lib().flh_oracle_gemm_i4_dequant(
            _p(a, _u8p), _p(bb, _u8p), _p(a_scale.view(np.uint16), _u16p),
            None if a_zero is None else _p(a_zero.view(np.uint16), _u16p),
            _p(bs.view(np.uint16), _u16p), None if bi is None else _p(bi.view(np.uint16), _u16p),
            _p(d, _u16p), ctypes.c_long(m), ctypes.c_long(hi - lo), ctypes.c_long(k),
            ctypes.c_long(ag), ctypes.c_long(bg), ctypes.c_int(int(bf16_out)))
        parts[i] = d

    with ThreadPoolExecutor(nt) as ex:
        list(ex.map(run, range(nt)))
    d = np.concatenate(parts, axis=1)
    return d if bf16_out else d.view(np.float16)


def bf16_bits_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(f: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
