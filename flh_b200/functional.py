"""Nibble packing and the elementary quantisation formulas, with the names and meaning of
flh/functional/quantization.py (pack_i4 :42-49, unpack_i4 :52-74, sym/asym helpers :4-38).
Offline / host-side helpers on torch tensors (any device); the hot path never calls them."""
from __future__ import annotations

import torch


def two_compl(x, bits: int):
    return torch.where(x < 0, 2 ** bits + x, x)


def get_minq_maxq(bits: int, sym: bool):
    if sym:
        maxq = torch.tensor(2 ** (bits - 1) - 1)
        return -maxq - 1, maxq
    return torch.tensor(0), torch.tensor(2 ** bits - 1)


def asym_quant(x, scale, zero, maxq):
    q = torch.clamp(torch.round(x / scale) + zero, 0, maxq)
    return q, scale, zero


def asym_dequant(q, scale, zero):
    return scale * (q - zero)


def asym_quant_dequant(x, scale, zero, maxq):
    return asym_dequant(*asym_quant(x, scale, zero, maxq))


def sym_quant(x, scale, maxq):
    return torch.clamp(torch.round(x / scale), -(maxq + 1), maxq), scale


def sym_dequant(q, scale):
    return scale * q


def sym_quant_dequant(x, scale, maxq):
    return sym_dequant(*sym_quant(x, scale, maxq))


def pack_i4(q: torch.Tensor) -> torch.Tensor:
    """Signed int tensor [.., K] with values in [-8, 7] -> uint8 [.., K/2]; byte j = element 2j in
    the low nibble, element 2j+1 in the high nibble, two's complement."""
    assert torch.is_signed(q), "The tensor to be packed should be signed int"
    assert bool(torch.all((q >= -8) & (q <= 7)))
    u = two_compl(q.to(torch.int16), 4).to(torch.uint8)
    return u[..., 0::2] | (u[..., 1::2] << 4)


def unpack_i4(x: torch.Tensor, signed: bool = True) -> torch.Tensor:
    """uint8 [.., K/2] -> int32 [.., K] (signed nibbles by default, 0..15 with signed=False)."""
    assert x.dtype == torch.uint8, "The tensor to be unpacked should be stored in uint8"
    lo = (x & 0x0F).to(torch.int32)
    hi = (x >> 4).to(torch.int32)
    if signed:
        lo = torch.where(lo >= 8, lo - 16, lo)
        hi = torch.where(hi >= 8, hi - 16, hi)
    return torch.stack((lo, hi), dim=-1).reshape(*x.shape[:-1], x.shape[-1] * 2)


def expand_i4_reference(packed):
    """Host restatement of flh_b200_expand_i4: packed int4 [rows, K/2] -> bytes [rows, K] holding 16 * code (the nibble in the
    byte's high half), per 32 elements the 16 even ones then the 16 odd ones."""
    rows, kp = packed.shape
    b = packed.view(rows, kp // 16, 16)
    even, odd = (b << 4) & 0xF0, b & 0xF0
    return torch.cat((even, odd), dim=-1).reshape(rows, 2 * kp)


def compress_i8(expanded):
    """Inverse of the int8 expansion (flh_b200_expand_i4 / expand_i4_reference): bytes [rows, K] -> packed int4 [rows, K/2] in
    the checkpoint layout (byte j = element 2j in the low nibble, 2j + 1 in the high one).  Lossless."""
    rows, k = expanded.shape
    b = expanded.view(rows, k // 32, 2, 16)
    return ((b[:, :, 0, :] >> 4) | (b[:, :, 1, :] & 0xF0)).reshape(rows, k // 2)
