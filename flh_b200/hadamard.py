"""Hadamard factor tables and the host-side (offline) transforms.

get_hadK follows flh/functional/hadamard.py:39-89: the same precedence of the `n % K == 0`
tests, so a width maps to the same (K x K factor) (x) (power-of-two butterfly) split.  The sign
tables are data extracted from that file by flh_b200/data/make_hadk_tables.py.
"""
from __future__ import annotations

import math
import os
from functools import lru_cache

import numpy as np
import torch

_ORDER = (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)
_DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "hadk_signs.npz")


def is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


@lru_cache(maxsize=None)
def _table(k: int) -> np.ndarray:
    z = np.load(_DATA)
    bits = np.unpackbits(z[f"had{k}"])[: k * k].reshape(k, k)
    return (1 - 2 * bits.astype(np.int8)).astype(np.int8)


def get_hadK(n: int):
    """(int8 K x K matrix of +-1 or None, K)."""
    for k in _ORDER:
        if n % k == 0:
            if not is_pow2(n // k):
                raise AssertionError(f"{n} / {k} is not a power of two")
            return _table(k), k
    if not is_pow2(n):
        raise AssertionError(f"{n} is neither a power of two nor K * 2^m for a known K")
    return None, 1


def matmul_hadU(X: torch.Tensor) -> torch.Tensor:
    """y = (hadK (x) H_p) x / sqrt(n) on the last dimension, in X's dtype; offline use (weight
    rotation).  Same butterfly order as flh/functional/hadamard.py:92-113."""
    n = X.shape[-1]
    signs, k = get_hadK(n)
    x = X.reshape(-1, k, n // k).clone()
    h = 1
    p = n // k
    while h < p:
        x = x.view(-1, k, p // (2 * h), 2, h)
        a, b = x[..., 0, :], x[..., 1, :]
        x = torch.stack((a + b, a - b), dim=-2).reshape(-1, k, p)
        h *= 2
    if k > 1:
        hk = torch.from_numpy(signs.astype(np.float64)).to(device=X.device, dtype=X.dtype)
        x = hk @ x
    # (a tensor divisor: torch's CUDA kernels turn a division by a Python scalar into a multiplication by its reciprocal,
    # which is not the same rounding as the host's division)
    return (x.reshape(X.shape) / torch.tensor(math.sqrt(n), dtype=x.dtype, device=x.device)).to(X.dtype)


def hadamard_group(X: torch.Tensor, group_size: int) -> torch.Tensor:
    """Block-diagonal normalised Hadamard over groups of the last dimension, computed in float64
    and cast back — fast_hadamard_transform's PyTorch branch (flh/nn/quantization.py:129-140)."""
    n = X.shape[-1]
    if group_size is None or group_size <= 0 or n % group_size != 0:
        return matmul_hadU(X.double()).to(X.dtype)
    y = matmul_hadU(X.double().reshape(-1, group_size)).reshape(X.shape)
    return y.to(X.dtype)
