"""PyTorch-on-CPU port of the reference's fake_quant path — the timed CPU baseline.

TEST INFRASTRUCTURE ONLY (tests/, the smoke entry and bench.py's CPU legs).  The reference's own
CPU implementation of the hot path is Python/PyTorch (fake_quant/), which cannot travel to the GPU
box, so it is restated here operation for operation with torch CPU tensors and pinned against an
output of the reference itself (tests/golden: cfg1_Y).

Restates
  get_hadamard_matrix          fake_quant/hadamard_utils.py:5-25  (Sylvester, / sqrt(n))
  matmul_had_cuda              fake_quant/hadamard_utils.py:44-47 (x @ H, dense)
  ActQuantizer.find_params     fake_quant/quant_utils.py:94-128   (per-token asymmetric)
  asym_quant / asym_dequant    fake_quant/quant_utils.py:17-27
  WeightQuantizer.find_params  fake_quant/quant_utils.py:244-256  (per-channel symmetric RTN)
  ActQuantWrapper.forward      fake_quant/quant_utils.py:160-181
"""
from __future__ import annotations

import torch


def hadamard_matrix(n: int, dtype=torch.float32) -> torch.Tensor:
    assert n > 0 and n & (n - 1) == 0, "Hadamard size must be a positive power of 2"
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / (n ** 0.5)).to(dtype)


def act_find_params(x: torch.Tensor, bits: int = 4, clip_ratio: float = 1.0):
    """Per-token asymmetric scale / zero of the rows of x (2-D)."""
    maxq = 2 ** bits - 1
    zero_t = torch.zeros(x.shape[0], dtype=x.dtype)
    xmin = torch.minimum(x.min(1)[0], zero_t) * clip_ratio
    xmax = torch.maximum(x.max(1)[0], zero_t) * clip_ratio
    both = (xmin == 0) & (xmax == 0)
    xmin[both] = -1
    xmax[both] = +1
    scale = (xmax - xmin) / maxq
    zero = torch.round(-xmin / scale)
    return scale.unsqueeze(1), zero.unsqueeze(1), maxq


def asym_quant(x, scale, zero, maxq):
    return torch.clamp(torch.round(x / scale) + zero, 0, maxq)


def asym_dequant(q, scale, zero):
    return scale * (q - zero)


def weight_rtn_channel_sym(w: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """Quantise-dequantise W per output channel, symmetric RTN."""
    maxq = 2 ** (bits - 1) - 1
    zero_t = torch.zeros(w.shape[0], dtype=w.dtype)
    xmin = torch.minimum(w.min(1)[0], zero_t)
    xmax = torch.maximum(w.max(1)[0], zero_t)
    xmax = torch.maximum(torch.abs(xmin), xmax).clamp(min=1e-5)
    scale = (xmax / maxq).unsqueeze(1)
    return scale * torch.clamp(torch.round(w / scale), -(maxq + 1), maxq)


def act_quant_wrapper_forward(x: torch.Tensor, w_deq: torch.Tensor, H: torch.Tensor | None) -> torch.Tensor:
    """ActQuantWrapper.forward with online_had, fp32_had and a 4-bit asymmetric input quantiser:
    x -> x.float() @ H -> quantise-dequantise per token -> F.linear with the (fake-quantised) weight."""
    dt = x.dtype
    if H is not None:
        x = (x.float() @ H).to(dt)
    scale, zero, maxq = act_find_params(x)
    x = asym_dequant(asym_quant(x, scale, zero, maxq), scale, zero).to(dt)
    return torch.nn.functional.linear(x, w_deq).to(dt)


def had_quant_pack(x: torch.Tensor, H: torch.Tensor | None):
    """The quantiser half of the path with packed output, as the CUDA kernels deliver it:
    (packed codes uint8 [M, K/2], scale [M], zero [M]); binary32 throughout, as the reference."""
    y = x.float() @ H if H is not None else x.float()
    scale, zero, maxq = act_find_params(y)
    q = asym_quant(y, scale, zero, maxq).to(torch.uint8)
    return (q[:, 0::2] | (q[:, 1::2] << 4)), scale[:, 0], zero[:, 0]
