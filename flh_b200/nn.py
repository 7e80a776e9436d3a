"""Host-side mirror of flh.nn for the W4A4 hot path: ActQuantizer, WeightQuantizer, LinearFLH
(flh/nn/quantization.py:143-484, flh/nn/linear.py:8-285) with the same constructor arguments,
buffer names and return conventions, running on the sm_100a kernels behind flh_b200._CUDA.

Two activation modes share the classes:
  group_sym   ActQuantizer(sym=True, group_size in {32,64,128}) — the flh._CUDA contract:
              per (token, group) symmetric int4, optional group Hadamard, returns
              (scale [.., K/gs], None, packed [.., K/2]);
  token_asym  ActQuantizer(sym=False, group_size <= 0) — per-token asymmetric int4 after an
              optional full-width Hadamard, returns (scale [.., 1], zero [.., 1], packed [.., K/2]).
LinearFLH.forward picks the GEMM epilogue from what it is given (a_zero or not; the shapes of
the scales).  Weight preparation (rotation, RTN, packing) is offline torch code, as it is in FLH.
"""
from __future__ import annotations

import math

import torch

from . import _CUDA
from .functional import pack_i4, unpack_i4
from .hadamard import hadamard_group, matmul_hadU


def fast_hadamard_transform(x, group_size=None, normalize=True, use_cuda=True):
    """flh/nn/quantization.py:115-140.  CUDA f16 input: group-128 kernel on a copy, / sqrt(128);
    otherwise the float64 host transform (grouped, or full-width when group_size is None/<=0)."""
    if use_cuda and x.dtype == torch.float16 and x.is_cuda:
        y = x.clone().view(-1, 128)
        return (_CUDA.hadamard_transform_half(y) / math.sqrt(128)).view(x.shape)
    return hadamard_group(x, group_size if group_size else -1)


class ActQuantizer(torch.nn.Module):
    def __init__(self, bits=8, group_size=-1, sym=True, input_clip_ratio=1.0, use_hadamard=True,
                 packed_output=False):
        super().__init__()
        self.bits, self.group_size, self.sym = bits, group_size, sym
        self.input_clip_ratio, self.use_hadamard, self.packed_output = input_clip_ratio, use_hadamard, packed_output
        if self.packed_output and self.bits != 4:
            raise ValueError("Packed output is only supported for 4-bit quantization")

    def forward(self, x):
        """Returns (scale, zero_point or None, packed uint8 codes), as flh/nn/quantization.py:156-162."""
        lead, K = x.shape[:-1], x.shape[-1]
        if self.sym:
            gs = self.group_size if self.group_size and self.group_size > 0 else 128
            xg = x.reshape(-1, gs)
            if self.use_hadamard:
                q, scales = _CUDA.hadamard_and_quantize_i4_gs(xg, gs)
                scales = scales / math.sqrt(gs)          # the kernel's transform is un-normalised
            else:
                q, scales = _CUDA.quant_and_pack_i4_gs(xg, gs)
            return scales.view(lead + (K // gs,)), None, q.view(lead + (K // 2,))
        q, s, z = _CUDA.quant_token_asym_i4(x.reshape(-1, K), hadamard=self.use_hadamard, clip=self.input_clip_ratio)
        return s.view(lead + (1,)), z.view(lead + (1,)), q.view(lead + (K // 2,))

    def forward_origin(self, x):
        """PyTorch twin of forward (flh/nn/quantization.py:163-241): float64 transform, then the
        same quantiser formulas in x's dtype.  Never used by forward()."""
        xt = x
        if self.use_hadamard:
            xt = hadamard_group(x, self.group_size) if self.sym else matmul_hadU(x.float()).to(x.dtype)
        if self.bits >= 16:
            return None, None, xt
        if self.input_clip_ratio < 1.0 and self.sym:
            c = xt.abs().amax(dim=-1, keepdim=True) * self.input_clip_ratio
            xt = torch.clamp(xt, -c, c)
        if self.sym:
            gs = self.group_size if self.group_size and self.group_size > 0 else xt.shape[-1]
            xg = xt.reshape(xt.shape[:-1] + (xt.shape[-1] // gs, gs))
            qmax = 2 ** (self.bits - 1) - 1
            scale = torch.clamp(xg.abs().amax(dim=-1, keepdim=True) / qmax, min=1e-8)
            q = (xg / scale).round().clamp(-qmax - 1, qmax).reshape(xt.shape)
            scale, zero = scale.squeeze(-1), torch.zeros_like(scale.squeeze(-1))
        else:
            xf = xt.float()
            z0 = torch.zeros(xf.shape[:-1], device=xf.device)
            xmin = torch.minimum(xf.amin(dim=-1), z0) * self.input_clip_ratio
            xmax = torch.maximum(xf.amax(dim=-1), z0) * self.input_clip_ratio
            both = (xmin == 0) & (xmax == 0)
            xmin, xmax = torch.where(both, -torch.ones_like(xmin), xmin), torch.where(both, torch.ones_like(xmax), xmax)
            maxq = 2 ** self.bits - 1
            scale = ((xmax - xmin) / maxq).unsqueeze(-1)
            zero = torch.round(-xmin.unsqueeze(-1) / scale)
            q = torch.clamp(torch.round(xf / scale) + zero, 0, maxq)
        if self.packed_output:
            qi = q.to(torch.int32)
            q = pack_i4(qi) if self.sym else ((qi[..., 0::2] & 15) | ((qi[..., 1::2] & 15) << 4)).to(torch.uint8)
        return scale, zero, q


Quantizer = ActQuantizer


class WeightQuantizer(torch.nn.Module):
    """Offline RTN weight quantiser (flh/nn/quantization.py:294-484): symmetric or asymmetric,
    per group, per output channel or per tensor.  The per-channel branch, unreachable in FLH
    because of an undefined name (:371-372), works here and follows
    fake_quant/quant_utils.py:244-256 for the symmetric case (1e-5 floor on the range)."""

    def __init__(self, bits=4, group_size=-1, sym=True, channel_wise=True, use_hadamard=True, clip_ratio=1.0):
        super().__init__()
        self.bits, self.group_size, self.sym = bits, group_size, sym
        self.channel_wise, self.use_hadamard, self.clip_ratio = channel_wise, use_hadamard, clip_ratio
        self.register_buffer("scale", None)
        self.register_buffer("zero_point", None)
        self.calibrated = False

    def _prep(self, w):
        if self.use_hadamard:
            w = fast_hadamard_transform(w, group_size=self.group_size, use_cuda=False)
        if self.clip_ratio < 1.0:
            g = self._grouped(w)
            c = g.abs().amax(dim=-1, keepdim=True) * self.clip_ratio
            w = torch.clamp(g, -c, c).reshape(w.shape)
        return w

    def _grouped(self, w):
        if self.group_size > 0:
            if w.shape[1] % self.group_size != 0:
                raise ValueError(f"in_features ({w.shape[1]}) must be divisible by group_size ({self.group_size})")
            return w.reshape(w.shape[0], w.shape[1] // self.group_size, self.group_size)
        if self.channel_wise:
            return w.reshape(w.shape[0], 1, w.shape[1])
        return w.reshape(1, 1, -1)

    def calibrate(self, weight):
        if self.bits >= 16:
            self.calibrated = True
            return
        g = self._grouped(self._prep(weight))
        with torch.no_grad():
            # divisors are tensors: torch's CUDA kernels replace a division by a Python scalar with a multiplication by its
            # reciprocal, and a weight converted on the GPU must come out bit-equal to one converted on the host
            if self.sym:
                qmax = torch.tensor(float(2 ** (self.bits - 1) - 1), dtype=g.dtype, device=g.device)
                if self.group_size <= 0 and self.channel_wise:
                    xmax = torch.maximum(g.amin(dim=-1).clamp(max=0).abs(), g.amax(dim=-1).clamp(min=0)).clamp(min=1e-5)
                    scale = xmax / qmax
                else:
                    scale = torch.clamp(g.abs().amax(dim=-1) / qmax, min=1e-8)
                zero = torch.zeros_like(scale)
            else:
                qmax = torch.tensor(float(2 ** self.bits - 1), dtype=g.dtype, device=g.device)
                mx, mn = g.amax(dim=-1), g.amin(dim=-1)
                scale = torch.clamp((mx - mn) / qmax, min=1e-8)
                zero = -mn / scale
        self.scale, self.zero_point = scale, zero       # [N, G], [N, 1] or [1, 1]
        self.calibrated = True

    def quantize(self, weight):
        w = self._prep(weight)
        if self.bits >= 16:
            return None, None, w
        if not self.calibrated:
            raise RuntimeError("WeightQuantizer must be calibrated before quantization")
        g = self._grouped(w)
        if self.sym:
            q = (g / self.scale.unsqueeze(-1)).round().clamp(-(2 ** (self.bits - 1)), 2 ** (self.bits - 1) - 1)
        else:
            q = (g / self.scale.unsqueeze(-1) + self.zero_point.unsqueeze(-1)).round().clamp(0, 2 ** self.bits - 1)
        return self.scale, self.zero_point, q.reshape(w.shape).to(w.dtype)

    def forward(self, weight):
        if not self.calibrated:
            self.calibrate(weight)
        return self.quantize(weight)


class LinearFLH(torch.nn.Module):
    """Packed W4 linear fed with already-quantised activations (flh/nn/linear.py:8-133).
    Buffers keep FLH's names and layouts: w_packed flat uint8 [(N*K+1)//2], w_scale [N, K/gs] (or
    [N, 1]), w_zero uint8 like w_scale — the checkpoint format of FLH_LlamaForCausalLM.save_quantized."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16, device="cpu",
                 dual_hadamard=False, in_group_size=None, out_group_size=None, no_hadamard=False, group_size=128):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.dual_hadamard, self.in_group_size, self.out_group_size = dual_hadamard, in_group_size, out_group_size
        self.weight_group_size, self.no_hadamard = group_size, no_hadamard
        ng = (in_features + group_size - 1) // group_size if group_size > 0 else 1
        self.register_buffer("w_packed", torch.zeros((out_features * in_features + 1) // 2, dtype=torch.uint8, device=device))
        self.register_buffer("w_scale", torch.zeros(out_features, ng, dtype=dtype, device=device))
        self.register_buffer("w_zero", torch.zeros(out_features, ng, dtype=torch.uint8, device=device))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.bias = None
        self._rowsum = None
        self._w_i8 = None          # optional int8 copy of the weights for large-batch GEMMs (prepack_int8)
        # 0: no full-width rotation on the input side; b >= 1: the weight was rotated with matmul_hadU over b equal
        # blocks of K (b = 1 is the plain full-width transform; b = tp is what a row-parallel shard needs)
        self.full_hadamard_blocks = 0

    # -- offline side ---------------------------------------------------------------------------
    def _pack_weights(self, w_int, scale, zero):
        self.w_scale.copy_(scale.reshape(self.w_scale.shape))
        self.w_zero.copy_(zero.reshape(self.w_zero.shape).clamp(0, 15).to(torch.uint8))
        self.w_packed.copy_(pack_i4(w_int.to(torch.int32).clamp(-8, 7)).reshape(-1))
        self._rowsum = None
        self._w_i8 = None

    def _unpack_weights(self):
        w = unpack_i4(self.w_packed.view(self.out_features, self.in_features // 2)).to(self.w_scale.dtype)
        g = self.w_scale.shape[1]
        w = w.view(self.out_features, g, -1)
        return ((w - self.w_zero.unsqueeze(-1).to(w.dtype)) * self.w_scale.unsqueeze(-1)).view(self.out_features, self.in_features)

    def get_weight(self, dtype=None):
        w = self._unpack_weights()
        return w if dtype is None else w.to(dtype)

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_bits=4, weight_group_size=128, weight_sym=True,
                   dual_hadamard=False, in_group_size=None, out_group_size=None, clip_ratio=1.0,
                   no_hadamard=False, full_hadamard=False, hadamard_blocks=1):
        """flh/nn/linear.py:190-285: rotate the weight on its input side (block-diagonal groups of
        in_group_size, or the full-width matmul_hadU transform with full_hadamard=True), optionally
        on its output side too, then RTN-quantise and pack.  hadamard_blocks = b applies the full-width
        transform to each of b equal blocks of K instead of to K as a whole: a row-parallel layer split over
        b ranks rotates each rank's K / b activations on its own, so its weight must be rotated the same way."""
        assert weight_bits == 4 and weight_sym, "the packed path stores symmetric int4 weights"
        W = module.weight.data.clone()
        lin = LinearFLH(module.in_features, module.out_features, bias=module.bias is not None, dtype=W.dtype,
                        device=W.device, dual_hadamard=dual_hadamard, in_group_size=in_group_size,
                        out_group_size=out_group_size, group_size=weight_group_size, no_hadamard=no_hadamard)
        if module.bias is not None:
            lin.bias.copy_(module.bias.data)
        if not no_hadamard:
            if full_hadamard:
                N_, K_ = W.shape
                assert K_ % hadamard_blocks == 0, "K must split evenly into hadamard_blocks"
                W = matmul_hadU(W.double().reshape(N_, hadamard_blocks, K_ // hadamard_blocks)).reshape(N_, K_).to(W.dtype)
                lin.full_hadamard_blocks = hadamard_blocks
            else:
                W = hadamard_group(W, in_group_size or -1)
            if dual_hadamard:
                W = hadamard_group(W.T.contiguous(), out_group_size or -1).T.contiguous()
                if module.bias is not None:
                    lin.bias.copy_(hadamard_group(lin.bias.unsqueeze(0), out_group_size or -1).squeeze(0))
        wq = WeightQuantizer(bits=weight_bits, group_size=weight_group_size, sym=weight_sym,
                             channel_wise=(weight_group_size == -1), use_hadamard=False, clip_ratio=clip_ratio)
        wq.calibrate(W)
        scale, zp, w_int = wq.quantize(W)
        lin._pack_weights(w_int, scale, zp)
        return lin

    # -- hot path ---------------------------------------------------------------------------------
    def w_rowsum(self, group):
        if self._rowsum is None or self._rowsum.shape[1] != self.in_features // group or self._rowsum.device != self.w_packed.device:
            self._rowsum = _CUDA.weight_rowsum(self.w_packed.view(self.out_features, self.in_features // 2), group)
        return self._rowsum

    PREPACK_MIN_ROWS = 256      # batches from which the int8 copy is used

    def prepack_int8(self):
        """Keep an int8 copy of the weights (1 byte per weight on top of the packed half byte) for large-batch
        GEMMs with per-channel weight scales: the tensor cores then read int8 tiles straight from TMA.  Decode-size
        batches keep streaming the packed weights.  No counterpart in the reference (int4 weights only)."""
        if self.w_scale.shape[1] == 1 and self._w_i8 is None:
            self._w_i8 = _CUDA.expand_i4(self.w_packed.view(self.out_features, self.in_features // 2))
        return self

    def forward(self, x, a_scale=None, a_zero=None, x_is_packed=True, is_symmetric=None, out_dtype=None, out=None):
        """x: packed activations [.., K/2]; a_scale [.., K/gs] (group mode) or [.., 1] (per token);
        a_zero None or like a_scale.  Returns [.., N] in the dtype of w_scale (flh/nn/linear.py:125-133); out = a
        contiguous [M, N] tensor to write into instead of allocating."""
        lead = x.shape[:-1]
        M = x.numel() // x.shape[-1]
        a_scale = a_scale.reshape(M, -1)
        ga, gb = self.in_features // a_scale.shape[1], self.in_features // self.w_scale.shape[1]
        rs = None
        if a_zero is not None:
            a_zero = a_zero.reshape(M, -1)
            rs = self.w_rowsum(min(ga, gb))
        if self._w_i8 is not None and a_scale.shape[1] == 1 and M >= self.PREPACK_MIN_ROWS:
            y = _CUDA.gemm_i8w_dequant(x.reshape(M, -1), self._w_i8, a_scale, self.w_scale, A_zero=a_zero, B_rowsum=rs,
                                       bias=self.bias, out_dtype=out_dtype or self.w_scale.dtype, out=out)
        else:
            y = _CUDA.gemm_i4_dequant(x.reshape(M, -1), self.w_packed.view(self.out_features, self.in_features // 2),
                                      a_scale, self.w_scale, A_zero=a_zero, B_rowsum=rs, bias=self.bias,
                                      out_dtype=out_dtype or self.w_scale.dtype, out=out)
        return y.view(lead + (self.out_features,))

    def forward_torch(self, x, a_scale=None, a_zero=None, x_is_packed=True, is_symmetric=None):
        """PyTorch twin (flh/nn/linear.py:134-152): unpack, (q - zero) * scale, F.linear."""
        if is_symmetric is None:      # as the reference infers it: symmetric unless a non-zero zero-point is given
            is_symmetric = a_zero is None or not bool(torch.any(a_zero != 0))
        signed = is_symmetric
        q = unpack_i4(x, signed=signed).float()
        g = a_scale.shape[-1]
        qg = q.view(*q.shape[:-1], g, -1)
        z = 0 if a_zero is None else a_zero.float().unsqueeze(-1)
        xf = ((qg - z) * a_scale.float().unsqueeze(-1)).view(q.shape)
        return torch.nn.functional.linear(xf, self._unpack_weights().float(), None if self.bias is None else self.bias.float())
