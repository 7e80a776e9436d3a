"""GPTQ calibration of a linear layer's weights on the GPU: the host-side mirror of flh/nn/gptq.py.

`FLHGPTQ` keeps the reference's interface (flh/nn/gptq.py:112-241): `add_batch` accumulates the Hessian of the
Hadamard-rotated layer inputs, `fasterquant` rotates the weights, fixes the quantiser's scales per static group
(or per channel), factors the damped Hessian and sweeps the columns in blocks, quantising one column at a time and
pushing its error onto the columns not yet visited.  What runs where:

  * the sweep inside a block (the reference's Python loop over columns, ~10 small launches per column) is ONE launch
    of the library's `flh_b200_gptq_block` kernel per block: a warp per weight row, the block of the factor in
    shared memory, the reference's binary32 arithmetic operation for operation;
  * the Hessian accumulation, the Cholesky factorisations and the update of the columns right of a block are dense
    linear algebra and go to torch's CUDA libraries (plain library GEMM / LAPACK calls, as in the reference).

Everything needs the CUDA library; there is no CPU path here.
"""
import copy
import math

import torch

from . import _CUDA as C
from . import _lib
from .nn import fast_hadamard_transform


class GPTQQuantizer:
    """flh/nn/gptq.py:27-109: scales (and zero-points) of a weight slice, per group or per channel."""

    def __init__(self, bits, groupsize=-1, sym=True, clip_ratio=1.0):
        self.bits = bits
        self.groupsize = groupsize
        self.sym = sym
        self.clip_ratio = clip_ratio
        self.maxq = 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1
        self.scale = None
        self.zero = None

    def ready(self):
        return self.scale is not None and bool(torch.all(self.scale != 0))

    def _clip_weight(self, W):
        if self.clip_ratio >= 1.0:
            return W
        if self.groupsize > 0 and W.shape[1] % self.groupsize == 0:
            Wg = W.view(W.shape[0], -1, self.groupsize)
            clip_val = Wg.abs().amax(dim=2, keepdim=True) * self.clip_ratio
            return torch.clamp(Wg, -clip_val, clip_val).view(W.shape)
        clip_val = W.abs().amax(dim=1, keepdim=True) * self.clip_ratio
        return torch.clamp(W, -clip_val, clip_val)

    def find_params(self, W, weight=True):
        W = self._clip_weight(W.float())
        if self.bits >= 16:
            return
        # a tensor divisor: CUDA torch turns division by a Python scalar into a multiplication by its reciprocal, which is
        # not the reference's (CPU) quotient in the last bit
        maxq = torch.tensor(float(self.maxq), device=W.device)
        if self.groupsize > 0 and W.shape[1] % self.groupsize == 0:
            Wg = W.view(W.shape[0], -1, self.groupsize)
            if self.sym:
                xmax = Wg.abs().amax(dim=2, keepdim=True).clamp(min=1e-5)
                self.scale = (xmax / maxq).view(W.shape[0], -1)
                self.zero = torch.zeros_like(self.scale)
            else:
                xmax, xmin = Wg.amax(dim=2, keepdim=True), Wg.amin(dim=2, keepdim=True)
                both = (xmin == 0) & (xmax == 0)
                xmin = torch.where(both, torch.full_like(xmin, -1.0), xmin)
                xmax = torch.where(both, torch.full_like(xmax, 1.0), xmax)
                self.scale = ((xmax - xmin) / maxq).clamp(min=1e-5).view(W.shape[0], -1)
                self.zero = torch.round(-xmin.view(W.shape[0], -1) / self.scale)
        else:
            flat = W.flatten(1)
            xmin, xmax = flat.min(1)[0], flat.max(1)[0]
            if self.sym:
                xmax = torch.maximum(xmax.abs(), xmin.abs()).clamp(min=1e-5)
                self.scale = (xmax / maxq).unsqueeze(1)
                self.zero = torch.zeros_like(self.scale)
            else:
                both = (xmin == 0) & (xmax == 0)
                xmin = torch.where(both, torch.full_like(xmin, -1.0), xmin)
                xmax = torch.where(both, torch.full_like(xmax, 1.0), xmax)
                self.scale = ((xmax - xmin) / maxq).clamp(min=1e-5).unsqueeze(1)
                self.zero = torch.round(-xmin.unsqueeze(1) / self.scale)


def gptq_block(W, i1, count, Hinv, scale, zero, group_of_col, maxq, sym, clip_ratio, Q, Err):
    """Columns [i1, i1 + count) of W (f32, row-major) through the library's block sweep; writes Q[:, i1:i1+count]
    and Err[:, :count] (include/flh_b200.h: flh_b200_gptq_block)."""
    rows, cols = W.shape
    for t in (W, Hinv, scale, Q, Err):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise RuntimeError("gptq_block takes contiguous float32 CUDA tensors")
    if not (group_of_col.is_cuda and group_of_col.dtype == torch.int32 and group_of_col.numel() >= count):
        raise RuntimeError("group_of_col must be an int32 CUDA tensor with one entry per block column")
    with C._guard(W.device):
        _lib.check(_lib.load().flh_b200_gptq_block(
            W.data_ptr() + 4 * i1, cols, Hinv.data_ptr() + 4 * (i1 * cols + i1), cols, scale.data_ptr(),
            zero.data_ptr() if zero is not None else None, scale.shape[1], group_of_col.data_ptr(), rows, count, int(maxq),
            1 if sym else 0, float(clip_ratio), Q.data_ptr() + 4 * i1, cols, Err.data_ptr(), C._stream(W)), "gptq_block")


class FLHGPTQ:
    """flh/nn/gptq.py:112-241 on the GPU.  `layer` is a torch.nn.Linear on a CUDA device."""

    def __init__(self, layer, dual_hadamard=False):
        self.layer = layer
        self.dual_hadamard = dual_hadamard
        self.dev = layer.weight.device
        if self.dev.type != "cuda":
            raise RuntimeError("flh_b200.gptq.FLHGPTQ runs on a CUDA device")
        self.rows, self.columns = layer.weight.shape
        self.H = torch.zeros((self.columns, self.columns), device=self.dev, dtype=torch.float32)
        self.nsamples = 0
        self.out_list = []

    def add_batch(self, inp, out, group_size=-1):
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        tmp = inp.shape[0] * inp.shape[1]
        inp = inp.reshape(-1, inp.shape[-1])
        inp = fast_hadamard_transform(inp.float(), group_size=group_size if group_size > 0 else None, use_cuda=False)
        inp = inp.t()
        self.H *= self.nsamples / (self.nsamples + tmp)
        self.nsamples += tmp
        inp = math.sqrt(2 / self.nsamples) * inp
        self.H += inp.matmul(inp.t())
        if out is not None:
            if out.dim() == 2:
                out = out.unsqueeze(0)
            self.out_list.append(out.reshape(-1, out.shape[-1]))

    def fasterquant(self, group_size=128, blocksize=128, percdamp=0.01, actorder=False, sym=True, bits=4,
                    dual_hadamard=None, clip_ratio=1.0):
        if dual_hadamard is None:
            dual_hadamard = self.dual_hadamard
        if blocksize > 128:
            raise RuntimeError("the block sweep kernel takes blocks of at most 128 columns")
        W = self.layer.weight.data.clone().float()
        group_size = group_size if group_size > 0 and self.columns % group_size == 0 else -1
        gs = group_size if group_size > 0 else None
        W = fast_hadamard_transform(W, group_size=gs, use_cuda=False)
        if dual_hadamard:
            W = fast_hadamard_transform(W.T, group_size=gs, use_cuda=False).T.contiguous()

        self.quantizer = GPTQQuantizer(bits=bits, groupsize=group_size, sym=sym, clip_ratio=clip_ratio)
        H = self.H
        del self.H
        dead = torch.diag(H) == 0
        H[dead, dead] = 1
        W[:, dead] = 0
        if clip_ratio < 1.0:
            W = self.quantizer._clip_weight(W)

        # the quantiser's parameters, fixed before the sweep: one column of scales per static group, or one per channel
        if group_size > 0:
            scales, zeros = [], []
            for i in range(0, self.columns, group_size):
                q = copy.deepcopy(self.quantizer)
                q.find_params(W[:, i:i + group_size])
                scales.append(q.scale)
                zeros.append(q.zero)
            scale = torch.cat(scales, dim=1).contiguous()
            zero = torch.cat(zeros, dim=1).contiguous()
        else:
            self.quantizer.find_params(W)
            scale, zero = self.quantizer.scale.contiguous(), self.quantizer.zero.contiguous()
        self.scale, self.zero = scale, zero

        cols = torch.arange(self.columns, device=self.dev)
        if actorder:
            perm = torch.argsort(torch.diag(H), descending=True)
            W = W[:, perm]
            H = H[perm][:, perm]
            invperm = torch.argsort(perm)
            cols = perm
        group_of_col = (cols // group_size if group_size > 0 else torch.zeros_like(cols)).to(torch.int32).contiguous()

        W = W.contiguous()
        Q = torch.zeros_like(W)
        damp = percdamp * torch.mean(torch.diag(H))
        diag = torch.arange(self.columns, device=self.dev)
        H[diag, diag] += damp
        H = torch.linalg.cholesky(H)
        H = torch.cholesky_inverse(H)
        Hinv = torch.linalg.cholesky(H, upper=True).contiguous()

        Err = torch.empty((self.rows, blocksize), device=self.dev, dtype=torch.float32)
        for i1 in range(0, self.columns, blocksize):
            i2 = min(i1 + blocksize, self.columns)
            count = i2 - i1
            gptq_block(W, i1, count, Hinv, scale, zero if not sym else None, group_of_col[i1:i2].contiguous(),
                       self.quantizer.maxq, sym, clip_ratio, Q, Err)
            if i2 < self.columns:               # only full blocks have columns to their right
                W[:, i2:] -= Err.matmul(Hinv[i1:i2, i2:])
        if actorder:
            Q = Q[:, invperm]
        self.layer.weight.data = Q.to(self.layer.weight.dtype).reshape(self.layer.weight.shape)

    def free(self):
        self.H = None
        torch.cuda.empty_cache()
