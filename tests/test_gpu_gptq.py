"""GPTQ calibration on the GPU (flh_b200.gptq, the library's flh_b200_gptq_block kernel) against the CPU restatement
and the golden vectors made by the reference's own FLHGPTQ."""
import os

import numpy as np
import pytest
import torch

from oracle import gptq_oracle as G
from test_gptq import CONFIGS, GOLD, golden_batches, golden_case

pytestmark = pytest.mark.gpu


def _spd_factor(n, seed):
    """Upper Cholesky factor of the inverse of a damped random Hessian, as fasterquant builds it (float32, torch CPU)."""
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(4 * n, n, generator=g) @ (torch.randn(n, n, generator=g) * 0.2 + torch.eye(n))
    H = (X.t() @ X) / X.shape[0]
    H += 0.01 * torch.mean(torch.diag(H)) * torch.eye(n)
    return torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True).contiguous()


@pytest.mark.parametrize("rows,cols,i1,count", [(70, 256, 128, 128), (16, 128, 0, 128), (33, 384, 256, 96), (5, 160, 128, 32), (1, 64, 0, 64)])
@pytest.mark.parametrize("sym,clip", [(True, 1.0), (True, 0.9), (False, 1.0), (False, 0.85)])
def test_block_sweep_is_bit_exact(cuda, rows, cols, i1, count, sym, clip):
    """One launch of the block kernel == the column-by-column loop of the restatement, bit for bit (Q and Err)."""
    from flh_b200 import gptq
    rs = np.random.RandomState(rows * 7 + count + int(sym) + int(clip * 100))
    W = (rs.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    W[:, i1 + 3] *= 8.0
    Hinv = _spd_factor(cols, rows + count)
    ngroups = 3
    bits = 4
    maxq = 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1
    scale = (np.abs(W).max(axis=1, keepdims=True) / maxq * (0.6 + 0.4 * rs.rand(rows, ngroups)) * (1 if sym else 2)).astype(np.float32)
    zero = np.rint(rs.rand(rows, ngroups) * 15).astype(np.float32)
    goc = rs.randint(0, ngroups, size=count).astype(np.int32)
    Q1, E1 = G.block_sweep(W[:, i1:i1 + count], Hinv[i1:i1 + count, i1:i1 + count].numpy(), scale, zero, goc, maxq, sym, clip)

    Wd, Hd = torch.from_numpy(W).cuda(), Hinv.cuda()
    Q = torch.zeros_like(Wd)
    Err = torch.empty((rows, count), dtype=torch.float32, device="cuda")
    gptq.gptq_block(Wd, i1, count, Hd, torch.from_numpy(scale).cuda(), None if sym else torch.from_numpy(zero).cuda(),
                    torch.from_numpy(goc).cuda(), maxq, sym, clip, Q, Err)
    got_q, got_e = Q[:, i1:i1 + count].cpu().numpy(), Err.cpu().numpy()
    # + 0.0 folds -0 into +0: clamp(-0, 0, maxq) of the asymmetric quantiser keeps the sign in numpy and drops it in
    # CUDA's fmaxf, the one place where the two are allowed to differ (the value is the same zero)
    bits = lambda a: (a + np.float32(0.0)).view(np.uint32)
    assert np.array_equal(bits(got_q), bits(Q1)), f"{(got_q != Q1).sum()} quantised weights differ"
    assert np.array_equal(bits(got_e), bits(E1)), f"{(got_e != E1).sum()} errors differ"
    assert float(Q[:, :i1].abs().sum()) == 0.0 and float(Q[:, i1 + count:].abs().sum()) == 0.0     # nothing outside the block


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_gpu_calibration_against_the_reference_golden(cuda, name):
    """FLHGPTQ on the GPU from the same layer and inputs as the reference's CPU run.  The block sweeps are exact; the
    Hessian, the factorisations and the updates between blocks go through the GPU's dense libraries, whose sums are
    ordered differently from the CPU's, so a weight that sits on a rounding boundary may land on the neighbouring
    code and shift the ones after it in its row.  Bound: at most 2 % of the weights differ from the reference's, and
    the layer-output error tr((W - Q) H (W - Q)^T) is within 1 % of the reference's."""
    from flh_b200 import gptq
    z, kw, W, H = golden_case(name)
    gs = CONFIGS[name][1]
    layer = torch.nn.Linear(W.shape[1], W.shape[0], bias=False).cuda()
    layer.weight.data = torch.from_numpy(z["weight"]).cuda()
    gq = gptq.FLHGPTQ(layer)
    for b in golden_batches(z):
        gq.add_batch(torch.from_numpy(b).cuda().unsqueeze(0), None, group_size=gs)
    assert np.allclose(gq.H.cpu().numpy(), H, rtol=1e-4, atol=1e-6 * np.abs(H).max())
    gq.fasterquant(**kw)
    Q = layer.weight.data.float().cpu().numpy()
    ref = z[f"Q_{name}"]
    differing = float((Q != ref).mean())
    assert differing <= 0.02, differing
    l_gpu, l_ref = G.proxy_loss(W, Q, H), G.proxy_loss(W, ref, H)
    assert abs(l_gpu - l_ref) <= 0.01 * l_ref, (l_gpu, l_ref)


def test_gpu_calibration_beats_rtn_on_a_wider_layer(cuda):
    """rows 256 x columns 1024 (eight blocks): GPTQ's layer-output error is well below round-to-nearest's with the same
    scales, and every weight is one of the 16 levels of its group."""
    from flh_b200 import gptq
    g = torch.Generator().manual_seed(5)
    rows, cols = 256, 1024
    weight = (torch.randn(rows, cols, generator=g) * 0.04)
    mix = torch.randn(cols, cols, generator=g) * 0.1 + torch.eye(cols)
    X = (torch.randn(2048, cols, generator=g) @ mix)
    layer = torch.nn.Linear(cols, rows, bias=False).cuda()
    layer.weight.data = weight.cuda()
    gq = gptq.FLHGPTQ(layer)
    gq.add_batch(X.cuda().unsqueeze(0), None, group_size=128)
    H = gq.H.clone()
    gq.fasterquant(group_size=128, sym=True)
    Q = layer.weight.data.float()
    Wr = gptq.fast_hadamard_transform(weight.cuda().float(), group_size=128, use_cuda=False)
    scale = gq.scale.repeat_interleave(128, dim=1)
    rtn = torch.clamp(torch.round(Wr / scale), -8, 7) * scale
    codes = Q / scale
    assert float((codes - torch.round(codes)).abs().max()) < 1e-3 and float(codes.min()) >= -8.001 and float(codes.max()) <= 7.001
    loss = lambda q: float(torch.einsum("ij,jk,ik->", (Wr - q).double(), H.double(), (Wr - q).double()))
    assert loss(Q) < 0.7 * loss(rtn), (loss(Q), loss(rtn))
