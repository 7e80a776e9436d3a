"""Parity at the full sizes of the benchmark configurations — the launch shapes the bench times: sampled rows against
the CPU oracle (the whole matrix would take the oracle minutes), plus properties that hold for every row.

  quantisers  M = 16384 for K in {4096, 11008, 14336}: group-128 symmetric (bit-exact), per-token asymmetric in the
              reference's summation order (bit-exact) and with the default transform (stated tolerance);
  GEMM        N = 22016 (4096 -> 22016) at M in {16, 2048, 8192}, group-128 scales and per-token x per-channel scales.
"""
import numpy as np
import pytest
import torch

from helpers import assert_token_tolerance, rs
from oracle import oracle as O
from test_gpu_gemm import make_case

pytestmark = pytest.mark.gpu


def big_activations(seed, m, k):
    """N(0,1) with 0.1 % of the channels x20 (the benchmark's law), drawn fast for hundreds of millions of values."""
    g = np.random.default_rng(seed)
    x = g.standard_normal((m, k), dtype=np.float32)
    ch = g.choice(k, max(1, round(k * 0.001)), replace=False)
    x[:, ch] *= 20.0
    return x.astype(np.float16)


@pytest.mark.parametrize("k", [4096, 11008, 14336])
def test_quantisers_at_16384_rows(cuda, k):
    m = 16384
    x = big_activations(500 + k, m, k)
    x[3] = 0.0                                   # an all-zero row
    xd = torch.from_numpy(x).cuda()
    rows = np.concatenate([[0, 1, 2, 3, m - 1], rs(k).choice(m, 27, replace=False)])

    # group-128 symmetric mode with the group transform: bit-exact
    q, s = cuda.hadamard_and_quantize_i4(xd.view(-1, 128))
    q, s = q.view(m, k // 2).cpu().numpy(), s.view(m, k // 128).cpu().numpy()
    qo, so = O.quant_group_sym(x[rows].reshape(-1, 128), True)
    assert np.array_equal(q[rows], qo.reshape(len(rows), k // 2))
    assert np.array_equal(s[rows].view(np.uint16), so.reshape(len(rows), k // 128).view(np.uint16))

    # per-token asymmetric, full-width transform in the reference's order: bit-exact
    qo, so, zo = O.quant_token_asym(x[rows], True)
    idx = torch.from_numpy(rows).cuda()
    q, s, z = cuda.quant_token_asym_i4(xd, hadamard=True, exact=True)
    assert np.array_equal(q[idx].cpu().numpy(), qo)
    assert np.array_equal(s[idx].cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(z[idx].cpu().numpy().view(np.uint16), zo.view(np.uint16))

    # default transform: stated tolerance on the sampled rows; every row of the launch must have produced parameters
    # (scale > 0, zero-point an integer in 0..15) and must agree with the exact launch on all but a sliver of codes
    q1, s1, z1 = cuda.quant_token_asym_i4(xd, hadamard=True)
    rate = assert_token_tolerance(q1[idx], s1[idx], z1[idx], qo, so, zo)
    assert bool((s1 > 0).all()) and bool(((z1 >= 0) & (z1 <= 15) & (z1 == z1.round())).all())
    lo, hi = (q1 & 15).to(torch.int16), (q1 >> 4).to(torch.int16)
    lo0, hi0 = (q & 15).to(torch.int16), (q >> 4).to(torch.int16)
    diff = ((lo - lo0).abs() + (hi - hi0).abs())
    all_rate = float((diff != 0).float().mean())
    assert int(diff.max()) <= 2 and all_rate <= 1e-3, (int(diff.max()), all_rate)
    print(f"K={k}: default transform, sampled rows vs oracle {rate:.2e}; all {m} rows vs the bit-exact launch {all_rate:.2e} of bytes differ")
    torch.cuda.synchronize()
    assert cuda.gemm_status()[0] == 0


@pytest.mark.parametrize("m", [16, 2048, 8192])
@pytest.mark.parametrize("mode", [(128, 128, False), (0, 0, True)], ids=["group128_sym", "token_asym_channel"])
def test_gemm_4096_to_22016(cuda, m, mode):
    """The widest benchmark GEMM (gate/up of Llama-2-13B-like width: 4096 -> 22016) at decode, prefill and large-prefill
    batches: sampled rows of the default algorithm against the oracle, bit for bit; and the independent kernels that
    serve the shape must agree with each other on every output."""
    n, k = 22016, 4096
    ap, bp, sa, sb, za, bi = make_case(700 + m, m, n, k, *mode, bias=True)
    dev = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()
    A, B, SA, SB, ZA, BI = dev(ap), dev(bp), dev(sa), dev(sb), dev(za), dev(bi)
    rsum = cuda.weight_rowsum(B, min(k // sa.shape[1], k // sb.shape[1])) if za is not None else None
    d = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI)            # AUTO
    rows = sorted({0, m - 1, m // 2, *rs(m).choice(m, min(m, 5), replace=False).tolist()})
    ref = O.gemm_i4_dequant(ap[rows], bp, sa[rows], sb, a_zero=None if za is None else za[rows], bias=bi)
    assert np.array_equal(d[rows].cpu().numpy().view(np.uint16), ref.view(np.uint16))
    if m >= 128:
        d2 = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI, algo=cuda.GEMM_TCGEN05)
        assert torch.equal(d.view(torch.int16), d2.view(torch.int16))
    else:
        d2 = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI, algo=cuda.GEMM_STREAM)
        assert torch.equal(d.view(torch.int16), d2.view(torch.int16))
    torch.cuda.synchronize()
    assert cuda.gemm_status()[0] == 0
