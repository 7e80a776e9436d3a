"""GPU parity of the int4 GEMM + dequant kernels against the CPU oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import int4_codes, rs, scales
from oracle import oracle as O

pytestmark = pytest.mark.gpu

STREAM, MMA, TC, SPLITK, DECODE_TC = 3, 2, 1, 4, 8


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_case(seed, m, n, k, a_group, b_group, asym, bias=False, neg_scales=False):
    a = int4_codes(seed, m, k, unsigned=asym)
    b = int4_codes(seed + 1, n, k)
    ga = 1 if a_group == 0 else k // a_group
    gb = 1 if b_group == 0 else k // b_group
    sa, sb = scales(seed + 2, m, ga), scales(seed + 3, n, gb)
    if neg_scales:
        sa = (rs(seed + 6).standard_normal((m, ga)) * 0.02).astype(np.float16)
        sb = (rs(seed + 7).standard_normal((n, gb)) * 0.02).astype(np.float16)
    za = rs(seed + 4).randint(0, 16, size=(m, ga)).astype(np.float16) if asym else None
    bi = (rs(seed + 5).standard_normal(n) * 0.1).astype(np.float16) if bias else None
    ap = O.pack_i4(a) if not asym else ((a[:, 0::2] & 15) | ((a[:, 1::2] & 15) << 4)).astype(np.uint8)
    return ap, O.pack_i4(b), sa, sb, za, bi


def run_case(cuda, algo, case, bf16=False):
    ap, bp, sa, sb, za, bi = case
    k = ap.shape[1] * 2
    rsum = None
    if za is not None:
        grp = min(k // sa.shape[1], k // sb.shape[1])
        rsum = cuda.weight_rowsum(_dev(bp), grp)
        assert np.array_equal(rsum.cpu().numpy(), O.weight_rowsum(bp, grp))
    d = cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), A_zero=None if za is None else _dev(za),
                             B_rowsum=rsum, bias=None if bi is None else _dev(bi),
                             out_dtype=torch.bfloat16 if bf16 else torch.float16, algo=algo)
    ref = O.gemm_i4_dequant(ap, bp, sa, sb, a_zero=za, bias=bi, bf16_out=bf16)
    got = d.view(torch.int16).cpu().numpy().view(np.uint16)
    want = ref.view(np.uint16)
    bad = got != want
    assert not bad.any(), f"{bad.sum()} of {bad.size} outputs differ; first at {np.argwhere(bad)[0]}"


MODES = [  # (a_group, b_group, asym): 0 stands for "whole K"
    (128, 128, False),   # the flh._CUDA contract
    (0, 0, True),        # per-token asymmetric x per-channel weights
    (0, 128, True),      # per-token asymmetric x group-128 weights
    (128, 0, False),
    (0, 0, False),
    (128, 128, True),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 33, 64])
def test_stream_kernel(cuda, mode, m):
    run_case(cuda, STREAM, make_case(10 * m, m, 256, 1024, *mode))


@pytest.mark.parametrize("m,n,k", [(1, 1024, 2048), (16, 128, 128), (16, 384, 1152), (32, 4096, 4096), (8, 4096, 11008)])
def test_stream_kernel_shapes(cuda, m, n, k):
    run_case(cuda, STREAM, make_case(m + n + k, m, n, k, 128, 128, False))
    run_case(cuda, STREAM, make_case(m + n + k + 1, m, n, k, 0, 0, True, bias=True), bf16=True)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 4096, 11008), (32, 1024, 2048), (7, 256, 4096), (64, 1024, 8192)])
def test_stream_splitk(cuda, m, n, k):
    """K cut across CTAs (decode shapes with few output columns).  Without group scales the partial sums
    are int32 and the result equals the oracle bit for bit; with group scales every split keeps its own
    binary32 chain and the chains are added in split order: within 1e-3 of the oracle, and the same bits
    on every run."""
    assert cuda._lib.load().flh_b200_gemm_pick_algo(m, n, k, 128, 128) == SPLITK
    run_case(cuda, SPLITK, make_case(m + n, m, n, k, 0, 0, True, bias=True))
    run_case(cuda, SPLITK, make_case(m + n + 1, m, n, k, 0, 0, False), bf16=True)
    ap, bp, sa, sb, _, _ = make_case(m + n + 2, m, n, k, 128, 128, False)
    A, B, SA, SB = _dev(ap), _dev(bp), _dev(sa), _dev(sb)
    d1 = cuda.gemm_i4_dequant(A, B, SA, SB, algo=SPLITK)
    d2 = cuda.gemm_i4_dequant(A, B, SA, SB, algo=SPLITK)
    d0 = cuda.gemm_i4_dequant(A, B, SA, SB, algo=STREAM)            # single chain == oracle
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    ref = O.gemm_i4_dequant(ap, bp, sa, sb)
    assert np.array_equal(d0.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    err = (d1.float() - d0.float()).abs()
    assert bool((err <= 1e-3 * d0.float().abs() + 1e-3 * d0.float().abs().mean()).all()), err.max().item()


def _close(d, ref16):
    """Within 1e-3 of the single-chain result (relative, with a floor of 1e-3 of the mean magnitude)."""
    got, ref = d.float().cpu().numpy(), ref16.astype(np.float32)
    err = np.abs(got - ref)
    return bool((err <= 1e-3 * np.abs(ref) + 1e-3 * np.abs(ref).mean()).all()), float(err.max())


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 33, 64])
def test_decode_tc_kernel(cuda, mode, m):
    """The tensor-core decode kernel (weights on the MMA's M side, K-ranges balanced across CTAs).  Without group
    scales the CTAs that share a tile hand over int32 sums: equal to the oracle bit for bit.  With group scales each
    CTA keeps its own binary32 chain and the chains are added in K order: within 1e-3 of the oracle, the same bits
    on every run."""
    case = make_case(30 * m, m, 256, 1024, *mode, bias=(m == 17))
    ap, bp, sa, sb, za, bi = case
    if mode[0] == 0 and mode[1] == 0:
        run_case(cuda, DECODE_TC, case, bf16=(m == 33))
        return
    k = ap.shape[1] * 2
    rsum = None if za is None else cuda.weight_rowsum(_dev(bp), min(k // sa.shape[1], k // sb.shape[1]))
    args = (_dev(ap), _dev(bp), _dev(sa), _dev(sb))
    kw = dict(A_zero=None if za is None else _dev(za), B_rowsum=rsum, bias=None if bi is None else _dev(bi), algo=DECODE_TC)
    d1, d2 = cuda.gemm_i4_dequant(*args, **kw), cuda.gemm_i4_dequant(*args, **kw)
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    ok, worst = _close(d1, O.gemm_i4_dequant(ap, bp, sa, sb, a_zero=za, bias=bi))
    assert ok, worst


@pytest.mark.parametrize("m,n,k", [(4, 128, 512), (16, 128, 128), (40, 128, 384)])
def test_decode_tc_whole_tiles(cuda, m, n, k):
    """A tile whose K lies in one CTA keeps a single chain: bit-exact with group scales too."""
    for mode in MODES:
        run_case(cuda, DECODE_TC, make_case(m + k, m, n, k, *mode))


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (5, 1024, 11008), (64, 1152, 2304), (32, 8192, 3584)])
def test_decode_tc_shapes(cuda, m, n, k):
    run_case(cuda, DECODE_TC, make_case(m + n + k, m, n, k, 0, 0, True, bias=True))
    run_case(cuda, DECODE_TC, make_case(m + n + k + 1, m, n, k, 0, 0, False), bf16=True)
    ap, bp, sa, sb, _, _ = make_case(m + n + 2, m, n, k, 128, 128, False)
    d = cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), algo=DECODE_TC)
    ok, worst = _close(d, O.gemm_i4_dequant(ap, bp, sa, sb))
    assert ok, worst
    st = cuda.gemm_status()
    assert st[0] == 0, st


def test_decode_kernels_share_one_workspace(cuda):
    """Split-K and the tensor-core decode kernel alternate on one stream's workspace: each leaves the arrival counters
    zero and treats the rest as scratch, so results do not depend on what ran before."""
    big = make_case(77, 64, 8192, 2048, 0, 0, True)
    small = make_case(78, 16, 1024, 4096, 128, 128, False)
    for _ in range(2):
        run_case(cuda, DECODE_TC, big)
        ap, bp, sa, sb, _, _ = small
        d = cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), algo=SPLITK)
        ok, worst = _close(d, O.gemm_i4_dequant(ap, bp, sa, sb))
        assert ok, worst
    run_case(cuda, DECODE_TC, make_case(79, 40, 1024, 4096, 0, 0, False))


def test_auto_picks_decode_tc_for_large_decode_shapes(cuda):
    pick = cuda._lib.load().flh_b200_gemm_pick_algo
    assert pick(64, 8192, 8192, 128, 128) == DECODE_TC          # 32 MiB of weights, 64 tokens
    assert pick(32, 8192, 8192, 8192, 8192) == DECODE_TC
    assert pick(16, 28672, 8192, 128, 128) == DECODE_TC         # 112 MiB
    assert pick(16, 152064, 4096, 4096, 4096) == STREAM         # more tiles than the counters cover
    assert pick(16, 22016, 4096, 128, 128) == STREAM            # 43 MiB at 16 tokens: the streaming kernel
    assert pick(16, 4096, 4096, 128, 128) == SPLITK
    assert pick(128, 8192, 8192, 128, 128) == TC


def test_reference_script_case(cuda):
    # test/test_gemm_dequant.py: M=1, N=1024, K=2048, signed codes, N(0,1)-like scales of both signs
    run_case(cuda, STREAM, make_case(0, 1, 1024, 2048, 128, 128, False, neg_scales=True))
    run_case(cuda, MMA, make_case(0, 1, 1024, 2048, 128, 128, False, neg_scales=True))


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m", [1, 64, 129, 300])
def test_mma_tile_kernel(cuda, mode, m):
    run_case(cuda, MMA, make_case(20 * m, m, 256, 1024, *mode))


def test_mma_tile_kernel_bias_bf16(cuda):
    run_case(cuda, MMA, make_case(5, 200, 384, 2048, 0, 0, True, bias=True), bf16=True)
    run_case(cuda, MMA, make_case(6, 130, 128, 128, 128, 128, False, bias=True))


@pytest.mark.parametrize("gs", [32, 64])
@pytest.mark.parametrize("m", [1, 16, 130, 300])
@pytest.mark.parametrize("groups", [("g", "g", False), ("g", "g", True), (0, "g", True), ("g", 0, False)])
def test_group_32_64(cuda, gs, m, groups):
    """K-groups of 32 and 64 (the reference's *_gs entry points, flh/kernels/gemm_and_dequant_i4_gs.cu:335-492), every
    group scaled with its own scales: bit-exact against the oracle, which folds one exact integer sum per group."""
    ag, bg, asym = groups
    ag, bg = (gs if ag == "g" else 0), (gs if bg == "g" else 0)
    run_case(cuda, 0, make_case(60 * m + gs, m, 256, 1024, ag, bg, asym, bias=(m == 16)), bf16=(m == 130))


@pytest.mark.parametrize("gs", [32, 64, 128])
def test_gs_binding(cuda, gs):
    """gemm_i4_dequant_o16_gs (flh/cuda/flh_cuda_bindings.cpp:253-299) with the scale shapes the reference's
    quantiser emits, [.., K / gs]: equal to the oracle; and a wrong scale shape raises as TORCH_CHECK does."""
    m, n, k = 70, 384, 2048
    ap, bp, sa, sb, _, _ = make_case(900 + gs, m, n, k, gs, gs, False)
    d = cuda.gemm_i4_dequant_o16_gs(_dev(ap), _dev(bp), _dev(sa), _dev(sb), gs)
    ref = O.gemm_i4_dequant(ap, bp, sa, sb)
    assert np.array_equal(d.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant_o16_gs(_dev(ap), _dev(bp), _dev(sa)[:, :-1].contiguous(), _dev(sb), gs)
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant_o16_gs(_dev(ap), _dev(bp), _dev(sa), _dev(sb), 48)


def test_c_symbol_of_the_reference(cuda):
    # flhDenseLayerGEMM_i4_o16: same signature as flh/kernels/gemm_and_dequant_i4.cu:471-480
    import ctypes
    from flh_b200 import _lib
    ap, bp, sa, sb, _, _ = make_case(3, 16, 256, 512, 128, 128, False)
    A, B, SA, SB = _dev(ap), _dev(bp), _dev(sa), _dev(sb)
    D = torch.empty((16, 256), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    _lib.load().flhDenseLayerGEMM_i4_o16(A.data_ptr(), B.data_ptr(), SA.data_ptr(), SB.data_ptr(), D.data_ptr(), 16, 256, 512)
    torch.cuda.synchronize()
    assert np.array_equal(D.cpu().numpy().view(np.uint16), O.gemm_i4_dequant(ap, bp, sa, sb).view(np.uint16))


def test_gemm_argument_errors(cuda):
    ap, bp, sa, sb, _, _ = make_case(3, 4, 128, 256, 128, 128, False)
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant_o16(_dev(ap).cpu(), _dev(bp), _dev(sa), _dev(sb))
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant_o16(_dev(ap), _dev(bp)[:, :64].contiguous(), _dev(sa), _dev(sb))
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant(_dev(ap), _dev(bp)[:100].contiguous(), _dev(sa), _dev(sb)[:100].contiguous())  # N % 128
    with pytest.raises(RuntimeError):
        cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), A_zero=_dev(sa))    # zero-point without row sums
