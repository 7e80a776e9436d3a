"""GPU parity of the int8-operand tcgen05 GEMM (operands expanded into a workspace first; one CTA per tile, or
two-CTA clusters on 256 x 256 tiles) against the CPU oracle, bit-exact.  Per-token / per-channel scales only."""
import numpy as np
import pytest
import torch

from test_gpu_gemm import TC, make_case, run_case, _dev
from oracle import oracle as O

pytestmark = pytest.mark.gpu

I8, I8_PAIR = 6, 7
ALGOS = [pytest.param(I8, id="cta1"), pytest.param(I8_PAIR, id="pair")]
UNGROUPED = [(0, 0, True), (0, 0, False)]      # (a_group, b_group, asym); 0 = whole K


@pytest.fixture(autouse=True)
def _status_clean(cuda):
    yield
    torch.cuda.synchronize()
    st = cuda.gemm_status()
    assert st[0] == 0, f"a bounded wait in a tcgen05 kernel ran out: code {st[0]} in CTA {st[1]}"


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("mode", UNGROUPED)
def test_i8_single_tile(cuda, algo, mode):
    run_case(cuda, algo, make_case(131, 128, 256, 512, *mode))
    run_case(cuda, algo, make_case(132, 256, 256, 128, *mode))


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("mode", UNGROUPED)
@pytest.mark.parametrize("m", [1, 100, 129, 257, 515])
def test_i8_ragged_m(cuda, algo, mode, m):
    run_case(cuda, algo, make_case(140 + m, m, 512, 1024, *mode, bias=True), bf16=(m % 2 == 1))


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("mode", UNGROUPED)
def test_i8_more_tiles_than_sms(cuda, algo, mode):
    # 180 tiles of 128 x 256 (90 of 256 x 256): persistent CTAs take several tiles, both TMEM buffers cycle
    run_case(cuda, algo, make_case(177, 300, 15360, 512, *mode))


@pytest.mark.parametrize("m,n,k", [(256, 1024, 4096), (512, 4096, 11008), (2048, 512, 128)])
@pytest.mark.parametrize("algo", ALGOS)
def test_i8_shapes(cuda, algo, m, n, k):
    run_case(cuda, algo, make_case(m + n, m, n, k, 0, 0, True, bias=True), bf16=True)
    run_case(cuda, algo, make_case(m + n + 1, m, n, k, 0, 0, False, neg_scales=True))


def test_i8_n_multiple_of_128_only(cuda):
    run_case(cuda, I8, make_case(178, 260, 384, 1024, 0, 0, True, bias=True))
    ap, bp, sa, sb, za, _ = make_case(179, 260, 384, 1024, 0, 0, False)
    with pytest.raises(RuntimeError, match="256"):      # rejected on the host: nothing is launched
        cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), algo=I8_PAIR)


def test_i8_rejects_group_scales(cuda):
    ap, bp, sa, sb, za, _ = make_case(180, 128, 256, 512, 128, 128, False)
    with pytest.raises(RuntimeError, match="per-token"):
        cuda.gemm_i4_dequant(_dev(ap), _dev(bp), _dev(sa), _dev(sb), algo=I8)


@pytest.mark.parametrize("algo", ALGOS)
def test_i8_prefill_size_against_converting_kernel(cuda, algo):
    # 4096 -> 12288 at M = 2048: the independent GPU paths must agree bit for bit; sampled rows against the oracle
    ap, bp, sa, sb, za, bi = make_case(199, 2048, 12288, 4096, 0, 0, True, bias=True)
    A, B, SA, SB, ZA, BI = _dev(ap), _dev(bp), _dev(sa), _dev(sb), _dev(za), _dev(bi)
    rsum = cuda.weight_rowsum(B, 4096)
    d1 = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI, algo=algo)
    d2 = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI, algo=TC)
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    rows = [0, 127, 128, 255, 256, 1000, 2047]
    ref = O.gemm_i4_dequant(ap[rows], bp, sa[rows], sb, a_zero=za[rows], bias=bi)
    assert np.array_equal(d1[rows].cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (300, 512, 1024), (515, 384, 2048), (2048, 4096, 4096)])
def test_i8_prepacked_weights(cuda, m, n, k):
    """Weights expanded once (expand_i4), activations per call: same bits as the general entry point."""
    for asym in (True, False):
        ap, bp, sa, sb, za, bi = make_case(300 + m, m, n, k, 0, 0, asym, bias=True)
        A, B, SA, SB, BI = _dev(ap), _dev(bp), _dev(sa), _dev(sb), _dev(bi)
        ZA = _dev(za) if asym else None
        rsum = cuda.weight_rowsum(B, k) if asym else None
        B8 = cuda.expand_i4(B)
        # the expansion itself: every 32 elements, the 16 even ones then the 16 odd ones, each 16 * q as a byte
        q = (O.unpack_i4(bp, True).astype(np.int32) * 16).astype(np.uint8).reshape(n, k // 32, 16, 2)
        want = np.concatenate([q[..., 0], q[..., 1]], axis=-1).reshape(n, k)
        assert np.array_equal(B8.cpu().numpy(), want)
        d1 = cuda.gemm_i8w_dequant(A, B8, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI)
        d2 = cuda.gemm_i4_dequant(A, B, SA, SB, A_zero=ZA, B_rowsum=rsum, bias=BI, algo=TC)
        assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
        if m <= 515:
            ref = O.gemm_i4_dequant(ap, bp, sa, sb, a_zero=za, bias=bi)
            assert np.array_equal(d1.cpu().numpy().view(np.uint16), ref.view(np.uint16))


def test_i8_auto_selection_and_module(cuda):
    from flh_b200 import _lib
    from flh_b200.nn import LinearFLH
    lib = _lib.load()
    assert lib.flh_b200_gemm_pick_algo(2048, 4096, 4096, 4096, 4096) == I8_PAIR
    assert lib.flh_b200_gemm_pick_algo(2048, 384, 4096, 4096, 4096) == I8
    assert lib.flh_b200_gemm_pick_algo(512, 4096, 4096, 4096, 4096) == TC
    assert lib.flh_b200_gemm_pick_algo(2048, 4096, 4096, 128, 128) == TC
    assert lib.flh_b200_gemm_workspace_bytes(2048, 4096, 4096, 4096, 4096, 0) == (2048 + 4096) * 4096
    # a module with and without the int8 copy gives the same output
    m, k, n = 1100, 1024, 768
    ap, bp, sa, sb, za, _ = make_case(400, m, n, k, 0, 0, True)
    lin = LinearFLH(k, n, device="cuda", group_size=-1)
    lin.w_packed.copy_(_dev(bp).reshape(-1)); lin.w_scale.copy_(_dev(sb))
    y0 = lin(_dev(ap), _dev(sa), _dev(za))
    y1 = lin.prepack_int8()(_dev(ap), _dev(sa), _dev(za))
    assert lin._w_i8 is not None and torch.equal(y0.view(torch.int16), y1.view(torch.int16))
