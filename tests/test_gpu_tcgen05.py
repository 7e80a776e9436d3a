"""GPU parity of the tcgen05 (TMA + TMEM) GEMM against the CPU oracle, bit-exact."""
import numpy as np
import pytest
import torch

from test_gpu_gemm import MODES, TC, MMA, make_case, run_case, _dev
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean(cuda):
    yield
    torch.cuda.synchronize()
    st = cuda.gemm_status()
    assert st[0] == 0, f"a bounded wait in the tcgen05 kernel ran out: code {st[0]} in CTA {st[1]}"


TCD = 5        # the direct-load variant (converter warps fetch packed operands from L2 into registers)


@pytest.mark.parametrize("mode", MODES)
def test_tcgen05_single_tile(cuda, mode):
    run_case(cuda, TC, make_case(31, 128, 256, 512, *mode))


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (1, 384, 1024), (515, 384, 1024), (300, 15360, 512), (256, 1024, 4096)])
def test_tcgen05_direct_variant(cuda, mode, m, n, k):
    run_case(cuda, TCD, make_case(m + n + k, m, n, k, *mode))


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m", [1, 100, 129, 515])
def test_tcgen05_ragged_m(cuda, mode, m):
    run_case(cuda, TC, make_case(40 + m, m, 384, 1024, *mode))


@pytest.mark.parametrize("m,n,k", [(256, 1024, 4096), (512, 4096, 11008), (2048, 512, 128)])
def test_tcgen05_shapes(cuda, m, n, k):
    run_case(cuda, TC, make_case(m + n, m, n, k, 128, 128, False))
    run_case(cuda, TC, make_case(m + n + 1, m, n, k, 0, 0, True, bias=True), bf16=True)


@pytest.mark.parametrize("mode", MODES)
def test_tcgen05_more_tiles_than_sms(cuda, mode):
    # 3 row blocks x 60 column blocks = 180 tiles: the persistent CTAs each take more than one tile
    run_case(cuda, TC, make_case(77, 300, 15360, 512, *mode))


def test_tcgen05_n_multiple_of_128_only(cuda):
    # N = 384 is not a multiple of 256: the 128-column variant
    run_case(cuda, TC, make_case(78, 260, 384, 1024, 128, 128, False))
    run_case(cuda, TC, make_case(79, 260, 384, 1024, 0, 0, True, bias=True))


def test_tcgen05_prefill_size_against_mma_path(cuda):
    # the benchmark shape 4096 -> 12288 at M = 2048: too big for the CPU oracle in seconds, so the two
    # independent GPU paths must agree bit for bit, and sampled rows are checked against the oracle.
    ap, bp, sa, sb, za, _ = make_case(99, 2048, 12288, 4096, 128, 128, False)
    A, B, SA, SB = _dev(ap), _dev(bp), _dev(sa), _dev(sb)
    d1 = cuda.gemm_i4_dequant(A, B, SA, SB, algo=TC)
    d2 = cuda.gemm_i4_dequant(A, B, SA, SB, algo=MMA)
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    rows = [0, 127, 128, 1000, 2047]
    ref = O.gemm_i4_dequant(ap[rows], bp, sa[rows], sb)
    assert np.array_equal(d1[rows].cpu().numpy().view(np.uint16), ref.view(np.uint16))
