"""The B200 kernels against the reference's own CUDA kernels (compiled for sm_100a from the FLH
checkout into oracle/_ref/libflh_ref.so), on the same device and inputs.

The reference divides with rcp.approx (not reproducible off the GPU), the B200 kernels with a
correctly rounded reciprocal, so the quantiser comparison is statistical: at most 0.1 % of codes may
differ, by one step.  GEMM outputs must agree within 1e-3 relative error."""
import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import activations
from test_gpu_gemm import make_case, _dev

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libflh_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libflh_ref.so was not built (needs the FLH checkout: make -C oracle ref)")
    lib = ctypes.CDLL(REF)
    for f in (lib.flh_ref_had_and_quant, lib.flh_ref_quant_and_pack):
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
        f.restype = None
    lib.flh_ref_gemm_i4_o16.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_size_t] * 3
    lib.flh_ref_gemm_i4_o16.restype = None
    return lib


@pytest.mark.parametrize("had", [True, False])
def test_quantiser_against_reference_kernel(cuda, ref, had):
    rows = 65536
    x = _dev(activations(4242, rows, 128, outlier_frac=0.01))
    q_ref = torch.empty((rows, 64), dtype=torch.uint8, device="cuda")
    s_ref = torch.empty((rows,), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    (ref.flh_ref_had_and_quant if had else ref.flh_ref_quant_and_pack)(x.data_ptr(), q_ref.data_ptr(), s_ref.data_ptr(), rows)
    assert ref.flh_ref_sync() == 0
    q, s = (cuda.hadamard_and_quantize_i4 if had else cuda.quant_and_pack_i4)(x)
    torch.cuda.synchronize()
    from oracle import oracle as O
    c, cr = O.unpack_i4(q.cpu().numpy()), O.unpack_i4(q_ref.cpu().numpy())
    assert np.abs(c - cr).max() <= 1
    rate = (c != cr).mean()
    srate = (s != s_ref).float().mean().item()
    print(f"hadamard={had}: code mismatch rate {rate:.2e}, scale mismatch rate {srate:.2e}")
    assert rate <= 1e-3
    sd = (s.float() - s_ref.float()).abs() / s_ref.float()
    assert sd.max().item() <= 1.0 / 1024 and srate <= 1e-2


@pytest.mark.parametrize("m", [1, 16, 128, 700])
def test_gemm_against_reference_kernel(cuda, ref, m):
    ap, bp, sa, sb, _, _ = make_case(500 + m, m, 1024, 2048, 128, 128, False)
    A, B, SA, SB = _dev(ap), _dev(bp), _dev(sa), _dev(sb)
    d_ref = torch.empty((m, 1024), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    ref.flh_ref_gemm_i4_o16(A.data_ptr(), B.data_ptr(), SA.data_ptr(), SB.data_ptr(), d_ref.data_ptr(), m, 1024, 2048)
    assert ref.flh_ref_sync() == 0
    for algo in (0, 2):
        d = cuda.gemm_i4_dequant(A, B, SA, SB, algo=algo)
        torch.cuda.synchronize()
        err = (d.float() - d_ref.float()).abs()
        tol = 1e-3 * d_ref.float().abs() + 1e-3 * d_ref.float().abs().mean()
        assert bool((err <= tol).all()), f"algo {algo}: max err {err.max().item()}"
        print(f"m={m} algo={algo}: bit-identical outputs {(d == d_ref).float().mean().item():.4f}")


def _time(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / iters


def test_speed_against_reference_kernels(cuda, ref):
    """The reference's own kernels, compiled for sm_100a, timed beside the B200 kernels on the same inputs
    (CUDA events, back-to-back launches on the legacy default stream, which is torch's current stream here)."""
    rows = 16384 * 32                                  # X[16384, 4096] as groups of 128
    x = torch.randn(rows, 128, device="cuda", dtype=torch.float16)
    q_ref = torch.empty((rows, 64), dtype=torch.uint8, device="cuda")
    s_ref = torch.empty((rows,), dtype=torch.float16, device="cuda")
    t_ref = _time(lambda: ref.flh_ref_had_and_quant(x.data_ptr(), q_ref.data_ptr(), s_ref.data_ptr(), rows))
    t_new = _time(lambda: cuda.hadamard_and_quantize_i4(x))
    print(f"\nhad+quant 524288x128: reference kernel {t_ref * 1e6:.1f} us, flh_b200 {t_new * 1e6:.1f} us, x{t_ref / t_new:.2f}")
    assert t_new < t_ref

    m, n, k = 2048, 12288, 4096
    ap, bp, sa, sb, _, _ = make_case(900, m, n, k, 128, 128, False)
    A, B, SA, SB = _dev(ap), _dev(bp), _dev(sa), _dev(sb)
    d_ref = torch.empty((m, n), dtype=torch.float16, device="cuda")
    t_ref = _time(lambda: ref.flh_ref_gemm_i4_o16(A.data_ptr(), B.data_ptr(), SA.data_ptr(), SB.data_ptr(), d_ref.data_ptr(), m, n, k), iters=10)
    t_new = _time(lambda: cuda.gemm_i4_dequant(A, B, SA, SB), iters=10)
    d = cuda.gemm_i4_dequant(A, B, SA, SB)
    torch.cuda.synchronize()
    same = (d == d_ref).float().mean().item()
    print(f"GEMM M={m} {k}->{n} g128: reference kernel {t_ref * 1e6:.1f} us ({2 * m * n * k / t_ref / 1e12:.0f} TOPS), "
          f"flh_b200 {t_new * 1e6:.1f} us ({2 * m * n * k / t_new / 1e12:.0f} TOPS), x{t_ref / t_new:.2f}; identical outputs {same:.4f}")
    assert same == 1.0 and t_new < t_ref

    m = 16
    A, SA = A[:m].contiguous(), SA[:m].contiguous()
    d_ref = torch.empty((m, n), dtype=torch.float16, device="cuda")
    t_ref = _time(lambda: ref.flh_ref_gemm_i4_o16(A.data_ptr(), B.data_ptr(), SA.data_ptr(), SB.data_ptr(), d_ref.data_ptr(), m, n, k))
    t_new = _time(lambda: cuda.gemm_i4_dequant(A, B, SA, SB))
    print(f"GEMM M={m} {k}->{n} g128: reference kernel {t_ref * 1e6:.1f} us, flh_b200 {t_new * 1e6:.1f} us, x{t_ref / t_new:.2f} "
          f"(single launches, host launch cost included in both)")
