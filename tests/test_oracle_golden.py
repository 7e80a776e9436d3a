"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""
import numpy as np

from helpers import activations, rs
from oracle import oracle as O


def test_quant_and_pack_matches_forward_origin(golden):
    # no transform: forward_origin computes max/7 and x/scale in binary16, as the kernel's formula does
    x = activations(101, 24, 512)
    q, s = O.quant_group_sym(x.reshape(-1, 128), False)
    assert np.array_equal(q.reshape(24, -1), golden["aq_sym_nohad_q"])
    assert np.array_equal(s.reshape(24, 4), golden["aq_sym_nohad_scale"])


def test_had_and_quant_close_to_forward_origin(golden):
    # forward_origin transforms in float64; the kernel (and the oracle) in binary16: the reference's
    # own check allows |dq| <= 1 (test/test_had_and_quant.py:20); here also a rate bound.
    x = activations(101, 24, 512)
    q, s = O.quant_group_sym(x.reshape(-1, 128), True)
    cq, cr = O.unpack_i4(q.reshape(24, -1)), O.unpack_i4(golden["aq_sym_had_q"])
    assert np.abs(cq - cr).max() <= 1
    assert (cq != cr).mean() < 0.005
    rel = np.abs(s.reshape(24, 4).astype(np.float32) / np.sqrt(128) / golden["aq_sym_had_scale"].astype(np.float32) - 1)
    assert rel.max() < 4e-3


def test_fht_f16_close_to_float64(golden):
    x = activations(101, 24, 512)
    f = O.fht_f16(x.reshape(-1, 128)).astype(np.float64).reshape(24, 512) / np.sqrt(128)
    ref = golden["fht128_f64"]
    assert np.abs(f - ref).max() <= 2e-3 * np.abs(ref).max()


def test_full_hadamard_bit_exact(golden):
    for n, m in ((4096, 3), (8192, 2), (11008, 2), (14336, 2), (28672, 1), (3584, 2), (1536, 2)):
        xi = activations(200 + n % 97, m, n).astype(np.float32)
        y = O.had_full_f32(xi)
        assert np.array_equal(y.view(np.uint32), golden[f"hadU_{n}"].view(np.uint32)), n


def test_token_asym_against_fake_quant(golden):
    for n, m in ((4096, 4), (11008, 2), (14336, 2)):
        xi = activations(300 + n % 97, m, n)
        q, s, z = O.quant_token_asym(xi, True, exact_norm=True)
        # reference functions evaluated with the f16-rounded scale: identical
        assert np.array_equal(q, golden[f"fq_{n}_q16"])
        assert np.array_equal(s, golden[f"fq_{n}_scale16"])
        assert np.array_equal(z.astype(np.float32), golden[f"fq_{n}_zero16"])
        # the kernel's arithmetic (normalisation folded into the scale): same stored triple here
        q2, s2, z2 = O.quant_token_asym(xi, True, exact_norm=False)
        assert np.array_equal(s, s2) and np.array_equal(z, z2)
        assert (O.unpack_i4(q2, False) != O.unpack_i4(q, False)).mean() <= 1e-4
        # against the pure reference (binary32 scale): <= 0.1 % of codes off by one
        c, c32 = O.unpack_i4(q2, False), O.unpack_i4(golden[f"fq_{n}_q32"], False)
        assert np.abs(c - c32).max() <= 1 and (c != c32).mean() <= 1e-3


def test_weight_rtn_and_pack_match_from_float(golden):
    qw, sw = O.rtn_group_sym(golden["lin_w_had"], 128)
    assert np.array_equal(O.pack_i4(qw), golden["lin_w_packed"])
    assert np.array_equal(sw.astype(np.float32), golden["lin_w_scale"])
    assert np.array_equal(O.unpack_i4(O.pack_i4(qw)), qw)


def test_gemm_against_forward_torch(golden):
    r = rs(401)
    r.standard_normal((64, 256))
    r.randint(-8, 8, size=(5, 256))
    xs = r.uniform(0.005, 0.02, size=(5, 2)).astype(np.float16)
    d = O.gemm_i4_dequant(golden["lin_x_packed"], golden["lin_w_packed"], xs, golden["lin_w_scale"].astype(np.float16))
    ref = golden["lin_fwd_torch"]
    assert np.abs(d.astype(np.float32) - ref).max() <= 1e-3 * np.abs(ref).max()
    c = O.gemm_i4_int32(golden["lin_x_packed"], golden["lin_w_packed"], 128)
    ci = np.einsum("mgk,ngk->mng", O.unpack_i4(golden["lin_x_packed"]).reshape(5, 2, 128),
                   O.unpack_i4(golden["lin_w_packed"]).reshape(64, 2, 128))
    assert np.array_equal(c, ci)


def test_gemm_zero_point_identity():
    # asymmetric epilogue == dequantise-then-matmul in float64
    m, n, k = 7, 128, 512
    a = rs(1).randint(0, 16, size=(m, k)); b = rs(2).randint(-8, 8, size=(n, k))
    sa = rs(3).uniform(0.005, 0.02, (m, 1)).astype(np.float16); za = rs(4).randint(0, 16, (m, 1)).astype(np.float16)
    for gb in (1, k // 128):
        sb = rs(5).uniform(0.005, 0.02, (n, gb)).astype(np.float16)
        d = O.gemm_i4_dequant(O.pack_i4(a), O.pack_i4(b), sa, sb, a_zero=za).astype(np.float64)
        af = (a - za.astype(np.float64)) * sa.astype(np.float64)
        bf = (b.reshape(n, gb, -1) * sb.astype(np.float64)[:, :, None]).reshape(n, k)
        ref = af @ bf.T
        assert np.abs(d - ref).max() <= 2e-3 * np.abs(ref).max()
    rsum = O.weight_rowsum(O.pack_i4(b), 128)
    assert np.array_equal(rsum, b.reshape(n, -1, 128).sum(-1))
