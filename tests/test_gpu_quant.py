"""GPU parity of the activation quantisers against the CPU oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import activations, assert_token_tolerance, rs
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("gs", [128, 64, 32])
@pytest.mark.parametrize("had", [True, False])
@pytest.mark.parametrize("rows", [1, 3, 257, 4099])
def test_group_sym_bit_exact(cuda, gs, had, rows):
    x = activations(1000 + rows + gs, rows, gs, outlier_frac=0.02)
    fn = cuda.hadamard_and_quantize_i4_gs if had else cuda.quant_and_pack_i4_gs
    q, s = fn(_dev(x), gs)
    qo, so = O.quant_group_sym(x, had)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("gs", [128, 64, 32])
@pytest.mark.parametrize("had", [True, False])
@pytest.mark.parametrize("rows", [4096, 20001, 200003])
def test_group_sym_many_groups(cuda, gs, had, rows):
    """Large inputs run the thread-per-group kernel (persistent warps, 32 groups per tile, ragged last tile)."""
    x = activations(900 + rows % 97 + gs, rows // 32 + 1, gs * 32).reshape(-1, gs)[:rows]
    x = np.ascontiguousarray(x)
    f = cuda.hadamard_and_quantize_i4_gs if had else cuda.quant_and_pack_i4_gs
    q, s = f(_dev(x), gs)
    qo, so = O.quant_group_sym(x, had)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)


def test_group_sym_edge_values(cuda):
    # all-zero groups (scale -> 1), tiny groups (scale in the subnormal correction range),
    # a saturating group, negative zero
    x = np.zeros((6, 128), dtype=np.float16)
    x[1, :] = 3e-6
    x[1, ::2] *= -1
    x[2, :] = np.linspace(-6e-5, 6e-5, 128)
    x[3, :] = 500.0                 # 128 * 500 is the largest sum the binary16 transform can hold
    x[3, 5] = -500.0
    x[4, :] = -0.0
    x[5, :] = rs(5).standard_normal(128) * 1e-3
    for had, fn in ((True, cuda.hadamard_and_quantize_i4), (False, cuda.quant_and_pack_i4)):
        if not had:
            x[3, :] = 60000.0       # near the binary16 maximum; only without the transform, where
            x[3, 5] = -60000.0      # nothing overflows (non-finite intermediates are unspecified)
        q, s = fn(_dev(x))
        qo, so = O.quant_group_sym(x, had)
        assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16)), had
        assert np.array_equal(q.cpu().numpy(), qo), had


def test_group_sym_full_size(cuda):
    # the benchmark sweep size M=4096, K=4096: round trip property + sampled oracle rows
    x = activations(77, 4096, 4096)
    q, s = cuda.hadamard_and_quantize_i4(_dev(x).view(-1, 128))
    q, s = q.cpu().numpy(), s.cpu().numpy()
    idx = rs(9).choice(q.shape[0], 4096, replace=False)
    qo, so = O.quant_group_sym(x.reshape(-1, 128)[idx], True)
    assert np.array_equal(q[idx], qo) and np.array_equal(s[idx].view(np.uint16), so.view(np.uint16))
    # dequantised codes reproduce the transformed input within half a step (plus f16 rounding)
    t = O.fht_f16(x.reshape(-1, 128)[idx]).astype(np.float32)
    deq = O.unpack_i4(q[idx]).astype(np.float32) * s[idx].astype(np.float32)[:, None]
    assert np.all(np.abs(deq - t) <= 0.51 * s[idx].astype(np.float32)[:, None] + 1e-2 * np.abs(t))


@pytest.mark.parametrize("n", [128, 64, 32])
@pytest.mark.parametrize("rows", [1, 5, 1024, 5000])
def test_fht_inplace_bit_exact(cuda, n, rows):
    x = activations(2000 + rows + n, rows, n, outlier_frac=0.02)
    fn = {128: cuda.hadamard_transform_half, 64: cuda.hadamard_transform_64_half, 32: cuda.hadamard_transform_32_half}[n]
    xd = _dev(x)
    y = fn(xd)
    assert y.data_ptr() == xd.data_ptr()          # in place, returns its argument
    assert np.array_equal(y.cpu().numpy().view(np.uint16), O.fht_f16(x).view(np.uint16))


TOKEN_SHAPES = [(1, 4096), (16, 4096), (5, 4096), (2, 2048), (5, 8192), (3, 16384), (2, 32768), (3, 64), (3, 128), (4, 256), (3, 512),
                (3, 1024), (3, 2048), (4, 11008), (3, 14336), (2, 28672), (3, 3584), (3, 7168), (2, 1536), (2, 768)]


FACTORED = {11008, 14336, 28672, 3584, 7168, 1536, 768}      # K = kfac * 2^m with kfac > 1


@pytest.mark.parametrize("m,k", TOKEN_SHAPES)
def test_token_asym_hadamard_bit_exact(cuda, m, k):
    """Binary32 transform in the reference's order: codes, scales and zero-points equal the oracle's bits.
    (For K = kfac * 2^m this is the sequential factor stage, exact_factor=True.)"""
    x = activations(3000 + k % 977 + m, m, k)
    q, s, z = cuda.quant_token_asym_i4(_dev(x), hadamard=True, exact=True)
    qo, so, zo = O.quant_token_asym(x, True)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)


# 2560 = 40 * 64, 3072 = 12 * 256 and 3584 = 28 * 128 have a factor with two to eight Sylvester bits beside it
TC_SHAPES = TOKEN_SHAPES + [(3, 2560), (300, 2560), (700, 3584), (2000, 4096), (1187, 4096), (4, 3072), (1, 4096), (2, 4096), (3, 4096),
                            (4, 4096), (5, 4096), (6, 4096), (7, 4096), (8, 4096), (64, 11008), (33, 14336), (1, 11008), (7, 11008), (301, 11008), (1001, 11008), (1, 14336), (16, 14336),
                            (256, 14336), (16, 11008), (256, 11008), (256, 4096), (131, 8192), (40, 7168), (9, 3584),
                            # 256 < P <= 512: the two-half form (28672 = 28 * 1024, 20480 = 20 * 1024, 24576 = 12 * 2048, 32768)
                            (1, 28672), (70, 28672), (301, 28672), (130, 32768), (3, 20480), (150, 20480), (3, 24576), (149, 24576)]


@pytest.mark.parametrize("m,k", TC_SHAPES)
def test_token_asym_default_transform_tolerance(cuda, m, k):
    """Default transform (hadamard = 1): the high part of the transform is summed by the tensor cores (or, for widths
    that kernel does not take, the factor by mma.sync), not in the reference's order, so the bound is the stated one,
    taken over ALL codes of ALL rows: at most 0.1 % differ, by one step; scales within one f16 ulp, zero-points
    within one."""
    x = activations(3000 + k % 977 + m, m, k)
    q, s, z = cuda.quant_token_asym_i4(_dev(x), hadamard=True)
    rate = assert_token_tolerance(q, s, z, *O.quant_token_asym(x, True))
    print(f"M={m} K={k}: {rate:.2e} of all codes differ from the oracle by one step")


def test_token_asym_default_transform_is_batch_independent(cuda):
    """A token row gets the same codes whatever batch it arrives in (the default transform takes one kernel, one
    summation order, for every M)."""
    for k in (4096, 3584, 11008, 28672):
        x = activations(4300 + k, 300, k)
        xd = _dev(x)
        qa, sa, za = cuda.quant_token_asym_i4(xd, hadamard=True)
        for rows in (slice(0, 1), slice(7, 23), slice(44, 300)):
            qb, sb, zb = cuda.quant_token_asym_i4(xd[rows].contiguous(), hadamard=True)
            assert torch.equal(qa[rows], qb) and torch.equal(sa[rows], sb) and torch.equal(za[rows], zb)


def test_token_asym_default_transform_bf16_strided(cuda):
    """The default transform on bfloat16 input with a padded row stride and a clip ratio (K = 11008, prefill-size batch,
    and K = 4096 with edge rows): same stated tolerance as the binary16 case."""
    for m, k in ((515, 11008), (300, 4096), (37, 28672)):
        xf = activations(4200 + k, m, k).astype(np.float32)
        xf[5] = 0.0
        xf[6] = np.abs(xf[6])
        xf[7] = -np.abs(xf[7])
        bits = O.f32_to_bf16_bits(xf)
        wide = torch.zeros((m, k + 64), dtype=torch.bfloat16, device="cuda")
        wide[:, :k] = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
        for clip in (1.0, 0.9):
            q, s, z = cuda.quant_token_asym_i4(wide[:, :k], hadamard=True, clip=clip)
            assert_token_tolerance(q, s, z, *O.quant_token_asym(bits, True, clip=clip, bf16=True))


@pytest.mark.parametrize("m,k", [(1, 4096), (7, 11008), (3, 192)])
def test_token_asym_plain_and_clip(cuda, m, k):
    x = activations(3500 + k % 977, m, k)
    for clip in (1.0, 0.9):
        q, s, z = cuda.quant_token_asym_i4(_dev(x), hadamard=False, clip=clip)
        qo, so, zo = O.quant_token_asym(x, False, clip=clip)
        assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
        assert np.array_equal(q.cpu().numpy(), qo)


def test_token_asym_bf16_strided_and_edges(cuda):
    k = 4096
    xf = activations(3600, 6, k).astype(np.float32)
    xf[1] = 0.0                      # all-zero row -> (-1, +1) range
    xf[2] = np.abs(xf[2])            # one-sided row: zero-point 0
    xf[3] = -np.abs(xf[3])           # one-sided negative row: zero-point 15
    bits = O.f32_to_bf16_bits(xf)
    wide = torch.zeros((6, k + 64), dtype=torch.bfloat16, device="cuda")
    wide[:, :k] = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    q, s, z = cuda.quant_token_asym_i4(wide[:, :k], hadamard=True, exact=True)      # row stride k + 64
    qo, so, zo = O.quant_token_asym(bits, True, bf16=True)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("m,k", [(1024, 4096), (1189, 4096), (4100, 4096), (512, 8192), (1777, 8192)])
@pytest.mark.parametrize("bf16", [False, True])
def test_token_asym_k4096_large_batches(cuda, m, k, bf16):
    """K = 4096 / 8192 with many rows run the warp-per-row kernel (one / two warps per row, persistent, next row
    prefetched): every row bit-equal to the oracle, with edge rows, a padded row stride, and a clip ratio that forces
    clamping."""
    xf = activations(3700 + m, m, k).astype(np.float32)
    xf[1] = 0.0
    xf[2] = np.abs(xf[2])
    xf[m - 1] = -np.abs(xf[m - 1])
    xf[m // 2, 7] = 3000.0           # one large outlier
    if bf16:
        bits = O.f32_to_bf16_bits(xf)
        wide = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")
        wide[:, :k] = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
        xin, xo = wide[:, :k], bits
    else:
        xo = xf.astype(np.float16)
        wide = torch.zeros((m, k + 64), dtype=torch.float16, device="cuda")
        wide[:, :k] = torch.from_numpy(xo).cuda()
        xin = wide[:, :k]
    for clip in (1.0, 0.9):
        q, s, z = cuda.quant_token_asym_i4(xin, hadamard=True, clip=clip, exact=True)
        qo, so, zo = O.quant_token_asym(xo, True, clip=clip, bf16=bf16)
        assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
        assert np.array_equal(q.cpu().numpy(), qo)
        assert_token_tolerance(*cuda.quant_token_asym_i4(xin, hadamard=True, clip=clip), qo, so, zo)      # default transform


@pytest.mark.parametrize("m,k", [(600, 4096), (777, 8192)])
@pytest.mark.parametrize("bf16", [False, True])
def test_token_asym_plain_large_batches(cuda, m, k, bf16):
    """Without the transform, K = 4096 / 8192 and many rows also run the warp-per-row kernel."""
    xf = activations(3800 + m, m, k).astype(np.float32)
    xf[3] = 0.0
    if bf16:
        xo = O.f32_to_bf16_bits(xf)
        xin = torch.from_numpy(xo.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        xo = xf.astype(np.float16)
        xin = torch.from_numpy(xo).cuda()
    for clip in (1.0, 0.9):
        q, s, z = cuda.quant_token_asym_i4(xin, hadamard=False, clip=clip)
        qo, so, zo = O.quant_token_asym(xo, False, clip=clip, bf16=bf16)
        assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
        assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("m,k", [(1, 4096), (130, 4096), (1500, 4096), (3, 8192), (700, 8192)])
@pytest.mark.parametrize("had", [False, True])
@pytest.mark.parametrize("bf16", [False, True])
def test_rmsnorm_quant_token_fused(cuda, m, k, had, bf16):
    """RMS-norm fused in front of the token quantiser: bit-equal to the oracle's normalisation (same summation order)
    followed by the oracle's quantiser; and within rounding of torch's own RMS-norm."""
    eps = 1e-5
    xf = (activations(3900 + m + k % 13, m, k).astype(np.float32) * 3.0)
    if m > 2:
        xf[1] = 0.0                                    # all-zero row: c = 1 / sqrt(eps), everything stays 0
    if bf16:
        xo = O.f32_to_bf16_bits(xf)
        xin = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")
        xin[:, :k] = torch.from_numpy(xo.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        xo = xf.astype(np.float16)
        xin = torch.zeros((m, k + 8), dtype=torch.float16, device="cuda")
        xin[:, :k] = torch.from_numpy(xo).cuda()
    q, s, z = cuda.rmsnorm_quant_token_asym_i4(xin[:, :k], eps, hadamard=had)
    yo = O.rmsnorm16(xo, eps, bf16=bf16)
    qo, so, zo = O.quant_token_asym(yo, had, bf16=bf16)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(z.cpu().numpy().view(np.uint16), zo.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)
    # the oracle's normalisation against torch's (another summation order, approximate rsqrt): one 16-bit ulp
    v = xin[:, :k].float()
    yt = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(xin.dtype).float().cpu().numpy()
    yof = O.bf16_bits_to_f32(yo) if bf16 else yo.astype(np.float32)
    ulp = np.maximum(np.abs(yt), 1e-3) * (2.0 ** -7 if bf16 else 2.0 ** -10)
    assert np.all(np.abs(yof - yt) <= ulp)


@pytest.mark.parametrize("m", [1, 33, 1000])
@pytest.mark.parametrize("had", [False, True])
def test_rmsnorm_quant_group_fused(cuda, m, had):
    """RMS-norm fused in front of the group-128 quantiser (rows of 4096): bit-equal to oracle norm + oracle quantiser."""
    x = (activations(4100 + m, m, 4096).astype(np.float32) * 3.0).astype(np.float16)
    if m > 2:
        x[2] = 0.0
    q, s = cuda.rmsnorm_quant_group_sym_i4(_dev(x), 1e-5, hadamard=had)
    yo = O.rmsnorm16(x, 1e-5)
    qo, so = O.quant_group_sym(yo.reshape(-1, 128), had)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), qo)


def test_rmsnorm_quant_rejects_other_widths(cuda):
    x = torch.zeros((4, 2048), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="4096"):
        cuda.rmsnorm_quant_token_asym_i4(x, 1e-5)


def test_token_asym_full_size_property(cuda):
    # the benchmark sweep size M=4096, K=4096: sampled rows against the oracle + a checksum of all codes
    x = activations(88, 4096, 4096)
    q, s, z = cuda.quant_token_asym_i4(_dev(x), hadamard=True, exact=True)
    q, s, z = q.cpu().numpy(), s.cpu().numpy(), z.cpu().numpy()
    idx = rs(10).choice(4096, 64, replace=False)
    qo, so, zo = O.quant_token_asym(x[idx], True)
    assert np.array_equal(q[idx], qo) and np.array_equal(s[idx], so) and np.array_equal(z[idx], zo)
    # dequantised codes stay within half a step of the normalised transform, on the sampled rows
    y = O.had_full_f32(x[idx].astype(np.float32))
    deq = (O.unpack_i4(q[idx], False) - z[idx].astype(np.float32)[:, None]) * s[idx].astype(np.float32)[:, None]
    assert np.all(np.abs(deq - y) <= 0.51 * s[idx].astype(np.float32)[:, None])


def test_argument_errors(cuda):
    x = torch.zeros((4, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        cuda.hadamard_and_quantize_i4(x.float())
    with pytest.raises(RuntimeError):
        cuda.hadamard_and_quantize_i4(x[:, :64])
    with pytest.raises(RuntimeError):
        cuda.hadamard_and_quantize_i4_gs(x, 48)
    with pytest.raises(RuntimeError):
        cuda.hadamard_transform_half(x.cpu())
    with pytest.raises(RuntimeError):
        cuda.quant_token_asym_i4(torch.zeros((2, 96), dtype=torch.float16, device="cuda"))   # K % 64
    q, s = cuda.quant_and_pack_i4(x[:0])            # empty input is fine
    assert q.shape == (0, 64) and s.shape == (0,)
