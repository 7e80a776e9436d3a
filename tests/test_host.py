"""CPU-side checks: the C ABI library loads and exports what include/flh_b200.h declares, argument
validation that needs no device, and the offline (host) weight path against the reference's buffers."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from flh_b200 import _lib
    lib = _lib.load()
    hdr = open(os.path.join(ROOT, "include", "flh_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(flh_b200_\w+|flhDenseLayerGEMM_i4_o16)\s*\(", hdr))
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), n
    assert names == set(_lib.SIGNATURES), names ^ set(_lib.SIGNATURES)
    assert lib.flh_b200_version() >= 100


def test_argument_validation_without_a_device():
    from flh_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(16)
    assert lib.flh_b200_quant_group_sym_i4(one, 4, 48, 1, one, one, None) == 1          # bad group size
    assert b"32, 64 or 128" in lib.flh_b200_last_error()
    assert lib.flh_b200_quant_group_sym_i4(ctypes.c_void_p(8), 4, 128, 1, one, one, None) == 2   # misaligned
    assert lib.flh_b200_hadamard_f16_inplace(one, 4, 100, None) == 1
    assert lib.flh_b200_quant_token_asym_i4(one, 0, 4, 100, 100, 1, 1, None, 1.0, one, one, one, None) == 1
    assert lib.flh_b200_quant_token_asym_i4(one, 0, 4, 11008, 11008, 1, 172, None, 1.0, one, one, one, None) == 1  # no sign bits
    assert lib.flh_b200_quant_token_asym_i4(one, 0, 4, 4096, 4100, 1, 1, None, 1.0, one, one, one, None) == 2      # stride
    assert lib.flh_b200_gemm_i4_dequant(one, one, one, None, one, None, None, one, 4, 100, 256, 128, 128, 0, 0, None, 0, None) == 1
    assert lib.flh_b200_gemm_i4_dequant(one, one, one, one, one, None, None, one, 4, 128, 256, 128, 128, 0, 0, None, 0, None) == 1
    assert b"b_rowsum" in lib.flh_b200_last_error()
    assert lib.flh_b200_gemm_i4_dequant(one, one, one, None, one, None, None, one, 65, 128, 256, 128, 128, 0, 3, None, 0, None) == 1
    # empty problems succeed without touching the device
    assert lib.flh_b200_quant_group_sym_i4(None, 0, 128, 1, None, None, None) == 0
    assert lib.flh_b200_gemm_i4_dequant(None, None, None, None, None, None, None, None, 0, 128, 256, 128, 128, 0, 0, None, 0, None) == 0
    assert lib.flh_b200_gemm_pick_algo(16, 22016, 4096, 128, 128) == 3      # enough row slabs: plain streaming
    assert lib.flh_b200_gemm_pick_algo(16, 4096, 4096, 128, 128) == 4       # few slabs: split-K
    assert lib.flh_b200_gemm_workspace_bytes(16, 4096, 4096, 128, 128, 0) == 4096 + 4 * 16 * 4096 * 4
    assert lib.flh_b200_gemm_workspace_bytes(2048, 4096, 4096, 128, 128, 0) == 0
    assert lib.flh_b200_gemm_pick_algo(2048, 4096, 4096, 128, 128) == 1


def test_pack_signs_host_helper():
    from flh_b200 import _lib
    from flh_b200.hadamard import get_hadK
    s, k = get_hadK(11008)
    assert k == 172
    words = (k + 31) // 32
    lib = _lib.load()
    nbytes = lib.flh_b200_sign_table_bytes(k)        # bit rows, then the bf16 matrix padded to a multiple of 16
    kp = (k + 15) // 16 * 16
    bits_bytes = (k * words * 4 + 15) // 16 * 16
    assert nbytes == bits_bytes + kp * kp * 2
    buf = np.zeros(nbytes // 4, dtype=np.uint32)
    assert lib.flh_b200_pack_signs(np.ascontiguousarray(s).ctypes.data_as(ctypes.c_void_p), k,
                                   buf.ctypes.data_as(ctypes.c_void_p)) == 0
    out = buf[:k * words].reshape(k, words)
    bits = ((out[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(k, -1)[:, :k]
    assert np.array_equal(bits == 1, s < 0)
    mat = buf.view(np.uint16)[bits_bytes // 2:].reshape(kp, kp)
    assert np.array_equal(mat[:k, :k], np.where(s < 0, 0xBF80, 0x3F80).astype(np.uint16))
    assert not mat[k:].any() and not mat[:, k:].any()


def test_get_hadK_precedence():
    from flh_b200.hadamard import get_hadK
    for n, k in ((4096, 1), (8192, 1), (11008, 172), (14336, 28), (28672, 28), (3584, 28), (1536, 12), (5120, 40), (6656, 52)):
        assert get_hadK(n)[1] == k
    with pytest.raises(AssertionError):
        get_hadK(4096 + 2)


def test_from_float_matches_reference_buffers(golden):
    from helpers import rs
    from flh_b200.nn import LinearFLH
    w = (rs(401).standard_normal((64, 256)) * 0.02).astype(np.float32)
    lin = torch.nn.Linear(256, 64, bias=False)
    lin.weight.data = torch.from_numpy(w)
    fl = LinearFLH.from_float(lin, weight_bits=4, weight_group_size=128, weight_sym=True, in_group_size=128)
    assert np.array_equal(fl.w_packed.numpy().reshape(64, 128), golden["lin_w_packed"])
    assert np.array_equal(fl.w_scale.numpy(), golden["lin_w_scale"])
    assert fl.w_zero.dtype == torch.uint8 and int(fl.w_zero.max()) == 0
    # the PyTorch twin reproduces the reference twin's output
    y = fl.forward_torch(torch.from_numpy(golden["lin_x_packed"]),
                         a_scale=torch.from_numpy(rs_scales()), a_zero=None)
    assert np.abs(y.numpy() - golden["lin_fwd_torch"]).max() <= 1e-5 * np.abs(golden["lin_fwd_torch"]).max()


def rs_scales():
    from helpers import rs
    r = rs(401)
    r.standard_normal((64, 256))
    r.randint(-8, 8, size=(5, 256))
    return r.uniform(0.005, 0.02, size=(5, 2)).astype(np.float16)


def test_weight_quantizer_channel_wise_matches_fake_quant(golden):
    # weights of the CPU-runnable benchmark configuration: W ~ N(0, 0.02) rotated by the 4096-point transform, per-channel symmetric RTN
    from flh_b200.nn import WeightQuantizer
    from flh_b200.hadamard import matmul_hadU
    torch.manual_seed(0)
    torch.randn(16, 4096); torch.randperm(4096)
    W = torch.randn(4096, 4096) * 0.02
    Wr = matmul_hadU(W.double()).float()
    wq = WeightQuantizer(bits=4, group_size=-1, sym=True, channel_wise=True, use_hadamard=False)
    scale, _, _ = wq(Wr)
    ref = golden["cfg1_w_scale"]
    assert np.abs(scale[:, 0].numpy() - ref).max() <= 2e-6 * np.abs(ref).max()


def test_pack_unpack_roundtrip():
    from flh_b200.functional import pack_i4, unpack_i4
    q = torch.randint(-8, 8, (5, 64), dtype=torch.int32)
    p = pack_i4(q)
    assert p.dtype == torch.uint8 and p.shape == (5, 32)
    assert torch.equal(unpack_i4(p), q)
    assert int(p[0, 0]) == (int(q[0, 0]) & 15) | ((int(q[0, 1]) & 15) << 4)


def test_oracle_rmsnorm_matches_torch():
    """The oracle's RMS-norm (fixed summation order, correctly rounded 1 / sqrt) against torch's on the CPU:
    at most one unit in the last place of the 16-bit result."""
    import torch
    from helpers import activations
    from oracle import oracle as O
    for k in (4096, 8192):
        x = (activations(77 + k, 9, k).astype(np.float32) * 2.5).astype(np.float16)
        y = O.rmsnorm16(x, 1e-5).astype(np.float32)
        v = torch.from_numpy(x).float()
        yt = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).half().float().numpy()
        assert np.all(np.abs(y - yt) <= np.maximum(np.abs(yt), 1e-3) * 2.0 ** -10)
        assert (y != yt).mean() < 1e-2
