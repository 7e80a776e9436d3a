"""The kernels either side of the quantised linears in the decoder wiring (flh/quantized_model/modeling_llama.py:389-470,
522-526): SiLU(gate) * up (alone, and fused with the transform and the quantiser), rotary embedding + KV-cache write."""
import numpy as np
import pytest
import torch

from helpers import assert_token_tolerance, rs
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _gate_up(seed, m, f, bf16=False):
    g = rs(seed)
    gu = (g.standard_normal((m, 2 * f)) * 2.5).astype(np.float32)
    gu[:, 5] *= 8.0
    if m > 3:
        gu[1] = 0.0
        gu[2, :f] = -30.0            # SiLU underflows to -0
        gu[3, :f] = 40.0             # SiLU(g) = g
    return O.f32_to_bf16_bits(gu) if bf16 else gu.astype(np.float16)


@pytest.mark.parametrize("m,f", [(1, 64), (7, 11008), (130, 4096), (33, 3584)])
@pytest.mark.parametrize("bf16", [False, True])
def test_silu_mul_bit_exact(cuda, m, f, bf16):
    gu = _gate_up(50 + m, m, f, bf16)
    wide = torch.zeros((m, 2 * f + 8), dtype=torch.bfloat16 if bf16 else torch.float16, device="cuda")
    wide[:, :2 * f] = torch.from_numpy(gu.view(np.int16)).cuda().view(wide.dtype)
    out = cuda.silu_mul(wide[:, :2 * f])                                   # padded row stride
    want = O.silu_mul16(gu, bf16=bf16)
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want.view(np.uint16))
    # against torch's own silu(gate) * up (its expf may differ in the last bit): one 16-bit ulp
    x = wide[:, :2 * f]
    ref = (torch.nn.functional.silu(x[:, :f]) * x[:, f:]).float().cpu().numpy()
    got = out.float().cpu().numpy()
    assert np.all(np.abs(got - ref) <= np.maximum(np.abs(ref), 1e-4) * (2.0 ** -7 if bf16 else 2.0 ** -10))


@pytest.mark.parametrize("m,f", [(1, 11008), (9, 11008), (300, 11008), (2100, 11008), (260, 4096), (70, 14336), (40, 7168), (5, 3584), (3, 28672)])
def test_silu_mul_quant_fused_equals_the_two_steps(cuda, m, f):
    """One kernel (SiLU * up made in shared memory, transform, quantiser) against the separate kernels, bit for bit; and
    against the oracle chain within the stated tolerance of the default transform.  F = 28672 is wider than the fused
    kernel takes: the entry point then runs the two steps itself."""
    gu = _gate_up(70 + m, m, f)
    gud = torch.from_numpy(gu).cuda()
    q, s, z = cuda.silu_mul_quant_token_asym_i4(gud, hadamard=True, fused=True)
    a = cuda.silu_mul(gud)
    q2, s2, z2 = cuda.quant_token_asym_i4(a, hadamard=True)
    assert torch.equal(q, q2) and torch.equal(s, s2) and torch.equal(z, z2)
    if m <= 300:
        assert_token_tolerance(q, s, z, *O.quant_token_asym(O.silu_mul16(gu), True))
    torch.cuda.synchronize()
    assert cuda.gemm_status()[0] == 0


def test_silu_mul_quant_bf16_and_clip(cuda):
    m, f = 150, 11008
    gu = _gate_up(91, m, f, bf16=True)
    wide = torch.zeros((m, 2 * f + 64), dtype=torch.bfloat16, device="cuda")
    wide[:, :2 * f] = torch.from_numpy(gu.view(np.int16)).cuda().view(torch.bfloat16)
    q, s, z = cuda.silu_mul_quant_token_asym_i4(wide[:, :2 * f], hadamard=True, clip=0.9, fused=True)
    q2, s2, z2 = cuda.quant_token_asym_i4(cuda.silu_mul(wide[:, :2 * f]), hadamard=True, clip=0.9)
    assert torch.equal(q, q2) and torch.equal(s, s2) and torch.equal(z, z2)
    assert_token_tolerance(q, s, z, *O.quant_token_asym(O.silu_mul16(gu, bf16=True), True, clip=0.9, bf16=True))


@pytest.mark.parametrize("B,S,nh,nkv,cur,T", [(2, 40, 4, 2, 0, 40), (3, 1, 8, 8, 37, 64), (1, 17, 32, 8, 5, 30), (2, 128, 4, 1, 0, 200)])
def test_rope_kv_equals_the_tensor_operations(cuda, B, S, nh, nkv, cur, T):
    from flh_b200.model import rope, rope_tables
    D = 128
    g = torch.Generator(device="cuda").manual_seed(7)
    qkv = torch.randn(B * S, (nh + 2 * nkv) * D, device="cuda", generator=g).half()
    pos = torch.arange(cur, cur + S, device="cuda")
    cos, sin = rope_tables(pos, D, 10000.0)
    kc = torch.randn(B, nkv, T, D, device="cuda", generator=g).half()
    vc = torch.randn(B, nkv, T, D, device="cuda", generator=g).half()
    kc0, vc0 = kc.clone(), vc.clone()
    qh = torch.empty(B, nh, S, D, dtype=torch.float16, device="cuda")
    cuda.rope_kv(qkv, cos, sin, qh, kc, vc, B, S, nh, nkv, cur)
    q_, k_, v_ = qkv.view(B, S, -1).split((nh * D, nkv * D, nkv * D), dim=-1)
    want_q = rope(q_.view(B, S, nh, D), pos, 10000.0).transpose(1, 2)
    want_k = rope(k_.view(B, S, nkv, D), pos, 10000.0).transpose(1, 2)
    assert torch.equal(qh, want_q)
    assert torch.equal(kc[:, :, cur:cur + S], want_k) and torch.equal(vc[:, :, cur:cur + S], v_.view(B, S, nkv, D).transpose(1, 2))
    # nothing outside the step's positions is touched
    keep = torch.ones(T, dtype=torch.bool, device="cuda")
    keep[cur:cur + S] = False
    assert torch.equal(kc[:, :, keep], kc0[:, :, keep]) and torch.equal(vc[:, :, keep], vc0[:, :, keep])
