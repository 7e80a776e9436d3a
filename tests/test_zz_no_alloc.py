"""The decode GEMM entry point that allocates nothing (flh_b200_gemm_i4_dequant_decode_noalloc).

Some callers cannot hand the library a workspace: a serving loop pinned to a fixed memory budget, a host
application that owns every allocation, code between two CUDA-graph launches.  For them the split-K
scratch sits in an array inside the library.  This test drives the entry point through the C ABI and
checks it, twice in a row (the second call meets the first call's leftovers in the shared array),
against the ordinary entry point run with a caller-allocated workspace: same kernel, same split order,
so the outputs must be the same bits.  It is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from test_gpu_gemm import SPLITK, make_case, _dev

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("mode", [(128, 128, False), (0, 0, True), (0, 128, True)])
def test_decode_noalloc_matches_workspace_entry(cuda, mode):
    from flh_b200 import _lib
    lib = _lib.load()
    m, n, k = 16, 4096, 4096
    ap, bp, sa, sb, za, bi = make_case(321, m, n, k, *mode, bias=True)
    A, B, SA, SB, BI = _dev(ap), _dev(bp), _dev(sa), _dev(sb), _dev(bi)
    ZA = None if za is None else _dev(za)
    ag, bg = k // sa.shape[1], k // sb.shape[1]
    RS = cuda.weight_rowsum(B, min(ag, bg)) if za is not None else None
    stream = torch.cuda.current_stream().cuda_stream

    # the existing entry point, split-K with a caller workspace
    assert lib.flh_b200_gemm_pick_algo(m, n, k, ag, bg) == SPLITK
    need = lib.flh_b200_gemm_workspace_bytes(m, n, k, ag, bg, SPLITK)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    want = torch.empty((m, n), dtype=torch.float16, device="cuda")
    _lib.check(lib.flh_b200_gemm_i4_dequant(_ptr(A), _ptr(B), _ptr(SA), _ptr(ZA), _ptr(SB), _ptr(RS), _ptr(BI), _ptr(want),
                                            m, n, k, ag, bg, 0, SPLITK, _ptr(ws), need, stream), "workspace entry")

    # the entry point under test: no workspace argument at all, two calls back to back
    for attempt in range(2):
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(lib.flh_b200_gemm_i4_dequant_decode_noalloc(_ptr(A), _ptr(B), _ptr(SA), _ptr(ZA), _ptr(SB), _ptr(RS), _ptr(BI),
                                                               _ptr(got), m, n, k, ag, bg, 0, stream), "no-alloc entry")
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20), "device memory was allocated"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {attempt + 1} differs"


def test_decode_noalloc_rejects_what_does_not_fit(cuda):
    from flh_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(256)
    # M = 32, N = 9216: two splits x 32 token rows x 9216 columns x 4 B > the 2 MiB inside the library
    rc = lib.flh_b200_gemm_i4_dequant_decode_noalloc(one, one, one, None, one, None, None, one, 32, 9216, 4096, 128, 128, 0, None)
    assert rc == 1
    msg = lib.flh_b200_last_error().decode()
    assert "scratch" in msg and "caller workspace" in msg
    # prefill-sized M is not this entry point's business
    assert lib.flh_b200_gemm_i4_dequant_decode_noalloc(one, one, one, None, one, None, None, one, 65, 4096, 4096, 128, 128, 0, None) == 1
