"""The library's one-launch all-reduce (include/flh_b200.h: flh_b200_ar_*) with all ranks on ONE GPU: every rank's
buffer lives on the device and the ranks run as one cooperative launch (launches that wait on one another must not
share a GPU).  The two-GPU form over IPC is covered in test_gpu_tp.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Ranks:
    def __init__(self, world, max_bytes):
        from flh_b200 import _lib
        self.lib, self.check, self.world = _lib.load(), _lib.check, world
        self.hs = [ctypes.c_void_p() for _ in range(world)]
        for r in range(world):
            self.check(self.lib.flh_b200_ar_create(world, r, max_bytes, ctypes.byref(self.hs[r])), "ar_create")
        for r in range(world):
            for q in range(world):
                if q != r:
                    self.check(self.lib.flh_b200_ar_attach(self.hs[r], q, self.hs[q]), "ar_attach")

    def run(self, xs, outs):
        n = xs[0].numel()
        arr = (ctypes.c_void_p * self.world)
        self.check(self.lib.flh_b200_allreduce_ranks(arr(*[h.value for h in self.hs]), self.world,
                                                     arr(*[x.data_ptr() for x in xs]), arr(*[o.data_ptr() for o in outs]), n,
                                                     1 if xs[0].dtype == torch.bfloat16 else 0,
                                                     torch.cuda.current_stream().cuda_stream), "allreduce_ranks")

    def status(self):
        out = (ctypes.c_int * 4)()
        res = []
        for h in self.hs:
            self.check(self.lib.flh_b200_ar_status(h, out), "ar_status")
            res.append(list(out))
        return res

    def close(self):
        for h in self.hs:
            self.check(self.lib.flh_b200_ar_destroy(h), "ar_destroy")


def _reference(xs):
    acc = torch.zeros_like(xs[0], dtype=torch.float32)
    for x in xs:                      # rank order, binary32, one rounding at the end
        acc = acc + x.float()
    return acc.to(xs[0].dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_all_ranks_in_one_launch(cuda, world, dtype):
    ranks = _Ranks(world, 1 << 20)
    try:
        g = torch.Generator(device="cuda").manual_seed(100 + world)
        # 8 elements (one 16-byte piece), a decode row, a piece count that does not divide by the CTAs, the full slot
        for call, n in enumerate((8, 8192, 8 * 12345, 64 * 8192, 8, 8192, 64 * 8192)):
            xs = [torch.randn(n, device="cuda", generator=g).to(dtype) for _ in range(world)]
            ref = _reference(xs)
            if call % 2 == 0:
                outs = [torch.empty_like(x) for x in xs]
            else:
                outs = xs                                  # in place
            ranks.run(xs, outs)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(outs[r].view(torch.int16), ref.view(torch.int16)), (world, n, r)
        assert all(s[0] == 0 for s in ranks.status())
    finally:
        ranks.close()


def test_rejects_what_it_cannot_take(cuda):
    from flh_b200 import _lib
    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.flh_b200_ar_create(9, 0, 1 << 20, ctypes.byref(h)) != 0          # more than 8 ranks
    assert lib.flh_b200_ar_create(2, 0, 100, ctypes.byref(h)) != 0              # slot size not a multiple of 16
    _lib.check(lib.flh_b200_ar_create(2, 0, 4096, ctypes.byref(h)), "ar_create")
    try:
        x = torch.zeros(4096, dtype=torch.float16, device="cuda")
        s = torch.cuda.current_stream().cuda_stream
        assert lib.flh_b200_allreduce(h, x.data_ptr(), x.data_ptr(), 2048, 0, s) != 0     # rank 1 not attached
        assert b"not attached" in lib.flh_b200_last_error()
        assert lib.flh_b200_allreduce(h, x.data_ptr(), x.data_ptr(), 4096, 0, s) != 0     # 8 KiB message, 4 KiB slots
        assert lib.flh_b200_allreduce(h, x.data_ptr(), x.data_ptr(), 12, 0, s) != 0       # not whole 16-byte pieces
    finally:
        _lib.check(lib.flh_b200_ar_destroy(h), "ar_destroy")


def test_wait_runs_out_when_a_peer_never_arrives(cuda):
    """Rank 0 of two launches alone; rank 1's buffer is mapped but rank 1 never calls.  The wait for its flag ends after
    its time limit: the launch completes, the status words name the peer, and the device stays usable."""
    ranks = _Ranks(2, 4096)
    try:
        x = torch.ones(2048, dtype=torch.float16, device="cuda")
        ranks.check(ranks.lib.flh_b200_allreduce(ranks.hs[0], x.data_ptr(), x.data_ptr(), 2048, 0,
                                                 torch.cuda.current_stream().cuda_stream), "allreduce")
        torch.cuda.synchronize()
        st = ranks.status()
        assert st[0][0] == 1 and st[0][1] == 1 and st[0][3] == 1, st      # a wait ran out, for rank 1, in call 1
        assert st[1][0] == 0
        assert float((x + 1).sum().item()) >= 0.0                          # the context still runs kernels
    finally:
        ranks.close()


@pytest.mark.parametrize("world,M,K", [(2, 64, 8192), (4, 32, 8192), (8, 16, 8192), (8, 1, 8192), (2, 5, 4096), (8, 18, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_add_norm_quant_equals_the_three_steps(cuda, world, M, K, dtype):
    """All-reduce + residual add + RMS-norm + per-token quantiser as one launch against all-reduce (binary32 sum in rank
    order, rounded once), a 16-bit add and flh_b200_rmsnorm_quant_token_asym_i4: residual stream, codes, scales and
    zero-points bit for bit, on every rank; two calls in a row (the second sees the first's residual)."""
    ranks = _Ranks(world, 1 << 20)
    try:
        g = torch.Generator(device="cuda").manual_seed(7 * world + M)
        arr = ctypes.c_void_p * world
        res = [(torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dtype)] * world
        res = [r.clone() for r in res]                       # the residual stream is replicated
        for call in range(2):
            ys = [(torch.randn(M, K, device="cuda", generator=g) * (0.3 + 0.1 * r)).to(dtype) for r in range(world)]
            if call == 1:
                ys[0][0].zero_()                             # a row whose partial outputs vanish on one rank
            want_res = (res[0].float() + _reference(ys).float()).to(dtype)
            want_q, want_s, want_z = cuda.rmsnorm_quant_token_asym_i4(want_res, 1e-5, hadamard=False)
            qs = [torch.empty(M, K // 2, dtype=torch.uint8, device="cuda") for _ in range(world)]
            ss = [torch.empty(M, dtype=torch.float16, device="cuda") for _ in range(world)]
            zs = [torch.empty(M, dtype=torch.float16, device="cuda") for _ in range(world)]
            ranks.check(ranks.lib.flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4_ranks(
                arr(*[h.value for h in ranks.hs]), world, arr(*[y.data_ptr() for y in ys]), arr(*[r.data_ptr() for r in res]),
                M, K, 1 if dtype == torch.bfloat16 else 0, 1e-5, 1.0, arr(*[q.data_ptr() for q in qs]),
                arr(*[s.data_ptr() for s in ss]), arr(*[z.data_ptr() for z in zs]), torch.cuda.current_stream().cuda_stream),
                "fused all-reduce")
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(res[r].view(torch.int16), want_res.view(torch.int16)), (call, r, "residual")
                assert torch.equal(ss[r].view(torch.int16), want_s.view(torch.int16)), (call, r, "scale")
                assert torch.equal(zs[r].view(torch.int16), want_z.view(torch.int16)), (call, r, "zero")
                assert torch.equal(qs[r], want_q), (call, r, "codes")
        assert all(s[0] == 0 for s in ranks.status())
    finally:
        ranks.close()
