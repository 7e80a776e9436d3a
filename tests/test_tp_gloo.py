"""Tensor-parallel sharding and the row-parallel all-reduce on CPU: two gloo ranks, with the GEMM
served by the CPU oracle in place of the CUDA library (the sharding, the scale/zero bookkeeping and
the collective are what is under test)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_backend():
    """Stand-ins for flh_b200._CUDA entry points, computing with the CPU oracle on CPU tensors."""
    from oracle import oracle as O

    def gemm(A, B, A_scale, B_scale, A_zero=None, B_rowsum=None, bias=None, out_dtype=torch.float16, algo=0, out=None):
        d = O.gemm_i4_dequant(A.numpy(), B.numpy(), A_scale.numpy(), B_scale.numpy(),
                              a_zero=None if A_zero is None else A_zero.numpy(),
                              bias=None if bias is None else bias.numpy())
        d = torch.from_numpy(d.copy())
        if out is not None:
            out.copy_(d)
            return out
        return d

    def rowsum(B, group):
        return torch.from_numpy(O.weight_rowsum(B.numpy(), group))

    return gemm, rowsum


def args_full_rows(x, asym, O):
    """(codes, scales, zero-points) of all rows of x, full width, as the linears take them."""
    M, K = x.shape
    if asym:
        q, s, z = O.quant_token_asym(x, False)
        return torch.from_numpy(q), torch.from_numpy(s).view(M, 1), torch.from_numpy(z).view(M, 1)
    q, s = O.quant_group_sym(x.reshape(-1, 128), False)
    return torch.from_numpy(q.reshape(M, K // 2)), torch.from_numpy(s.reshape(M, K // 128)), None


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import flh_b200
        from flh_b200.nn import LinearFLH
        from flh_b200.tp import ColumnParallelLinearFLH, RowParallelLinearFLH, shard_column, shard_row
        from oracle import oracle as O
        gemm, rowsum = _oracle_backend()
        flh_b200._CUDA.gemm_i4_dequant = gemm
        flh_b200._CUDA.weight_rowsum = rowsum

        g = torch.Generator().manual_seed(7)                 # same weights on every rank
        K, N, M = 512, 256, 5
        for gs, asym in ((128, False), (-1, True)):
            lin = torch.nn.Linear(K, N, bias=True)
            lin.weight.data = torch.randn(N, K, generator=g) * 0.02
            lin.bias.data = torch.randn(N, generator=g) * 0.1
            full = LinearFLH.from_float(lin.half(), weight_group_size=gs, in_group_size=128)
            x = torch.randn(M, K, generator=g).half().numpy()
            if asym:
                q, s, z = O.quant_token_asym(x, False)
                qs = [O.quant_token_asym(np.ascontiguousarray(x[:, r * K // world:(r + 1) * K // world]), False) for r in range(world)]
                args_full = (torch.from_numpy(q), torch.from_numpy(s).view(M, 1), torch.from_numpy(z).view(M, 1))
                args_mine = tuple(torch.from_numpy(a).view(M, -1) for a in qs[rank])
            else:
                q, s = O.quant_group_sym(x.reshape(-1, 128), False)
                q, s = q.reshape(M, K // 2), s.reshape(M, K // 128)
                kk = K // world
                args_full = (torch.from_numpy(q), torch.from_numpy(s), None)
                args_mine = (torch.from_numpy(q[:, rank * kk // 2:(rank + 1) * kk // 2].copy()),
                             torch.from_numpy(s[:, rank * kk // 128:(rank + 1) * kk // 128].copy()), None)
            y_full = full(*args_full)

            # column-parallel: the gathered shards are the full output, bit for bit
            col = ColumnParallelLinearFLH(shard_column(full, rank, world), gather_output=True)
            y_col = col(*args_full)
            assert torch.equal(y_col.view(torch.int16), y_full.view(torch.int16)), "column-parallel"

            # row-parallel: all-reduced f16 partials == the f16 sum of the two partials, and close to
            # the single-device result
            row = RowParallelLinearFLH(shard_row(full, rank, world))
            part = row.shard(*args_mine)
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            y_row = row(*args_mine)
            want = (parts[0].float() + parts[1].float()).half()
            assert torch.equal(y_row.view(torch.int16), want.view(torch.int16)), "row-parallel sum"
            if not asym:    # same quantised activations as the full layer: only the summation order differs
                err = (y_row.float() - y_full.float()).abs().max() / y_full.float().abs().max()
                assert err < 2e-3, f"row-parallel vs single device: {err}"
            # sequence-parallel form: the reduce-scatter hands rank r the summed rows of its token slice — the same bits as
            # the all-reduced rows — and the all-gather of per-rank quantised rows rebuilds the full quantised batch
            M2 = 8                                           # rows divisible by ranks x blocks
            x2 = torch.randn(M2, K, generator=g).half().numpy()
            kk = K // world
            if asym:
                a2 = tuple(torch.from_numpy(a).view(M2, -1) for a in O.quant_token_asym(np.ascontiguousarray(x2[:, rank * kk:(rank + 1) * kk]), False))
            else:
                q2, s2 = O.quant_group_sym(np.ascontiguousarray(x2[:, rank * kk:(rank + 1) * kk]).reshape(-1, 128), False)
                a2 = (torch.from_numpy(q2.reshape(M2, kk // 2)), torch.from_numpy(s2.reshape(M2, kk // 128)), None)
            y_all = row(*a2)
            from flh_b200.tp import gather_quantised, gather_rows, local_rows
            whole_rows = args_full_rows(x2, asym, O)
            for blocks in (1, 2):                            # M2 = 8 rows: 4 or 2 x 2 per rank
                y_mine = row.forward_scatter(*a2, blocks=blocks)
                assert torch.equal(y_mine.view(torch.int16), local_rows(y_all, rank, world, blocks).contiguous().view(torch.int16)), "reduce-scatter"
                assert torch.equal(gather_rows(y_mine, None, blocks).view(torch.int16), y_all.view(torch.int16)), "gather of local rows"
                mine = tuple(None if a is None else local_rows(a, rank, world, blocks).contiguous() for a in whole_rows)
                got = gather_quantised(*mine, blocks=blocks)
                for a, b in zip(got, whole_rows):
                    assert (a is None and b is None) or torch.equal(a, b), "all-gather of quantised rows"
        # row-parallel with the online full-width transform (the down_proj of the per-token mode): every rank rotates
        # its own K / tp activations, so the weight is rotated per block of K / tp = 3584 = 28 * 128; the summed output
        # must approximate the float layer x @ W^T as well as the single-device layer does
        K, N, M = 7168, 128, 4
        lin = torch.nn.Linear(K, N, bias=False)
        lin.weight.data = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(M, K, generator=g).half()
        ref = x.float() @ lin.weight.data.half().float().t()
        whole = LinearFLH.from_float(lin.half(), weight_group_size=-1, full_hadamard=True)
        with pytest.raises(ValueError):
            shard_row(whole, rank, world)                    # rotated over K as a whole: not splittable
        q, s, z = O.quant_token_asym(x.numpy(), True)
        y_whole = whole(torch.from_numpy(q), torch.from_numpy(s).view(M, 1), torch.from_numpy(z).view(M, 1))
        blocked = LinearFLH.from_float(lin.half(), weight_group_size=-1, full_hadamard=True, hadamard_blocks=world)
        kk = K // world
        qm, sm, zm = O.quant_token_asym(np.ascontiguousarray(x.numpy()[:, rank * kk:(rank + 1) * kk]), True)
        row = RowParallelLinearFLH(shard_row(blocked, rank, world))
        y_row = row(torch.from_numpy(qm), torch.from_numpy(sm).view(M, 1), torch.from_numpy(zm).view(M, 1))
        # W4A4 quantisation noise, as a relative Frobenius error; a shard rotated the wrong way is uncorrelated (~1.4)
        err_whole = (y_whole.float() - ref).norm() / ref.norm()
        err_row = (y_row.float() - ref).norm() / ref.norm()
        assert err_whole < 0.3 and err_row < 1.5 * err_whole + 0.02, (err_row, err_whole)
        # without tp.enable_one_shot() (no CUDA device here) the row-parallel layer stays on the process group's all-reduce:
        # the fused decode form declines before running anything, all_reduce_sum is the group's sum
        from flh_b200 import tp
        assert tp._ONE_SHOT == {}
        res = torch.zeros(M, N).half()
        assert row.forward_add_norm_quant(torch.from_numpy(qm), torch.from_numpy(sm).view(M, 1), torch.from_numpy(zm).view(M, 1), res, 1e-5) is None
        assert float(res.abs().max()) == 0.0
        t = torch.full((16,), float(rank + 1))
        tp.all_reduce_sum(t)
        assert torch.all(t == float(sum(range(1, world + 1))))
        if rank == 0:
            open(os.path.join(tmp, "ok"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()
