"""Column/row-parallel W4A4 linears on two GPUs (NCCL) against the single-GPU layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import flh_b200
        from flh_b200.nn import ActQuantizer, LinearFLH
        from flh_b200.tp import ColumnParallelLinearFLH, RowParallelLinearFLH, shard_column, shard_row
        dev = torch.device("cuda", rank)
        g = torch.Generator().manual_seed(11)
        K, N, M = 2048, 1024, 96
        for gs, sym in ((128, True), (-1, False)):
            lin = torch.nn.Linear(K, N, bias=False)
            lin.weight.data = torch.randn(N, K, generator=g) * 0.02
            full = LinearFLH.from_float(lin.half(), weight_group_size=gs, in_group_size=128).to(dev)
            x = torch.randn(M, K, generator=g).half().to(dev)
            aq = ActQuantizer(bits=4, group_size=128 if sym else -1, sym=sym, use_hadamard=False, packed_output=True)
            s, z, q = aq(x)
            y_full = full(q, s, z)
            col = ColumnParallelLinearFLH(shard_column(full, rank, world), gather_output=True)
            y_col = col(q, s, z)
            assert torch.equal(y_col.view(torch.int16), y_full.view(torch.int16)), "column-parallel"
            # row-parallel: every rank quantises its own K-slice of the activations
            kk = K // world
            s2, z2, q2 = aq(x[:, rank * kk:(rank + 1) * kk].contiguous())
            row = RowParallelLinearFLH(shard_row(full, rank, world))
            y_row = row(q2, s2, z2)
            ref = x.float() @ full.get_weight(torch.float32).t()
            err_full = (y_full.float() - ref).abs().max() / ref.abs().max()
            err_row = (y_row.float() - ref).abs().max() / ref.abs().max()
            assert err_row < 2.0 * err_full + 1e-2, (err_row, err_full)    # same quantisation noise level
            if sym:     # group-128 quantisation is unchanged by the K split: only the f16 summation differs
                rel = (y_row.float() - y_full.float()).abs().max() / y_full.float().abs().max()
                assert rel < 2e-3, rel
        # sequence-parallel prefill (residual stream sharded by tokens: reduce-scatter + all-gather of int4 codes) against the
        # all-reduce form, whole decoder, both activation modes: with two ranks both sums are a + b, so the logits are equal
        from flh_b200.model import Decoder, DecoderConfig
        for mode in ("token_asym", "group_sym"):
            cfg = DecoderConfig(hidden=4096, n_heads=32, n_kv_heads=8, ffn=14336, n_layers=2, vocab=1000, act_mode=mode, tp=world)
            model = Decoder(cfg, dev, seed=4)
            for shape in ((2, 96), (2, 2048)):               # 4,096 rows: two blocks of 2,048, block-cyclic ownership
                ids = torch.randint(10, 900, shape, generator=torch.Generator().manual_seed(1)).to(dev)
                cfg.seq_parallel, cfg.sp_blocks = True, 2 if shape[1] == 2048 else 1
                y_sp = model(ids)
                cfg.seq_parallel, cfg.sp_blocks = False, 1
                y_ar = model(ids)
                rel = (y_sp.float() - y_ar.float()).abs().max() / y_ar.float().abs().max()
                assert rel < 1e-3, (mode, shape, float(rel))
            ids = torch.randint(10, 900, (2, 96), generator=torch.Generator().manual_seed(1)).to(dev)
            # a batch whose rows do not divide by the ranks falls back to the all-reduce form
            cfg.seq_parallel = True
            odd = model(ids[:, :95][:1])
            assert odd.shape == (1, 1, 1000)
        # the library's one-launch all-reduce over IPC-mapped buffers: same bits on every rank, equal to the binary32 sum in
        # rank order; eager calls and a CUDA-graph replay (the call number lives on the device); then behind a row-parallel linear
        from flh_b200 import tp
        ar = tp.enable_one_shot(max_bytes=1 << 20)
        gen = torch.Generator().manual_seed(77)
        for n in (8, 8192, 8 * 777, 64 * 8192):
            parts = [torch.randn(n, generator=gen).half() for _ in range(world)]
            ref = parts[0].float()
            for q in parts[1:]:
                ref = ref + q.float()
            y = parts[rank].to(dev)
            assert ar.takes(y)
            tp.all_reduce_sum(y)
            assert torch.equal(y.cpu().view(torch.int16), ref.half().view(torch.int16)), n
        y = torch.full((8192,), float(rank + 1), dtype=torch.float16, device=dev)
        buf = y.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                buf.copy_(y)
                ar.reduce(buf)
            for _ in range(5):
                graph.replay()
        side.synchronize()
        assert torch.all(buf == float(sum(range(1, world + 1))))
        assert ar.status()[0] == 0
        big = torch.ones(2 << 20, dtype=torch.float16, device=dev)           # 4 MiB: over the slot size, goes to NCCL
        assert not ar.takes(big)
        tp.all_reduce_sum(big)
        assert torch.all(big == float(world))
        y_nccl = row(q2, s2, z2)                                             # 96 x 1024 f16: the one-launch form now
        tp.disable_one_shot()
        y_ref = row(q2, s2, z2)
        rel = (y_nccl.float() - y_ref.float()).abs().max() / y_ref.float().abs().max()
        assert rel < 1e-3, rel
        # decode through the decoder: with the one-launch form on, both all-reduces of a layer run fused with the residual add,
        # the RMS-norm and the next quantiser — same logits bit for bit (two ranks: every sum is a + b)
        cfg = DecoderConfig(hidden=4096, n_heads=32, n_kv_heads=8, ffn=14336, n_layers=3, vocab=1000, act_mode="token_asym", tp=world)
        model = Decoder(cfg, dev, seed=4)
        ids = torch.randint(10, 900, (5, 1), generator=torch.Generator().manual_seed(3)).to(dev)
        logits = []
        for fused in (False, True):
            cache = model.new_cache(5, 40)
            for c in cache:
                c[0].copy_(torch.randn(c[0].shape, generator=torch.Generator().manual_seed(8)).half())
                c[1].copy_(torch.randn(c[1].shape, generator=torch.Generator().manual_seed(9)).half())
            if fused:
                tp.enable_one_shot(max_bytes=1 << 20)
            logits.append(model(ids, cache=cache, start=32))
        assert tp._ONE_SHOT[None].status()[0] == 0
        tp.disable_one_shot()
        assert torch.equal(logits[0].view(torch.int16), logits[1].view(torch.int16)), "fused decode"
        if rank == 0:
            open(os.path.join(tmp, "ok"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_tp2_nccl(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()
