"""Megatron-style tensor parallelism for packed W4A4 linears (one process per GPU).

The reference has no multi-GPU code; the sharding follows its checkpoint layout (LinearFLH buffers,
flh/nn/linear.py:20-30) so that a shard is a slice of the single-GPU tensors:

  column-parallel (q/k/v, gate/up)  rows  [r N/tp, (r+1) N/tp) of w_packed [N, K/2] and w_scale;
                                    replicated activations, no collective;
  row-parallel (o_proj, down_proj)  columns [r K/tp, (r+1) K/tp) of every row (K/tp a multiple of 128);
                                    each rank quantises ITS slice of the activations (per-(token, shard)
                                    scale / zero-point; a full-width Hadamard becomes block-diagonal per
                                    shard), runs the GEMM and the f16 partial outputs are summed with one
                                    all-reduce — the only collective of the path.

The all-reduce is NCCL's, except for the small messages of decode once `enable_one_shot()` was called: those go
through the library's own one-launch all-reduce over peer-mapped buffers (include/flh_b200.h: flh_b200_allreduce).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

import ctypes

from . import _lib, timing
from .nn import LinearFLH


class OneShotAllReduce:
    """The library's one-launch all-reduce (include/flh_b200.h: flh_b200_ar_*) for one process group: each rank
    allocates its buffer, the 64-byte IPC handles travel through the group's object all-gather, every rank maps the
    others.  `reduce(y)` sums y (f16 / bf16, contiguous, numel a multiple of 8, at most max_bytes) in place on the
    current stream; every rank gets the same bits (slots are summed in rank order in binary32)."""

    def __init__(self, group=None, max_bytes: int = 2 << 20, device=None):
        self.group, self.max_bytes = group, int(max_bytes)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        lib = _lib.load()
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.flh_b200_ar_create(self.world, self.rank, self.max_bytes, ctypes.byref(self._h)), "ar_create")
            mine = ctypes.create_string_buffer(64)
            _lib.check(lib.flh_b200_ar_export(self._h, mine), "ar_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(mine.raw), group=group)
            for r, hb in enumerate(handles):
                if r != self.rank:
                    _lib.check(lib.flh_b200_ar_import(self._h, r, ctypes.create_string_buffer(hb, 64)), "ar_import")
        dist.barrier(group=group)          # nobody launches before everybody has mapped everybody

    def takes(self, y) -> bool:
        return (y.is_cuda and y.dtype in (torch.float16, torch.bfloat16) and y.is_contiguous() and y.numel() % 8 == 0
                and 0 < y.numel() * 2 <= self.max_bytes and y.data_ptr() % 16 == 0)

    def reduce(self, y):
        _lib.check(_lib.load().flh_b200_allreduce(self._h, y.data_ptr(), y.data_ptr(), y.numel(),
                                                  1 if y.dtype == torch.bfloat16 else 0,
                                                  torch.cuda.current_stream(y.device).cuda_stream), "allreduce")
        return y

    def takes_fused(self, y, residual) -> bool:
        """The fused form: y, residual [M, K] f16 / bf16 contiguous, K = 4096 or 8192, at most 128 rows."""
        K = y.shape[-1]
        return (self.takes(y) and residual.shape == y.shape and residual.dtype == y.dtype and residual.is_contiguous()
                and residual.data_ptr() % 16 == 0 and K in (4096, 8192) and y.numel() // K <= 128)

    def reduce_add_norm_quant(self, y, residual, eps: float, clip: float = 1.0):
        """residual += all-reduce(y) (in place), then RMS-norm (weight 1) + per-token asymmetric int4 of the new residual:
        -> (q u8[M, K/2], scale f16[M], zero f16[M]).  One launch (include/flh_b200.h:
        flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4)."""
        K = y.shape[-1]
        M = y.numel() // K
        q = torch.empty((M, K // 2), dtype=torch.uint8, device=y.device)
        s = torch.empty((M,), dtype=torch.float16, device=y.device)
        z = torch.empty((M,), dtype=torch.float16, device=y.device)
        _lib.check(_lib.load().flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4(
            self._h, y.data_ptr(), residual.data_ptr(), M, K, 1 if y.dtype == torch.bfloat16 else 0, float(eps), float(clip),
            q.data_ptr(), s.data_ptr(), z.data_ptr(), torch.cuda.current_stream(y.device).cuda_stream), "allreduce_add_rmsnorm_quant")
        return q, s, z

    def status(self):
        out = (ctypes.c_int * 4)()
        _lib.check(_lib.load().flh_b200_ar_status(self._h, out), "ar_status")
        return list(out)

    def close(self):
        if self._h:
            dist.barrier(group=self.group)  # no peer still reads or writes this buffer
            _lib.check(_lib.load().flh_b200_ar_destroy(self._h), "ar_destroy")
            self._h = ctypes.c_void_p()


_ONE_SHOT = {}       # process group -> OneShotAllReduce


def enable_one_shot(group=None, max_bytes: int = 2 << 20):
    """From now on row-parallel linears of `group` sum messages of up to max_bytes with the one-launch all-reduce."""
    if group not in _ONE_SHOT:
        _ONE_SHOT[group] = OneShotAllReduce(group, max_bytes)
    return _ONE_SHOT[group]


def disable_one_shot(group=None):
    ar = _ONE_SHOT.pop(group, None)
    if ar is not None:
        ar.close()


def all_reduce_sum(y, group=None):
    """Sum y over the ranks of `group`, in place: the one-launch form for small messages when enabled, else NCCL."""
    ar = _ONE_SHOT.get(group)
    if ar is not None and ar.takes(y):
        return ar.reduce(y)
    dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


def _clone_meta(lin: LinearFLH, in_features: int, out_features: int) -> LinearFLH:
    out = LinearFLH(in_features, out_features, bias=lin.bias is not None, dtype=lin.w_scale.dtype,
                    device=lin.w_packed.device, dual_hadamard=lin.dual_hadamard, in_group_size=lin.in_group_size,
                    out_group_size=lin.out_group_size, no_hadamard=lin.no_hadamard, group_size=lin.weight_group_size)
    out.full_hadamard_blocks = lin.full_hadamard_blocks
    return out


def shard_column(lin: LinearFLH, rank: int, world: int) -> LinearFLH:
    """Rows [rank*N/world, (rank+1)*N/world) of the weight."""
    N, K = lin.out_features, lin.in_features
    assert N % world == 0 and (N // world) % 128 == 0, "N / tp must be a multiple of 128"
    n = N // world
    out = _clone_meta(lin, K, n)
    out.w_packed.copy_(lin.w_packed.view(N, K // 2)[rank * n:(rank + 1) * n].reshape(-1))
    out.w_scale.copy_(lin.w_scale[rank * n:(rank + 1) * n])
    out.w_zero.copy_(lin.w_zero[rank * n:(rank + 1) * n])
    if lin.bias is not None:
        out.bias.copy_(lin.bias[rank * n:(rank + 1) * n])
    return out


def shard_row(lin: LinearFLH, rank: int, world: int) -> LinearFLH:
    """Columns [rank*K/world, (rank+1)*K/world) of every weight row.  The bias stays on rank 0 only, so
    that the all-reduced sum carries it once.  A weight rotated with the full-width transform can only be
    split where the transform is block-diagonal: it must have been made with
    LinearFLH.from_float(full_hadamard=True, hadamard_blocks=world), because each rank rotates its K / world
    activations by themselves and (W H_K)[:, shard] is not W[:, shard] H_{K/world}."""
    N, K = lin.out_features, lin.in_features
    assert K % world == 0 and (K // world) % 128 == 0, "K / tp must be a multiple of 128"
    if lin.full_hadamard_blocks not in (0, world) and world > 1:
        raise ValueError(f"this weight was rotated over {lin.full_hadamard_blocks} block(s) of K; a row-parallel split over "
                         f"{world} ranks needs from_float(full_hadamard=True, hadamard_blocks={world})")
    k = K // world
    out = _clone_meta(lin, k, N)
    if lin.full_hadamard_blocks:
        out.full_hadamard_blocks = 1                # the shard's own K is rotated as a whole
    out.w_packed.copy_(lin.w_packed.view(N, K // 2)[:, rank * k // 2:(rank + 1) * k // 2].reshape(-1))
    g = lin.w_scale.shape[1]
    if g > 1:
        gs = g // world
        out.w_scale.copy_(lin.w_scale[:, rank * gs:(rank + 1) * gs])
        out.w_zero.copy_(lin.w_zero[:, rank * gs:(rank + 1) * gs])
    else:
        out.w_scale.copy_(lin.w_scale)
        out.w_zero.copy_(lin.w_zero)
    if lin.bias is not None:
        out.bias.copy_(lin.bias if rank == 0 else torch.zeros_like(lin.bias))
    return out


class ColumnParallelLinearFLH(torch.nn.Module):
    def __init__(self, shard: LinearFLH, group=None, gather_output: bool = False):
        super().__init__()
        self.shard, self.group, self.gather_output = shard, group, gather_output

    def forward(self, x, a_scale=None, a_zero=None, **kw):
        with timing.region("gemm"):
            y = self.shard(x, a_scale, a_zero, **kw)
        if self.gather_output and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            parts = [torch.empty_like(y) for _ in range(dist.get_world_size(self.group))]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelLinearFLH(torch.nn.Module):
    """Row-parallel linear: this rank's K-slice of the GEMM, then the all-reduce of the f16 partial outputs.

    Large batches (prefill) are cut into `overlap_chunks` blocks of token rows: the all-reduce of block i runs on NCCL's
    stream while the GEMM of block i + 1 runs on the compute stream, so most of the 134 MB exchange of a 70B-shaped
    prefill hides behind the tensor cores.  The result is the same bits as the unchunked form: rows are independent in
    the GEMM and NCCL reduces element by element."""

    OVERLAP_MIN_ROWS = 2048      # batches from which the GEMM is cut into blocks
    OVERLAP_BLOCK_ROWS = 2048    # rows per block (a multiple of the GEMM's 256-row tile)

    def __init__(self, shard: LinearFLH, group=None):
        super().__init__()
        self.shard, self.group = shard, group

    def forward(self, x, a_scale=None, a_zero=None, **kw):
        """x, a_scale, a_zero: this rank's slice of the quantised activations."""
        multi = dist.is_initialized() and dist.get_world_size(self.group) > 1
        M = x.numel() // x.shape[-1]
        if multi and M >= 2 * self.OVERLAP_BLOCK_ROWS and M >= self.OVERLAP_MIN_ROWS and not torch.cuda.is_current_stream_capturing():
            lead = x.shape[:-1]
            xs, ss = x.reshape(M, -1), a_scale.reshape(M, -1)
            zs = None if a_zero is None else a_zero.reshape(M, -1)
            y = torch.empty((M, self.shard.out_features), dtype=kw.get("out_dtype") or self.shard.w_scale.dtype, device=x.device)
            works = []
            for r0 in range(0, M, self.OVERLAP_BLOCK_ROWS):
                r1 = min(M, r0 + self.OVERLAP_BLOCK_ROWS)
                with timing.region("gemm"):
                    self.shard(xs[r0:r1], ss[r0:r1], None if zs is None else zs[r0:r1], out=y[r0:r1], **kw)
                works.append(dist.all_reduce(y[r0:r1], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            with timing.region("allreduce"):          # what is left of the exchange after the last GEMM block
                for w in works:
                    w.wait()
            return y.view(lead + (self.shard.out_features,))
        with timing.region("gemm"):
            y = self.shard(x, a_scale, a_zero, **kw)
        if multi:
            with timing.region("allreduce"):
                all_reduce_sum(y, self.group)
        return y

    def forward_add_norm_quant(self, x, a_scale, a_zero, residual, eps: float, clip: float = 1.0, **kw):
        """Decode: the GEMM, then ONE launch for the all-reduce, the residual add, the RMS-norm and the per-token quantiser
        of the next linear's input.  `residual` is updated in place; returns (q, scale, zero), or None — before anything
        ran — when the one-launch all-reduce is not enabled for this group or does not take the shape (the caller then
        runs the separate steps)."""
        ar = _ONE_SHOT.get(self.group)
        if ar is None or not (dist.is_initialized() and dist.get_world_size(self.group) > 1):
            return None
        M, K = x.numel() // x.shape[-1], self.shard.out_features
        dtype = kw.get("out_dtype") or self.shard.w_scale.dtype
        if (M > 128 or K not in (4096, 8192) or M * K * 2 > ar.max_bytes or dtype not in (torch.float16, torch.bfloat16)
                or residual.dtype != dtype or residual.numel() != M * K or not residual.is_contiguous() or residual.data_ptr() % 16):
            return None
        with timing.region("gemm"):
            y = self.shard(x, a_scale, a_zero, **kw)
        assert ar.takes_fused(y.view(M, K), residual.view(M, K))
        with timing.region("allreduce"):
            return ar.reduce_add_norm_quant(y.view(M, K), residual.view(M, K), eps, clip)

    def forward_scatter(self, x, a_scale=None, a_zero=None, blocks: int = 1, **kw):
        """Sequence-parallel form: this rank's K-slice of the GEMM over ALL token rows, then a reduce-scatter — every rank
        receives only the summed rows it owns (half the bytes of the all-reduce; the other half, the all-gather, is done
        later on the QUANTISED activations, 4x smaller, see gather_quantised).

        blocks > 1: the rows are cut into `blocks` equal blocks; the reduce-scatter of block b runs on NCCL's stream while the
        GEMM of block b + 1 runs on the compute stream.  Rank r then owns rows [r T/(tp blocks), (r + 1) T/(tp blocks)) OF
        EVERY BLOCK (block-cyclic ownership, `local_rows`), and its output holds them block after block."""
        M = x.numel() // x.shape[-1]
        world = dist.get_world_size(self.group)
        xs, ss = x.reshape(M, -1), a_scale.reshape(M, -1)
        zs = None if a_zero is None else a_zero.reshape(M, -1)
        N = self.shard.out_features
        out = torch.empty((M // world, N), dtype=kw.get("out_dtype") or self.shard.w_scale.dtype, device=x.device)
        assert blocks >= 1 and M % (world * blocks) == 0, "rows must divide by ranks x blocks"
        mb, tb = M // blocks, M // blocks // world
        y = torch.empty((M, N), dtype=out.dtype, device=x.device)
        works = []
        for b in range(blocks):
            r0, r1 = b * mb, (b + 1) * mb
            with timing.region("gemm"):
                self.shard(xs[r0:r1], ss[r0:r1], None if zs is None else zs[r0:r1], out=y[r0:r1], **kw)
            works.append(dist.reduce_scatter_tensor(out[b * tb:(b + 1) * tb], y[r0:r1], op=dist.ReduceOp.SUM, group=self.group,
                                                    async_op=True))
        with timing.region("allreduce"):              # what is left of the exchange after the last GEMM block
            for w in works:
                w.wait()
        return out


def local_rows(x, rank: int, world: int, blocks: int = 1):
    """This rank's rows of x [T, ..] under the ownership forward_scatter(blocks=...) produces: rows
    [r T/(tp blocks), (r + 1) T/(tp blocks)) of every block, block after block (blocks = 1: one contiguous slice)."""
    T = x.shape[0]
    tb = T // blocks // world
    return x.view(blocks, world, tb, *x.shape[1:])[:, rank].reshape(blocks * tb, *x.shape[1:])


def _natural_order(o, world: int, blocks: int):
    """[rank][block][rows] (what an all-gather of local rows returns) -> [block][rank][rows] = natural row order."""
    if blocks <= 1:
        return o
    tb = o.shape[0] // world // blocks
    return o.view(world, blocks, tb, *o.shape[1:]).transpose(0, 1).reshape(o.shape)


def gather_rows(x, group=None, blocks: int = 1):
    """All-gather of local rows (see local_rows) back into natural row order."""
    world = dist.get_world_size(group)
    x = x.contiguous()
    o = torch.empty((x.shape[0] * world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(o, x, group=group)
    return _natural_order(o, world, blocks)


def gather_quantised(q, s, z, group=None, blocks: int = 1):
    """All-gather of quantised token rows (codes u8 [t, K/2], scales [t, g], zero-points [t, g] or None) along the token
    dimension: the local rows of every rank -> all T rows in natural order.  The int4 codes are a quarter of the f16
    activations an all-reduce would have carried; scales and zero-points travel as one tensor."""
    world = dist.get_world_size(group)
    with timing.region("allreduce"):
        sz = s if z is None else torch.cat((s, z), dim=-1)           # one small exchange instead of two
        outs, works = [], []
        for t in (q, sz):
            t = t.contiguous()
            o = torch.empty((t.shape[0] * world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            works.append(dist.all_gather_into_tensor(o, t, group=group, async_op=True))
            outs.append(o)
        for w in works:
            w.wait()
        qf, szf = _natural_order(outs[0], world, blocks), _natural_order(outs[1], world, blocks)
    if z is None:
        return [qf, szf, None]
    g = s.shape[-1]
    return [qf, szf[..., :g].contiguous(), szf[..., g:].contiguous()]
