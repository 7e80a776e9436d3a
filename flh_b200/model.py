"""Llama-shaped W4A4 decoder on the flh_b200 hot path (the caller either side of the kernels).

Mirrors the wiring of FLH_LlamaAttention / FLH_LlamaMLP (flh/quantized_model/modeling_llama.py:374-470,
522-526): RMSNorm (weight folded into the next linear) -> activation quantiser -> packed linears; RoPE;
f16 attention with a KV cache; quantiser -> o_proj; quantiser -> gate/up -> SiLU*up -> quantiser ->
down_proj.  Differences, all on the host side: q/k/v and gate/up are merged into one GEMM each (one
quantiser output feeds them), and the linears can be tensor-parallel (flh_b200.tp).

Two activation modes:
  "group_sym"   FLH's CUDA contract: per-(token, 128) symmetric int4, group-128 weight scales, no online
                transform (FLH builds every ActQuantizer with use_hadamard=False, :317-319, 478-480);
  "token_asym"  the fake_quant wiring (fake_quant/main.py:31-35, 63-84): per-token asymmetric int4,
                per-channel symmetric weights, full-width online Hadamard in front of down_proj.
Weights are random (no checkpoint in reach): `random_init` draws packed codes and scales directly on the
device; `from_float_layer` rotates, RTN-quantises and packs real float weights (tests).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _CUDA, timing
from .nn import ActQuantizer, LinearFLH
from .tp import ColumnParallelLinearFLH, RowParallelLinearFLH, gather_quantised, gather_rows, local_rows


@dataclass
class DecoderConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    ffn: int = 11008
    n_layers: int = 32
    vocab: int = 32000
    rope_theta: float = 10000.0
    eps: float = 1e-5
    act_mode: str = "group_sym"          # or "token_asym"
    tp: int = 1
    fuse_norm: bool = True               # RMS-norm fused into the per-token quantiser where the kernel exists
    fuse_glue: bool = True               # rotary embedding + KV-cache write, and SiLU(gate) * up (+ transform + quantiser), as
                                         # kernels of this library instead of PyTorch tensor operations
    sp_blocks: int = 1                   # sequence-parallel: row blocks per row-parallel GEMM; with 2 the reduce-scatter of one block
                                         # runs beside the GEMM of the next (from 2,048 rows per block).  Measured slower at 8 GPUs
                                         # (NCCL's kernels take SMs from the GEMM, two exchanges cost two latencies): off
    seq_parallel: bool = True            # tensor-parallel prefill with the residual stream sharded by tokens: row-parallel
                                         # outputs are reduce-scattered, norm + quantiser run on T / tp rows, and the all-gather
                                         # carries int4 codes (a quarter of the f16 bytes)

    @property
    def head_dim(self):
        return self.hidden // self.n_heads


LLAMA2_7B = dict(hidden=4096, n_heads=32, n_kv_heads=32, ffn=11008, n_layers=32)
LLAMA3_70B = dict(hidden=8192, n_heads=64, n_kv_heads=8, ffn=28672, n_layers=80, rope_theta=500000.0)


def _random_linear(k, n, cfg, device, gen):
    """A LinearFLH with uniform random int4 codes and scales ~ U(0.005, 0.02)."""
    gs = 128 if cfg.act_mode == "group_sym" else -1
    lin = LinearFLH(k, n, dtype=torch.float16, device=device, group_size=gs, in_group_size=128)
    lin.w_packed.copy_(torch.randint(0, 256, lin.w_packed.shape, dtype=torch.uint8, device=device, generator=gen))
    lin.w_scale.copy_((torch.rand(lin.w_scale.shape, device=device, generator=gen) * 0.015 + 0.005).half() / math.sqrt(k / 64))
    return lin


class RMSNorm(torch.nn.Module):
    """flh/nn/normalization.py: x * rsqrt(mean(x^2) + eps) * weight (weight is 1 once folded)."""

    def __init__(self, dim, eps):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim, dtype=torch.float16), requires_grad=False)

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_tables(pos, d, theta):
    """cos, sin [S, d / 2] binary32 of the rotary angles pos * theta^(-2i/d) — the values rope() multiplies with."""
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=pos.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope(x, pos, theta):
    """Rotary embedding, half-split convention (HF Llama): x [B, S, H, D], pos [S]."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, device, gen=None, group=None):
        super().__init__()
        self.cfg, self.group = cfg, group
        tp = cfg.tp
        hd = cfg.head_dim
        self.nh, self.nkv = cfg.n_heads // tp, max(cfg.n_kv_heads // tp, 1)
        sym = cfg.act_mode == "group_sym"
        mk = lambda had: ActQuantizer(bits=4, group_size=128 if sym else -1, sym=sym, use_hadamard=had, packed_output=True)
        self.q_in, self.q_attn, self.q_mlp = mk(False), mk(False), mk(False)
        self.q_down = mk(not sym)        # token_asym: full-width online transform in front of down_proj
        self.norm1, self.norm2 = RMSNorm(cfg.hidden, cfg.eps).to(device), RMSNorm(cfg.hidden, cfg.eps).to(device)
        if gen is not None:              # random weights, already per-rank shards
            self.qkv = ColumnParallelLinearFLH(_random_linear(cfg.hidden, (self.nh + 2 * self.nkv) * hd, cfg, device, gen), group)
            self.o = RowParallelLinearFLH(_random_linear(self.nh * hd, cfg.hidden, cfg, device, gen), group)
            self.gate_up = ColumnParallelLinearFLH(_random_linear(cfg.hidden, 2 * cfg.ffn // tp, cfg, device, gen), group)
            self.down = RowParallelLinearFLH(_random_linear(cfg.ffn // tp, cfg.hidden, cfg, device, gen), group)

    def _norm_quant(self, norm, quant, x):
        """RMS-norm then quantise.  Per-token mode at hidden sizes 4096 / 8192: one fused kernel (the norm weight is 1,
        as FLH leaves it after folding it into the next linear); otherwise the two steps."""
        cfg = self.cfg
        if cfg.fuse_norm and cfg.act_mode == "token_asym" and cfg.hidden in (4096, 8192) and not quant.use_hadamard:
            lead = x.shape[:-1]
            q, s, z = _CUDA.rmsnorm_quant_token_asym_i4(x.reshape(-1, cfg.hidden), norm.eps, hadamard=False)
            return s.view(lead + (1,)), z.view(lead + (1,)), q.view(lead + (cfg.hidden // 2,))
        if cfg.fuse_norm and cfg.act_mode == "group_sym" and cfg.hidden == 4096 and quant.group_size == 128 and x.dtype == torch.float16:
            lead = x.shape[:-1]
            q, s = _CUDA.rmsnorm_quant_group_sym_i4(x.reshape(-1, cfg.hidden), norm.eps, hadamard=quant.use_hadamard)
            if quant.use_hadamard:
                s = s / math.sqrt(128)                   # the kernel's transform is un-normalised (as in ActQuantizer.forward)
            return s.view(lead + (cfg.hidden // 128,)), None, q.view(lead + (cfg.hidden // 2,))
        return quant(norm(x))

    def forward(self, x, pos, cache=None, tables=None, shape=None, pre=None, next_layer=None):
        """x [B, S, hidden] f16 (or, sequence-parallel, this rank's B S / tp rows with shape = (B, S, blocks)); pos [S]
        absolute positions; cache = (k, v) [B, nkv, T, D] with a write cursor `cache[2]`, or None for a cache-less prefill;
        tables = rope_tables(pos, ...) shared by the layers.
        Tensor-parallel decode with tp.enable_one_shot(): the all-reduce behind o_proj / down_proj, the residual add, the
        RMS-norm and the quantiser of the next linear's input run as ONE launch, and x is then updated in place.  For
        down_proj the next linear belongs to `next_layer`: the layer returns (x, pre) and the caller hands `pre` (that
        layer's quantised input) to it."""
        cfg = self.cfg
        sp = x.dim() == 2                                # sequence-parallel: x holds this rank's T / tp of the B * S rows (tp.local_rows)
        if sp:
            B, S, blocks = shape
        else:
            B, S, _ = x.shape
        hd = cfg.head_dim
        if pre is not None:
            s, z, q = pre
        else:
            with timing.region("quant"):
                s, z, q = self._norm_quant(self.norm1, self.q_in, x)
        if sp:
            q, s, z = gather_quantised(q, s, z, self.qkv.group, blocks)
            q, s = q.view(B, S, -1), s.view(B, S, -1)
            z = None if z is None else z.view(B, S, -1)
        qkv = self.qkv(q, s, z)
        with timing.region("glue"):
            mask, causal = None, S > 1
            cur = 0 if cache is None else cache[2]
            if cfg.fuse_glue and qkv.dtype == torch.float16:
                # one kernel: rotary embedding of q and k, q laid out for the attention call, k and v written at their cache positions
                if tables is None:
                    tables = rope_tables(pos, hd, cfg.rope_theta)
                if cache is not None:
                    kc, vc = cache[0], cache[1]
                else:
                    kc = torch.empty((B, self.nkv, S, hd), dtype=qkv.dtype, device=qkv.device)
                    vc = torch.empty_like(kc)
                qh = torch.empty((B, self.nh, S, hd), dtype=qkv.dtype, device=qkv.device)
                _CUDA.rope_kv(qkv.view(B * S, -1), tables[0], tables[1], qh, kc, vc, B, S, self.nh, self.nkv, cur)
                kh, vh = kc[:, :, :cur + S], vc[:, :, :cur + S]
            else:
                qh, kh, vh = qkv.split((self.nh * hd, self.nkv * hd, self.nkv * hd), dim=-1)
                qh = rope(qh.view(B, S, self.nh, hd), pos, cfg.rope_theta).transpose(1, 2)
                kh = rope(kh.view(B, S, self.nkv, hd), pos, cfg.rope_theta).transpose(1, 2)
                vh = vh.view(B, S, self.nkv, hd).transpose(1, 2)
                if cache is not None:
                    kc, vc = cache[0], cache[1]
                    kc[:, :, cur:cur + S] = kh
                    vc[:, :, cur:cur + S] = vh
                    kh, vh = kc[:, :, :cur + S], vc[:, :, :cur + S]
            if cur > 0 and S > 1:
                # a chunk appended to a filled cache: query i sees keys 0 .. cur + i (torch's is_causal aligns the
                # triangle with the top-left corner, which is only right for cur = 0)
                mask, causal = torch.ones(S, cur + S, dtype=torch.bool, device=x.device).tril(diagonal=cur), False
        with timing.region("attention"):
            att = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=causal, enable_gqa=self.nh != self.nkv)
            att = att.transpose(1, 2).reshape(B, S, self.nh * hd)
        with timing.region("quant"):
            s, z, q = self.q_attn(att)
        fused = None
        can_fuse = not sp and cfg.tp > 1 and cfg.fuse_norm and cfg.act_mode == "token_asym" and S == 1 and x.is_contiguous()
        if can_fuse:
            # decode: the all-reduce of o_proj, the residual add, the RMS-norm and the quantiser of gate_up's input as ONE launch
            # (tp.enable_one_shot; returns None when that is off or does not take the shape).  x is updated in place.
            fused = self.o.forward_add_norm_quant(q, s, z, x, self.norm2.eps, self.q_mlp.input_clip_ratio)
        if fused is not None:
            lead = x.shape[:-1]
            q, s, z = fused[0].view(lead + (cfg.hidden // 2,)), fused[1].view(lead + (1,)), fused[2].view(lead + (1,))
        else:
            y = self.o.forward_scatter(q, s, z, blocks=blocks) if sp else self.o(q, s, z)
            with timing.region("glue"):
                x = x + y
            with timing.region("quant"):
                s, z, q = self._norm_quant(self.norm2, self.q_mlp, x)
        if sp:
            q, s, z = gather_quantised(q, s, z, self.gate_up.group, blocks)
        gu = self.gate_up(q, s, z)
        if cfg.fuse_glue and cfg.act_mode == "token_asym":
            # SiLU(gate) * up, then the online transform and the quantiser (two launches: measured faster than the one-kernel
            # form, whose epilogue warps would have to make the SiLU rows on top of the quantiser's work)
            with timing.region("quant"):
                lead = gu.shape[:-1]
                q, s, z = _CUDA.silu_mul_quant_token_asym_i4(gu.view(-1, gu.shape[-1]), hadamard=self.q_down.use_hadamard,
                                                             clip=self.q_down.input_clip_ratio)
                s, z, q = s.view(lead + (1,)), z.view(lead + (1,)), q.view(lead + (q.shape[-1],))
        else:
            with timing.region("glue"):
                if cfg.fuse_glue:
                    a = _CUDA.silu_mul(gu.view(-1, gu.shape[-1])).view(gu.shape[:-1] + (gu.shape[-1] // 2,))
                else:
                    g, u = gu.chunk(2, dim=-1)
                    a = F.silu(g) * u
            with timing.region("quant"):
                s, z, q = self.q_down(a)
        if can_fuse and next_layer is not None:
            fused = self.down.forward_add_norm_quant(q, s, z, x, next_layer.norm1.eps, next_layer.q_in.input_clip_ratio)
            if fused is not None:
                lead = x.shape[:-1]
                return x, (fused[1].view(lead + (1,)), fused[2].view(lead + (1,)), fused[0].view(lead + (cfg.hidden // 2,)))
        y = self.down.forward_scatter(q, s, z, blocks=blocks) if sp else self.down(q, s, z)
        with timing.region("glue"):
            return x + y


class Decoder(torch.nn.Module):
    """Embedding -> layers -> final norm -> f16 lm_head (the head stays f16 in FLH, :1032-1046)."""

    def __init__(self, cfg: DecoderConfig, device, seed=0, group=None, with_head=True):
        super().__init__()
        self.cfg, self.device = cfg, device
        gen = torch.Generator(device=device).manual_seed(seed + (dist.get_rank() if dist.is_initialized() else 0))
        self.embed = torch.nn.Embedding(cfg.vocab, cfg.hidden, device=device, dtype=torch.float16)
        # replicated parameters are the same on every rank (the shards above differ by rank): the sequence-parallel form
        # hands rows of the residual stream from rank to rank
        rep = torch.Generator(device=device).manual_seed(seed + 7919)
        self.embed.weight.data.copy_(torch.randn(cfg.vocab, cfg.hidden, device=device, generator=rep).half())
        self.layers = torch.nn.ModuleList(DecoderLayer(cfg, device, gen, group) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.hidden, cfg.eps).to(device)
        self.head = torch.nn.Linear(cfg.hidden, cfg.vocab, bias=False, device=device, dtype=torch.float16) if with_head else None
        if self.head is not None:
            self.head.weight.data.copy_((torch.randn(cfg.vocab, cfg.hidden, device=device, generator=rep) * cfg.hidden ** -0.5).half())

    def prepack_int8(self):
        """Prefill-heavy serving: every W4 linear with per-channel scales keeps an int8 copy of its weights too."""
        for m in self.modules():
            if isinstance(m, LinearFLH):
                m.prepack_int8()
        return self

    def new_cache(self, batch, max_len):
        c = self.cfg
        nkv = max(c.n_kv_heads // c.tp, 1)
        return [[torch.zeros(batch, nkv, max_len, c.head_dim, dtype=torch.float16, device=self.device),
                 torch.zeros(batch, nkv, max_len, c.head_dim, dtype=torch.float16, device=self.device), 0]
                for _ in range(c.n_layers)]

    @torch.no_grad()
    def forward(self, ids, cache=None, start=0):
        B, S = ids.shape
        x = self.embed(ids)
        pos = torch.arange(start, start + S, device=ids.device)
        tables = rope_tables(pos, self.cfg.head_dim, self.cfg.rope_theta) if self.cfg.fuse_glue else None
        world = dist.get_world_size() if dist.is_initialized() else 1
        sp = self.cfg.seq_parallel and self.cfg.tp > 1 and world == self.cfg.tp and S > 1 and (B * S) % world == 0
        if sp:                                           # this rank's rows of the B * S token rows (tp.local_rows)
            blocks = self.cfg.sp_blocks if (B * S) % (world * self.cfg.sp_blocks) == 0 and B * S // self.cfg.sp_blocks >= 2048 else 1
            x = local_rows(x.view(B * S, -1), dist.get_rank(), world, blocks).contiguous()
        pre = None
        for i, layer in enumerate(self.layers):
            if cache is not None:
                cache[i][2] = start
            out = layer(x, pos, None if cache is None else cache[i], tables, shape=(B, S, blocks) if sp else None, pre=pre,
                        next_layer=self.layers[i + 1] if i + 1 < len(self.layers) else None)
            x, pre = out if isinstance(out, tuple) else (out, None)
        if sp:
            x = gather_rows(x, None, blocks).view(B, S, -1)
        x = self.norm(x)
        return x if self.head is None else self.head(x[:, -1:])
