"""FLH's on-disk format for a quantised Llama-shaped model, and conversion into it.

Format (FLH_LlamaForCausalLM.save_quantized / load_quantized, flh/quantized_model/modeling_llama.py:1079-1137, 1140-1253):
a directory with
    model.pt                   torch.save of the state dict, f16, on CPU; every packed linear is three tensors
                               `<name>.w_packed` (flat uint8, two int4 per byte), `<name>.w_scale` [N, K/gs] or [N, 1],
                               `<name>.w_zero` (uint8, same shape) (+ `<name>.bias`), under the Hugging Face Llama names
                               model.layers.<i>.self_attn.{q,k,v,o}_proj / mlp.{gate,up,down}_proj,
                               model.embed_tokens.weight, model.layers.<i>.{input,post_attention}_layernorm.weight,
                               model.norm.weight, lm_head.weight;
    quantization_config.json   weight_bits, weight_group_size, act_bits, act_group_size, weight_sym, act_sym,
                               clip_ratio, dtype;
    config.json                the Llama architecture (hidden_size, intermediate_size, num_attention_heads, ...).
This module writes and reads exactly that, for flh_b200.model.Decoder:
  * the decoder keeps q/k/v and gate/up merged (one GEMM each); they are split back into the reference's separate tensors
    on save and concatenated on load — both lossless, the merged weight is a row concatenation;
  * load_quantized can build ONE RANK of a tensor-parallel model directly: it memory-maps model.pt and copies only that
    rank's rows (column-parallel) or K-columns (row-parallel) to the device, never the full model;
  * quantize_decoder converts float weights on the device they live on (a GPU: rotation in float64, RTN, packing — the
    arithmetic of LinearFLH.from_float, flh/nn/linear.py:190-285, run by the same code on CUDA tensors).
Two keys of quantization_config.json are additions (ignored by the reference's loader): "act_mode" and
"down_hadamard_blocks" (how the down_proj weights were rotated for the online full-width transform).
"""
from __future__ import annotations

import json
import os

import torch

from .model import Decoder, DecoderConfig, DecoderLayer, RMSNorm
from .nn import LinearFLH
from .tp import ColumnParallelLinearFLH, RowParallelLinearFLH

_ARCH_KEYS = {"hidden_size": "hidden", "intermediate_size": "ffn", "num_attention_heads": "n_heads",
              "num_key_value_heads": "n_kv_heads", "num_hidden_layers": "n_layers", "vocab_size": "vocab",
              "rms_norm_eps": "eps", "rope_theta": "rope_theta"}


def _split_rows(lin: LinearFLH, sizes):
    """The merged linear as separate (w_packed flat, w_scale, w_zero, bias) per block of output rows."""
    N, K = lin.out_features, lin.in_features
    wp = lin.w_packed.view(N, K // 2)
    out, r0 = [], 0
    for n in sizes:
        out.append((wp[r0:r0 + n].reshape(-1), lin.w_scale[r0:r0 + n], lin.w_zero[r0:r0 + n],
                    None if lin.bias is None else lin.bias[r0:r0 + n]))
        r0 += n
    assert r0 == N
    return out


def _put(sd, prefix, parts):
    wp, ws, wz, b = parts
    sd[prefix + ".w_packed"] = wp.detach().cpu().contiguous()
    sd[prefix + ".w_scale"] = ws.detach().cpu().half().contiguous()
    sd[prefix + ".w_zero"] = wz.detach().cpu().contiguous()
    if b is not None:
        sd[prefix + ".bias"] = b.detach().cpu().half().contiguous()


def state_dict_reference_layout(model: Decoder) -> dict:
    """The model's tensors under the reference's state-dict names (CPU, f16).  Single-GPU models only."""
    cfg = model.cfg
    assert cfg.tp == 1, "save the unsharded model; load_quantized shards it per rank"
    hd = cfg.head_dim
    sd = {"model.embed_tokens.weight": model.embed.weight.detach().cpu().half()}
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        q, k, v = _split_rows(layer.qkv.shard, (cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.n_kv_heads * hd))
        _put(sd, p + "self_attn.q_proj", q)
        _put(sd, p + "self_attn.k_proj", k)
        _put(sd, p + "self_attn.v_proj", v)
        _put(sd, p + "self_attn.o_proj", _split_rows(layer.o.shard, (cfg.hidden,))[0])
        g, u = _split_rows(layer.gate_up.shard, (cfg.ffn, cfg.ffn))
        _put(sd, p + "mlp.gate_proj", g)
        _put(sd, p + "mlp.up_proj", u)
        _put(sd, p + "mlp.down_proj", _split_rows(layer.down.shard, (cfg.hidden,))[0])
        sd[p + "input_layernorm.weight"] = layer.norm1.weight.detach().cpu().half()
        sd[p + "post_attention_layernorm.weight"] = layer.norm2.weight.detach().cpu().half()
    sd["model.norm.weight"] = model.norm.weight.detach().cpu().half()
    if model.head is not None:
        sd["lm_head.weight"] = model.head.weight.detach().cpu().half()
    return sd


def save_quantized(model: Decoder, save_directory: str) -> None:
    """Writes model.pt, quantization_config.json and config.json as FLH_LlamaForCausalLM.save_quantized does."""
    os.makedirs(save_directory, exist_ok=True)
    cfg = model.cfg
    torch.save(state_dict_reference_layout(model), os.path.join(save_directory, "model.pt"), pickle_protocol=4)
    sym = cfg.act_mode == "group_sym"
    gs = model.layers[0].qkv.shard.weight_group_size if len(model.layers) else (128 if sym else -1)
    quant = {"weight_bits": 4, "weight_group_size": gs, "act_bits": 4, "act_group_size": 128 if sym else -1,
             "weight_sym": True, "act_sym": sym, "clip_ratio": 1.0, "dtype": "float16",
             "act_mode": cfg.act_mode,
             "down_hadamard_blocks": model.layers[0].down.shard.full_hadamard_blocks if len(model.layers) else 0}
    with open(os.path.join(save_directory, "quantization_config.json"), "w") as f:
        json.dump(quant, f, indent=2)
    arch = {hf: getattr(cfg, ours) for hf, ours in _ARCH_KEYS.items()}
    arch.update(model_type="llama", architectures=["LlamaForCausalLM"], hidden_act="silu", torch_dtype="float16",
                tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    with open(os.path.join(save_directory, "config.json"), "w") as f:
        json.dump(arch, f, indent=2)


def _load_state_dict(path):
    """model.pt as a dict of CPU tensors, memory-mapped where torch can.  The reference writes it with pickle protocol 4
    (modeling_llama.py:1107), which torch's restricted unpickler does not read: such a file — a plain dict of tensors
    written by save_quantized — is then read with the full unpickler."""
    import pickle
    for kw in ({"mmap": True, "weights_only": True}, {"weights_only": True}, {"mmap": True, "weights_only": False},
               {"weights_only": False}):
        try:
            return torch.load(path, map_location="cpu", **kw)
        except (TypeError, RuntimeError, pickle.UnpicklingError):
            continue
    raise RuntimeError(f"cannot read {path}")


def _linear_from(sd, names, k, device, gs, rows=None, cols=None):
    """One LinearFLH from the saved tensors of `names` (concatenated along the output rows), restricted to rows
    [rows[0], rows[1]) of EACH named tensor or to K-columns [cols[0], cols[1]); only the slice is copied to the device."""
    wps, wss, wzs, bs = [], [], [], []
    for nm in names:
        n = sd[nm + ".w_scale"].shape[0]
        wp = sd[nm + ".w_packed"].view(n, k // 2)
        ws, wz = sd[nm + ".w_scale"], sd[nm + ".w_zero"]
        b = sd.get(nm + ".bias")
        if rows is not None:
            r0, r1 = rows(n)
            wp, ws, wz = wp[r0:r1], ws[r0:r1], wz[r0:r1]
            b = None if b is None else b[r0:r1]
        if cols is not None:
            c0, c1 = cols
            wp = wp[:, c0 // 2:c1 // 2]
            if ws.shape[1] > 1:
                g = ws.shape[1] * (c1 - c0) // k
                g0 = ws.shape[1] * c0 // k
                ws, wz = ws[:, g0:g0 + g], wz[:, g0:g0 + g]
        wps.append(wp); wss.append(ws); wzs.append(wz); bs.append(b)
    wp, ws, wz = torch.cat(wps), torch.cat(wss), torch.cat(wzs)
    kk = wp.shape[1] * 2
    lin = LinearFLH(kk, wp.shape[0], bias=bs[0] is not None, dtype=torch.float16, device=device, group_size=gs, in_group_size=128)
    lin.w_packed.copy_(wp.reshape(-1))
    lin.w_scale.copy_(ws)
    lin.w_zero.copy_(wz)
    if bs[0] is not None:
        lin.bias.copy_(torch.cat(bs))
    return lin


def load_quantized(load_directory: str, device="cuda", tp_rank: int = 0, tp_world: int = 1, group=None,
                   n_layers: int | None = None) -> Decoder:
    """Builds the Decoder (or rank tp_rank of tp_world of it) from a directory written by save_quantized — ours or the
    reference's.  model.pt is memory-mapped; a tensor-parallel rank copies only its own slices to the device:
    q/k/v and gate/up by output rows (whole heads per rank), o_proj and down_proj by K-columns."""
    with open(os.path.join(load_directory, "quantization_config.json")) as f:
        quant = json.load(f)
    with open(os.path.join(load_directory, "config.json")) as f:
        arch = json.load(f)
    if quant.get("weight_bits", 4) != 4 or quant.get("act_bits", 4) != 4:
        raise ValueError("flh_b200 serves W4A4 checkpoints")
    path = os.path.join(load_directory, "model.pt")
    sd = _load_state_dict(path)
    kw = {ours: arch[hf] for hf, ours in _ARCH_KEYS.items() if hf in arch}
    kw.setdefault("n_kv_heads", kw["n_heads"])
    if n_layers is not None:
        kw["n_layers"] = n_layers
    act_mode = quant.get("act_mode") or ("group_sym" if quant.get("act_sym", True) else "token_asym")
    cfg = DecoderConfig(**kw, act_mode=act_mode, tp=tp_world)
    blocks = int(quant.get("down_hadamard_blocks", 0))
    if act_mode == "token_asym" and blocks not in (0, tp_world) and tp_world > 1:
        raise ValueError(f"down_proj was rotated over {blocks} block(s) of K; tensor parallelism over {tp_world} ranks needs "
                         f"a checkpoint converted with hadamard_blocks={tp_world}")
    gs = quant.get("weight_group_size", 128)
    hd = cfg.head_dim
    assert cfg.n_heads % tp_world == 0 and cfg.ffn % tp_world == 0 and (cfg.ffn // tp_world) % 128 == 0
    part = lambda n: (tp_rank * (n // tp_world), (tp_rank + 1) * (n // tp_world))       # this rank's rows of an n-row tensor
    kv_part = part if cfg.n_kv_heads >= tp_world else (lambda n: (0, n))                # fewer KV heads than ranks: replicated

    model = Decoder.__new__(Decoder)
    torch.nn.Module.__init__(model)
    model.cfg, model.device = cfg, torch.device(device)
    model.embed = torch.nn.Embedding(cfg.vocab, cfg.hidden, device=device, dtype=torch.float16)
    model.embed.weight.data.copy_(sd["model.embed_tokens.weight"])
    layers = []
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        layer = DecoderLayer(cfg, device, gen=None, group=group)
        qkv = [_linear_from(sd, [p + "self_attn.q_proj"], cfg.hidden, device, gs, rows=part),
               _linear_from(sd, [p + "self_attn.k_proj"], cfg.hidden, device, gs, rows=kv_part),
               _linear_from(sd, [p + "self_attn.v_proj"], cfg.hidden, device, gs, rows=kv_part)]
        layer.qkv = ColumnParallelLinearFLH(_concat(qkv, device, gs), group)
        o_k = cfg.n_heads * hd
        layer.o = RowParallelLinearFLH(_linear_from(sd, [p + "self_attn.o_proj"], o_k, device, gs,
                                                    cols=(tp_rank * o_k // tp_world, (tp_rank + 1) * o_k // tp_world)), group)
        gu = [_linear_from(sd, [p + "mlp.gate_proj"], cfg.hidden, device, gs, rows=part),
              _linear_from(sd, [p + "mlp.up_proj"], cfg.hidden, device, gs, rows=part)]
        layer.gate_up = ColumnParallelLinearFLH(_concat(gu, device, gs), group)
        down = _linear_from(sd, [p + "mlp.down_proj"], cfg.ffn, device, gs,
                            cols=(tp_rank * cfg.ffn // tp_world, (tp_rank + 1) * cfg.ffn // tp_world))
        down.full_hadamard_blocks = 1 if blocks else 0
        layer.down = RowParallelLinearFLH(down, group)
        for lin in (layer.o.shard, layer.down.shard):      # the all-reduced sum must carry a bias once
            if lin.bias is not None and tp_rank != 0:
                lin.bias.zero_()
        layer.norm1.weight.data.copy_(sd[p + "input_layernorm.weight"])
        layer.norm2.weight.data.copy_(sd[p + "post_attention_layernorm.weight"])
        layers.append(layer)
    model.layers = torch.nn.ModuleList(layers)
    model.norm = RMSNorm(cfg.hidden, cfg.eps).to(device)
    model.norm.weight.data.copy_(sd["model.norm.weight"])
    model.head = None
    if "lm_head.weight" in sd:
        model.head = torch.nn.Linear(cfg.hidden, cfg.vocab, bias=False, device=device, dtype=torch.float16)
        model.head.weight.data.copy_(sd["lm_head.weight"])
    return model


def _concat(lins, device, gs):
    """Row concatenation of LinearFLH modules with the same K (q|k|v, gate|up)."""
    k = lins[0].in_features
    n = sum(l.out_features for l in lins)
    out = LinearFLH(k, n, bias=lins[0].bias is not None, dtype=torch.float16, device=device, group_size=gs, in_group_size=128)
    out.w_packed.copy_(torch.cat([l.w_packed.view(l.out_features, k // 2) for l in lins]).reshape(-1))
    out.w_scale.copy_(torch.cat([l.w_scale for l in lins]))
    out.w_zero.copy_(torch.cat([l.w_zero for l in lins]))
    if out.bias is not None:
        out.bias.copy_(torch.cat([l.bias for l in lins]))
    return out


@torch.no_grad()
def quantize_decoder(float_layers, cfg: DecoderConfig, device, embed=None, norm=None, head=None,
                     hadamard_blocks: int = 1) -> Decoder:
    """Float weights -> a single-GPU quantised Decoder, converted ON `device` (rotation in float64, RTN, packing run as
    torch kernels where the weights live: the arithmetic of LinearFLH.from_float, flh/nn/linear.py:190-285).

    float_layers: per layer a dict of float weight matrices [out, in] under the names q, k, v, o, gate, up, down.
    group_sym mode: group-128 weights, no rotation (as the reference builds its model: every ActQuantizer has
    use_hadamard=False and the linears no_hadamard=True, modeling_llama.py:317-372, 478-520).  token_asym mode: per-channel
    weights; down_proj rotated by the full-width transform over `hadamard_blocks` blocks of K (= the tensor-parallel
    degree it will be served at) to match the online transform in front of it."""
    sym = cfg.act_mode == "group_sym"
    gs = 128 if sym else -1
    model = Decoder.__new__(Decoder)
    torch.nn.Module.__init__(model)
    model.cfg, model.device = cfg, torch.device(device)

    def conv(w, full_had=False):
        lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=device, dtype=torch.float16)
        lin.weight.data.copy_(w)
        return LinearFLH.from_float(lin, weight_group_size=gs, in_group_size=128, no_hadamard=not full_had,
                                    full_hadamard=full_had, hadamard_blocks=hadamard_blocks)

    layers = []
    for fl in float_layers:
        layer = DecoderLayer(cfg, device, gen=None, group=None)
        layer.qkv = ColumnParallelLinearFLH(_concat([conv(fl["q"]), conv(fl["k"]), conv(fl["v"])], device, gs))
        layer.o = RowParallelLinearFLH(conv(fl["o"]))
        layer.gate_up = ColumnParallelLinearFLH(_concat([conv(fl["gate"]), conv(fl["up"])], device, gs))
        layer.down = RowParallelLinearFLH(conv(fl["down"], full_had=not sym))
        layers.append(layer)
    model.layers = torch.nn.ModuleList(layers)
    model.embed = torch.nn.Embedding(cfg.vocab, cfg.hidden, device=device, dtype=torch.float16)
    if embed is not None:
        model.embed.weight.data.copy_(embed)
    model.norm = RMSNorm(cfg.hidden, cfg.eps).to(device)
    if norm is not None:
        model.norm.weight.data.copy_(norm)
    model.head = None
    if head is not None:
        model.head = torch.nn.Linear(cfg.hidden, cfg.vocab, bias=False, device=device, dtype=torch.float16)
        model.head.weight.data.copy_(head)
    return model
