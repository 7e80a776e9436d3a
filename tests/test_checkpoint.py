"""On-disk format (flh/quantized_model/modeling_llama.py:1079-1253) and conversion (flh/nn/linear.py:190-285):
save -> load round trips, the reference's tensor names, per-rank sharded loading, and on-device conversion."""
import json
import os

import numpy as np
import pytest
import torch


def _tiny(mode, device="cpu", seed=3):
    from flh_b200.model import Decoder, DecoderConfig
    cfg = DecoderConfig(hidden=256, n_heads=4, n_kv_heads=2, ffn=512, n_layers=2, vocab=64, act_mode=mode)
    return Decoder(cfg, torch.device(device), seed=seed)


@pytest.mark.parametrize("mode", ["group_sym", "token_asym"])
def test_save_load_round_trip_and_names(tmp_path, mode):
    from flh_b200.checkpoint import load_quantized, save_quantized, state_dict_reference_layout
    m = _tiny(mode)
    m.layers[0].norm1.weight.data.mul_(1.5)
    save_quantized(m, str(tmp_path))
    assert sorted(os.listdir(tmp_path)) == ["config.json", "model.pt", "quantization_config.json"]
    quant = json.load(open(tmp_path / "quantization_config.json"))
    assert {"weight_bits", "weight_group_size", "act_bits", "act_group_size", "weight_sym", "act_sym", "clip_ratio", "dtype"} <= set(quant)
    assert quant["weight_bits"] == 4 and quant["act_sym"] == (mode == "group_sym") and quant["dtype"] == "float16"
    sd = torch.load(tmp_path / "model.pt", weights_only=False)
    # the reference's tensor names and layouts: flat uint8 w_packed, [N, K/gs] (or [N, 1]) f16 scales, uint8 zeros
    for nm, n, k in (("model.layers.0.self_attn.q_proj", 256, 256), ("model.layers.1.self_attn.k_proj", 128, 256),
                     ("model.layers.0.self_attn.o_proj", 256, 256), ("model.layers.1.mlp.gate_proj", 512, 256),
                     ("model.layers.0.mlp.down_proj", 256, 512)):
        g = k // 128 if mode == "group_sym" else 1
        assert sd[nm + ".w_packed"].shape == (n * k // 2,) and sd[nm + ".w_packed"].dtype == torch.uint8
        assert sd[nm + ".w_scale"].shape == (n, g) and sd[nm + ".w_scale"].dtype == torch.float16
        assert sd[nm + ".w_zero"].shape == (n, g) and sd[nm + ".w_zero"].dtype == torch.uint8
    for nm in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.1.input_layernorm.weight",
               "model.layers.0.post_attention_layernorm.weight"):
        assert sd[nm].dtype == torch.float16
    m2 = load_quantized(str(tmp_path), device="cpu")
    a, b = state_dict_reference_layout(m), state_dict_reference_layout(m2)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert m2.cfg.act_mode == mode and m2.cfg.n_kv_heads == 2 and m2.cfg.ffn == 512


def test_sharded_load_equals_sharding_the_full_model(tmp_path):
    from flh_b200.checkpoint import load_quantized, save_quantized
    from flh_b200.tp import shard_row
    m = _tiny("group_sym")
    save_quantized(m, str(tmp_path))
    world = 2
    for rank in range(world):
        s = load_quantized(str(tmp_path), device="cpu", tp_rank=rank, tp_world=world)
        assert s.cfg.tp == world
        for lf, ls in zip(m.layers, s.layers):
            hd = 64
            full = lf.qkv.shard.w_packed.view(-1, 128)                  # rows: 4 q heads, 2 k heads, 2 v heads of 64
            want = torch.cat([full[rank * 128:(rank + 1) * 128], full[256 + rank * hd:256 + (rank + 1) * hd],
                              full[384 + rank * hd:384 + (rank + 1) * hd]])
            assert torch.equal(ls.qkv.shard.w_packed.view(-1, 128), want)
            assert ls.qkv.shard.out_features == 256 and ls.gate_up.shard.out_features == 512
            gu = lf.gate_up.shard.w_scale
            assert torch.equal(ls.gate_up.shard.w_scale, torch.cat([gu[rank * 256:(rank + 1) * 256], gu[512 + rank * 256:512 + (rank + 1) * 256]]))
            for name in ("o", "down"):
                ref = shard_row(getattr(lf, name).shard, rank, world)
                got = getattr(ls, name).shard
                assert torch.equal(got.w_packed, ref.w_packed) and torch.equal(got.w_scale, ref.w_scale)


def test_load_refuses_a_rotation_that_does_not_match_the_split(tmp_path):
    from flh_b200.checkpoint import load_quantized, save_quantized
    m = _tiny("token_asym")
    for layer in m.layers:
        layer.down.shard.full_hadamard_blocks = 1            # rotated over K as a whole
    save_quantized(m, str(tmp_path))
    load_quantized(str(tmp_path), device="cpu")
    with pytest.raises(ValueError, match="hadamard_blocks"):
        load_quantized(str(tmp_path), device="cpu", tp_rank=0, tp_world=2)


def test_reference_linear_accepts_the_saved_tensors(tmp_path):
    """The three tensors of one saved linear load into the reference's own LinearFLH (strict) and dequantise to the same weight."""
    import sys
    ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("FLH_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(ref, "flh", "nn")):
        pytest.skip("no FLH checkout (set FLH_REFERENCE)")
    sys.dont_write_bytecode = True
    if ref not in sys.path:
        sys.path.insert(0, ref)
    from flh.nn.linear import LinearFLH as RefLinear
    from flh_b200.checkpoint import save_quantized
    m = _tiny("group_sym")
    save_quantized(m, str(tmp_path))
    sd = torch.load(tmp_path / "model.pt", weights_only=False)
    pre = "model.layers.1.mlp.down_proj."
    rl = RefLinear(512, 256, bias=False, dtype=torch.float16, device="cpu", group_size=128)
    rl.load_state_dict({k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}, strict=True)
    ours = m.layers[1].down.shard.get_weight(torch.float32)
    assert torch.equal(rl.get_weight(torch.float32), ours)


def test_compress_i8_inverts_expand_layout():
    """The int8 copy kept for prefill GEMMs converts back to the packed checkpoint layout without loss."""
    from flh_b200.functional import compress_i8, expand_i4_reference
    g = torch.Generator().manual_seed(5)
    packed = torch.randint(0, 256, (24, 96), dtype=torch.uint8, generator=g)
    assert torch.equal(compress_i8(expand_i4_reference(packed)), packed)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["group_sym", "token_asym"])
def test_loaded_model_runs_like_the_saved_one(cuda, tmp_path, mode):
    from flh_b200.checkpoint import load_quantized, save_quantized
    m = _tiny(mode, "cuda")
    save_quantized(m, str(tmp_path))
    m = m.to("cuda")                     # save_quantized leaves the model where it was; make sure
    m2 = load_quantized(str(tmp_path), device="cuda")
    ids = torch.randint(0, 64, (2, 24), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    assert torch.equal(m(ids), m2(ids))


@pytest.mark.gpu
def test_conversion_on_the_gpu_matches_the_host_and_the_golden_buffers(cuda, golden):
    """Rotation (float64), RTN and packing run as torch kernels on the GPU give the same bits as on the host, and the
    same bits as the reference's LinearFLH.from_float (golden buffers)."""
    from helpers import rs
    from flh_b200.nn import LinearFLH
    from flh_b200._CUDA import expand_i4
    from flh_b200.functional import compress_i8
    w = (rs(401).standard_normal((64, 256)) * 0.02).astype(np.float32)
    lin = torch.nn.Linear(256, 64, bias=False)
    lin.weight.data = torch.from_numpy(w)
    fl = LinearFLH.from_float(lin.cuda(), weight_bits=4, weight_group_size=128, weight_sym=True, in_group_size=128)
    assert fl.w_packed.is_cuda
    assert np.array_equal(fl.w_packed.cpu().numpy().reshape(64, 128), golden["lin_w_packed"])
    assert np.array_equal(fl.w_scale.cpu().numpy(), golden["lin_w_scale"])
    # a larger layer with the full-width transform over two blocks (what a 2-way row-parallel down_proj needs)
    g = torch.Generator().manual_seed(9)
    big = torch.nn.Linear(7168, 256, bias=False)
    big.weight.data = torch.randn(256, 7168, generator=g) * 0.02
    host = LinearFLH.from_float(big.half(), weight_group_size=-1, full_hadamard=True, hadamard_blocks=2)
    dev = LinearFLH.from_float(big.half().cuda(), weight_group_size=-1, full_hadamard=True, hadamard_blocks=2)
    same = (dev.w_packed.cpu() == host.w_packed).float().mean().item()
    assert same > 0.9999 and torch.allclose(dev.w_scale.cpu().float(), host.w_scale.float(), rtol=1e-3)   # 28 x 28 factor: float64 matmul order
    # the int8 prefill copy converts back to the packed layout
    p2 = dev.w_packed.view(256, 3584)
    assert torch.equal(compress_i8(expand_i4(p2)), p2)
