"""The Llama-shaped W4A4 decoder on the CUDA kernels against its PyTorch twin (forward_origin /
forward_torch on the same packed weights), and the KV-cache decode step against the prefill."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _twin(monkeypatch):
    from flh_b200.nn import ActQuantizer, LinearFLH
    monkeypatch.setattr(ActQuantizer, "forward", lambda self, x: ActQuantizer.forward_origin(self, x))
    monkeypatch.setattr(LinearFLH, "forward",
                        lambda self, x, a_scale=None, a_zero=None, **kw: LinearFLH.forward_torch(self, x, a_scale, a_zero).half())


@pytest.mark.parametrize("mode", ["group_sym", "token_asym"])
def test_decoder_matches_pytorch_twin(cuda, monkeypatch, mode):
    from flh_b200.model import Decoder, DecoderConfig
    cfg = DecoderConfig(hidden=256, n_heads=4, n_kv_heads=2, ffn=512, n_layers=2, vocab=128, act_mode=mode)
    m = Decoder(cfg, torch.device("cuda"), seed=3)
    ids = torch.randint(0, 128, (2, 40), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    y = m(ids).float()
    with monkeypatch.context() as mp:
        _twin(mp)
        m.cfg.fuse_glue = False                      # the twin run uses PyTorch tensor operations for rope / KV / SiLU * up too
        y_ref = m(ids).float()
        m.cfg.fuse_glue = True
    # whole-model tolerance: 3 % of the logit scale (f16 accumulation, and the rare activation code that
    # flips by one step between the binary16/binary32 kernels and the float64/float32 twins; which codes
    # flip depends on the low bits of torch's attention output, so the figure moves between 1.5 and 2.2 %)
    err = (y - y_ref).abs().max() / y_ref.abs().max()
    assert err < 3e-2, err


def test_decode_step_matches_prefill(cuda):
    from flh_b200.model import Decoder, DecoderConfig
    cfg = DecoderConfig(hidden=256, n_heads=4, n_kv_heads=4, ffn=512, n_layers=2, vocab=128, act_mode="group_sym")
    m = Decoder(cfg, torch.device("cuda"), seed=5)
    ids = torch.randint(0, 128, (3, 17), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    full = m(ids).float()                              # logits of the last position, no cache
    cache = m.new_cache(3, 32)
    m(ids[:, :16], cache=cache, start=0)
    step = m(ids[:, 16:], cache=cache, start=16).float()
    err = (full - step).abs().max() / full.abs().max()
    assert err < 2e-2, err


@pytest.mark.parametrize("mode", ["group_sym", "token_asym"])
def test_llama7b_shaped_layer_matches_pytorch_twin(cuda, monkeypatch, mode):
    """One decoder layer at the Llama-2-7B shape (hidden 4096, 32 heads, FFN 11008 -> merged QKV at N = 12288, the
    tensor-core transform in front of down_proj, 256 tokens) against its PyTorch twin (forward_origin / forward_torch and
    tensor operations for rope, SiLU * up) on the same packed weights.
    Tolerance.  The twins are not bit-level models of the kernels: forward_origin transforms in float64 and quantises
    against an un-rounded binary32 scale, the kernels against the f16 scale they store, so by construction 2-5e-4 of the
    activation codes differ by one step (tests/test_oracle_golden.py measures that rate against the reference's own
    functions).  One such flip moves one of the K terms of a dot product by one quantisation step, about
    0.5 sigma_x * |w|; against an output of standard deviation sqrt(K) sigma_x sigma_w with |w| / sigma_w <= 1.7 for
    uniform int4 codes that is 0.5 * 1.7 / sqrt(4096) = 1.3 % of the output's standard deviation, i.e. about 0.3 % of
    max |y| per flip per output; a row of 4096 ... 11008 activations carries 2 to 5 flips per linear, the layer chains three
    quantised linears and an attention, and the maximum is taken over a million outputs: a few percent of max |y| at
    the worst output, while the error over all outputs (relative Frobenius norm) stays near 1e-3.  Measured on B200:
    max-norm 1.0e-2 (group_sym) and 2.6e-2 (token_asym).  Bounds used: 5 % of max |y| at the worst output, 1 % in
    Frobenius norm."""
    from flh_b200.model import Decoder, DecoderConfig
    cfg = DecoderConfig(hidden=4096, n_heads=32, n_kv_heads=32, ffn=11008, n_layers=1, vocab=512, act_mode=mode)
    m = Decoder(cfg, torch.device("cuda"), seed=11, with_head=False)
    ids = torch.randint(0, 512, (2, 128), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    y = m(ids).float()
    with monkeypatch.context() as mp:
        _twin(mp)
        m.cfg.fuse_glue = False
        m.cfg.fuse_norm = False
        y_ref = m(ids).float()
    err = ((y - y_ref).abs().max() / y_ref.abs().max()).item()
    fro = ((y - y_ref).norm() / y_ref.norm()).item()
    print(f"{mode}: max |y - y_twin| / max |y_twin| = {err:.2e}, Frobenius {fro:.2e}")
    assert err < 5e-2 and fro < 1e-2, (err, fro)
