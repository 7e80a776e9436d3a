"""Golden vectors for the GPTQ restatement, made by the reference's OWN code on CPU.

    python tests/golden/make_gptq_golden.py /path/to/FLH

Imports the unmodified flh/nn/gptq.py (FLHGPTQ) from the checkout with flh_b200._CUDA bound as flh._CUDA (the
calibration code itself never calls it on CPU tensors), feeds a small torch.nn.Linear and a few input batches through
add_batch + fasterquant for several configurations, and stores inputs and returned weights in gptq_golden.npz.

Only symmetric weights: with sym=False and static groups the reference's find_params divides xmin of shape
[rows, 1, 1] by a scale already reshaped to [rows, 1] (flh/nn/gptq.py:73-74), which broadcasts to a rows x rows table
of zero-points mixing the rows' scales; that table is not restated, so there is nothing to pin for it.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CONFIGS = [  # name, kwargs of fasterquant, group_size of add_batch
    ("sym_g128", dict(group_size=128, sym=True), 128),
    ("sym_channel", dict(group_size=-1, sym=True), -1),
    ("sym_g128_clip", dict(group_size=128, sym=True, clip_ratio=0.9), 128),
    ("sym_g128_actorder", dict(group_size=128, sym=True, actorder=True), 128),
    ("sym_g128_block64", dict(group_size=128, sym=True, blocksize=64), 128),
]


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLH_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "flh", "nn")):
        raise SystemExit("usage: make_gptq_golden.py /path/to/FLH   (or set FLH_REFERENCE)")
    sys.dont_write_bytecode = True
    sys.path.insert(0, ROOT)
    sys.path.insert(0, ref)
    import flh_b200
    flh_b200._CUDA.install()
    from flh.nn.gptq import FLHGPTQ

    rows, cols, tokens, nbatch = 32, 256, 256, 2     # twice as many tokens as columns: a well-conditioned Hessian
    g = torch.Generator().manual_seed(1234)
    weight = (torch.randn(rows, cols, generator=g) * 0.05).half().float()
    weight[:, 7] *= 6.0                                   # an outlier column, as rotated LLM weights still have a few
    # inputs with correlated features, so that the Hessian is far from diagonal and error feedback matters
    mix = torch.randn(cols, cols, generator=g) * 0.15 + torch.eye(cols)
    # stored as int8 sixteenths (exact in float32), which keeps the fixture small
    batches = [torch.clamp(torch.round((torch.randn(tokens, cols, generator=g) @ mix) * 16), -127, 127) / 16 for _ in range(nbatch)]
    out = {"weight": weight.numpy(), "batches_x16": np.stack([(b * 16).numpy() for b in batches]).astype(np.int8)}
    for name, kw, gs in CONFIGS:
        layer = torch.nn.Linear(cols, rows, bias=False)
        layer.weight.data = weight.clone()
        gq = FLHGPTQ(layer)
        for b in batches:
            gq.add_batch(b.unsqueeze(0), None, group_size=gs)
        out[f"Hs_{name}"] = gq.H[::16, ::16].clone().numpy()          # a 16 x 16 sample pins the Hessian
        gq.fasterquant(**kw)
        out[f"Q_{name}"] = layer.weight.data.float().numpy()
    np.savez_compressed(os.path.join(HERE, "gptq_golden.npz"), **out)
    print("wrote gptq_golden.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
