"""The CPU restatement of the reference's GPTQ calibration (oracle/gptq_oracle.py) against golden vectors made by
the reference's own FLHGPTQ on CPU (tests/golden/make_gptq_golden.py)."""
import os

import numpy as np
import pytest

from oracle import gptq_oracle as G

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gptq_golden.npz")

CONFIGS = {  # name -> (kwargs of fasterquant, group_size of add_batch)
    "sym_g128": (dict(group_size=128, sym=True), 128),
    "sym_channel": (dict(group_size=-1, sym=True), -1),
    "sym_g128_clip": (dict(group_size=128, sym=True, clip_ratio=0.9), 128),
    "sym_g128_actorder": (dict(group_size=128, sym=True, actorder=True), 128),
    "sym_g128_block64": (dict(group_size=128, sym=True, blocksize=64), 128),
}


def golden_batches(z):
    return [b.astype(np.float32) / np.float32(16.0) for b in z["batches_x16"]]       # stored as int8 sixteenths


def golden_case(name):
    z = np.load(GOLD)
    kw, gs = CONFIGS[name]
    batches = [G.rotate(b, gs) for b in golden_batches(z)]
    W = G.rotate(z["weight"], kw["group_size"])
    return z, kw, W, G.hessian(batches, gs)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_oracle_reproduces_the_reference(name):
    z, kw, W, H = golden_case(name)
    assert np.array_equal(H[::16, ::16], z[f"Hs_{name}"]), "Hessian of the rotated inputs"
    Q, _, _ = G.fasterquant(W, H, **kw)
    assert np.array_equal(Q.view(np.uint32), z[f"Q_{name}"].view(np.uint32)), \
        f"{(Q != z[f'Q_{name}']).sum()} of {Q.size} weights differ from the reference's"


def test_error_feedback_beats_round_to_nearest():
    z, kw, W, H = golden_case("sym_g128")
    Q, scale, zero = G.fasterquant(W, H, **kw)
    rtn = np.concatenate([G.quantize_col(W[:, j], scale[:, j // 128], zero[:, j // 128], 7, True, 1.0)[:, None]
                          for j in range(W.shape[1])], axis=1)
    assert G.proxy_loss(W, Q, H) < 0.8 * G.proxy_loss(W, rtn, H)
