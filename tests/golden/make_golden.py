"""Generate the golden vectors under tests/golden/ from the FLH reference itself.

Run where the FLH checkout is readable (it is imported, never modified):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/FLH

Every array written here is an OUTPUT of reference code (the PyTorch twins of the
CUDA path and the fake_quant pipeline) on seeded inputs.  Inputs are regenerated
at test time from the same seeds with numpy's frozen RandomState generator (or
torch.manual_seed for the one case that follows a reference script's own
seeding), so only outputs are stored.
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def rs(seed):
    return np.random.RandomState(seed)


def activations(seed, m, k, outlier_frac=0.001, dtype=np.float16):
    """N(0,1) activations with a fraction of channels scaled x20 (the benchmark's input law)."""
    r = rs(seed)
    x = r.standard_normal((m, k)).astype(np.float32)
    n_out = max(1, int(round(k * outlier_frac)))
    ch = r.choice(k, n_out, replace=False)
    x[:, ch] *= 20.0
    return x.astype(dtype)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main(ref_root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "fake_quant"))
    import flh  # noqa
    from flh.nn.quantization import ActQuantizer, fast_hadamard_transform
    from flh.nn.linear import LinearFLH
    from flh.functional.hadamard import matmul_hadU
    from flh.functional.quantization import pack_i4, unpack_i4
    import quant_utils as fq  # fake_quant/quant_utils.py
    import hadamard_utils as fh  # fake_quant/hadamard_utils.py

    torch.set_num_threads(4)
    out = {}

    # --- (1) ActQuantizer.forward_origin, symmetric group-128, binary16 input -----------
    x = activations(101, 24, 512)
    xt = torch.from_numpy(x)
    for had in (False, True):
        aq = ActQuantizer(bits=4, group_size=128, sym=True, use_hadamard=had, packed_output=True)
        scale, zp, q = aq.forward_origin(xt)
        tag = "had" if had else "nohad"
        out[f"aq_sym_{tag}_scale"] = scale.numpy()
        out[f"aq_sym_{tag}_q"] = q.numpy()
    # --- (2) fast_hadamard_transform (binary64 path), group 128 -------------------------
    out["fht128_f64"] = fast_hadamard_transform(xt.double(), group_size=128).numpy()

    # --- (3) matmul_hadU in binary32 ----------------------------------------------------
    for n, m in ((4096, 3), (8192, 2), (11008, 2), (14336, 2), (28672, 1), (3584, 2), (1536, 2)):
        xi = activations(200 + n % 97, m, n).astype(np.float32)
        y = matmul_hadU(torch.from_numpy(xi)).numpy()
        out[f"hadU_{n}"] = y

    # --- (4) fake_quant per-token asymmetric quantiser on the transformed activations ---
    for n, m in ((4096, 4), (11008, 2), (14336, 2)):
        xi = activations(300 + n % 97, m, n)                        # binary16 input
        y = matmul_hadU(torch.from_numpy(xi).float())
        aq = fq.ActQuantizer()
        aq.configure(bits=4, groupsize=-1, sym=False, clip_ratio=1.0)
        aq.find_params(y)
        q32, s32, z32 = aq.quantizer(y)                              # pure reference (binary32 scale)
        out[f"fq_{n}_scale32"] = s32[:, 0].numpy()
        out[f"fq_{n}_zero32"] = z32[:, 0].numpy()
        out[f"fq_{n}_q32"] = pack_nib(q32.numpy())
        # the same reference functions evaluated with the scale rounded to binary16 first
        sh = s32[:, :1].half().float()
        xmin = torch.minimum(y.min(1)[0], torch.zeros(y.shape[0]))
        xmax = torch.maximum(y.max(1)[0], torch.zeros(y.shape[0]))
        assert not bool(((xmin == 0) & (xmax == 0)).any())
        zh = torch.round(-xmin[:, None] / sh)
        qh, _, _ = fq.asym_quant(y, sh, zh, aq.maxq)
        out[f"fq_{n}_scale16"] = sh[:, 0].half().numpy()
        out[f"fq_{n}_zero16"] = zh[:, 0].numpy()
        out[f"fq_{n}_q16"] = pack_nib(qh.numpy())

    # --- (5) LinearFLH.from_float buffers and forward_torch -----------------------------
    r = rs(401)
    lin = torch.nn.Linear(256, 64, bias=False)
    w = (r.standard_normal((64, 256)) * 0.02).astype(np.float32)
    lin.weight.data = torch.from_numpy(w)
    fl = LinearFLH.from_float(lin, weight_bits=4, weight_group_size=128, weight_sym=True,
                              in_group_size=128)
    out["lin_w_packed"] = fl.w_packed.numpy().reshape(64, 128)
    out["lin_w_scale"] = fl.w_scale.numpy()
    out["lin_w_had"] = fast_hadamard_transform(torch.from_numpy(w), group_size=128).numpy()
    xq = r.randint(-8, 8, size=(5, 256)).astype(np.int64)
    xs = (r.uniform(0.005, 0.02, size=(5, 2))).astype(np.float16)
    xqp = pack_i4(torch.from_numpy(xq).int())
    assert torch.equal(unpack_i4(xqp).long(), torch.from_numpy(xq))
    # a_zero=None trips an attribute error inside the twin's group branch; zeros are equivalent
    y = fl.forward_torch(xqp, a_scale=torch.from_numpy(xs).float(), a_zero=torch.zeros(5, 2), x_is_packed=True,
                         is_symmetric=True)
    out["lin_fwd_torch"] = y.numpy()
    out["lin_x_packed"] = xqp.numpy()

    # --- (6) the CPU-runnable benchmark configuration: CPU fake-quant linear, seed 0 ---------------------------
    torch.manual_seed(0)
    X = torch.randn(16, 4096)
    ch = torch.randperm(4096)[:8]
    X[:, ch] *= 20.0
    W = torch.randn(4096, 4096) * 0.02
    H = fh.get_hadamard_matrix(4096, device="cpu")
    lin = torch.nn.Linear(4096, 4096, bias=False)
    wq = fq.WeightQuantizer()
    wq.configure(4, perchannel=True, sym=True, mse=False)
    Wr = (W.double() @ H.double()).float()
    wq.find_params(Wr)
    lin.weight.data = wq.quantize(Wr)
    wrap = fq.ActQuantWrapper(lin)
    wrap.quantizer.configure(bits=4, groupsize=-1, sym=False, clip_ratio=1.0)
    wrap.online_had = True
    wrap.fp32_had = True
    wrap.group_size = 0            # matmul_had_cuda(x, group_size): <= 0 selects the full matrix

    def had_cpu(x, group_size):
        return x @ H.to(x.dtype)
    fh_matmul = fh.matmul_had_cuda
    fh.matmul_had_cuda = had_cpu   # the stock helper builds its matrix on cuda:0
    try:
        with torch.no_grad():
            Y = wrap(X)
    finally:
        fh.matmul_had_cuda = fh_matmul
    out["cfg1_Y"] = Y.numpy()
    out["cfg1_w_scale"] = wq.scale[:, 0].numpy()
    out["cfg1_sha_X"] = np.frombuffer(bytes.fromhex(sha(X.numpy())), dtype=np.uint8)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote golden.npz:", os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes;", len(out), "arrays")


def pack_nib(q):
    q = q.astype(np.int64)
    return ((q[:, 0::2] & 15) | ((q[:, 1::2] & 15) << 4)).astype(np.uint8)


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("FLH_REFERENCE"):
        raise SystemExit("usage: %s <FLH checkout>   (or set FLH_REFERENCE)" % sys.argv[0])
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["FLH_REFERENCE"])
