"""CPU restatement of the reference's GPTQ weight calibration (flh/nn/gptq.py), TEST INFRASTRUCTURE ONLY: the
checker for flh_b200.gptq and the library's flh_b200_gptq_block kernel.  Nothing in the product imports this file.

Pinned against the reference's own code: tests/golden/gptq_golden.npz holds inputs and the weights that the
unmodified FLHGPTQ.fasterquant (run on CPU by tests/golden/make_gptq_golden.py) returned for them.

The column sweep is written with numpy float32 scalars-per-column so that every product, difference and quotient is
rounded exactly where the reference's torch expressions round them (flh/nn/gptq.py:207-228); the dense linear algebra
(Cholesky factorisations, the update of the columns right of a block) uses torch's CPU routines, the same ones the
reference calls.
"""
import numpy as np
import torch


def clip_weight(W, groupsize, clip_ratio):
    """flh/nn/gptq.py:40-50"""
    if clip_ratio >= 1.0:
        return W
    if groupsize > 0 and W.shape[1] % groupsize == 0:
        Wg = W.reshape(W.shape[0], -1, groupsize)
        cv = (np.abs(Wg).max(axis=2, keepdims=True) * np.float32(clip_ratio)).astype(np.float32)
        return np.clip(Wg, -cv, cv).reshape(W.shape)
    cv = (np.abs(W).max(axis=1, keepdims=True) * np.float32(clip_ratio)).astype(np.float32)
    return np.clip(W, -cv, cv)


def find_params(W, bits, groupsize, sym, clip_ratio):
    """flh/nn/gptq.py:52-96 -> (scale, zero), float32 [rows, groups] (one column when per channel)."""
    W = clip_weight(W.astype(np.float32), groupsize, clip_ratio)
    maxq = np.float32(2 ** (bits - 1) - 1 if sym else 2 ** bits - 1)
    if groupsize > 0 and W.shape[1] % groupsize == 0:
        Wg = W.reshape(W.shape[0], -1, groupsize)
        if sym:
            xmax = np.maximum(np.abs(Wg).max(axis=2), np.float32(1e-5))
            scale = (xmax / maxq).astype(np.float32)
            return scale, np.zeros_like(scale)
        xmax, xmin = Wg.max(axis=2), Wg.min(axis=2)
    else:
        xmin, xmax = W.min(axis=1, keepdims=True), W.max(axis=1, keepdims=True)
        if sym:
            xmax = np.maximum(np.maximum(np.abs(xmax), np.abs(xmin)), np.float32(1e-5))
            scale = (xmax / maxq).astype(np.float32)
            return scale, np.zeros_like(scale)
    both = (xmin == 0) & (xmax == 0)
    xmin = np.where(both, np.float32(-1.0), xmin).astype(np.float32)
    xmax = np.where(both, np.float32(1.0), xmax).astype(np.float32)
    scale = np.maximum(((xmax - xmin) / maxq).astype(np.float32), np.float32(1e-5))
    zero = np.rint((-xmin / scale).astype(np.float32)).astype(np.float32)
    return scale, zero


def quantize_col(w, scale, zero, maxq, sym, clip_ratio):
    """flh/nn/gptq.py:9-24, 98-109 for one column: w, scale, zero are float32 [rows]."""
    x = w
    if clip_ratio < 1.0:
        cv = (scale * np.float32(maxq)).astype(np.float32) * np.float32(clip_ratio)
        x = np.clip(x, -cv, cv)
    if sym:
        q = np.clip(np.rint((x / scale).astype(np.float32)), -(maxq + 1), maxq).astype(np.float32)
        return (scale * q).astype(np.float32)
    q = np.clip(np.rint(((x / scale).astype(np.float32) + zero).astype(np.float32)), 0, maxq).astype(np.float32)
    return (scale * (q - zero).astype(np.float32)).astype(np.float32)


def block_sweep(W1, Hinv1, scale, zero, group_of_col, maxq, sym, clip_ratio):
    """The loop over the columns of one block (flh/nn/gptq.py:207-228): returns (Q1, Err1); W1 is not modified."""
    W1 = W1.astype(np.float32).copy()
    Hinv1 = Hinv1.astype(np.float32)
    rows, count = W1.shape
    Q1, Err1 = np.zeros_like(W1), np.zeros_like(W1)
    for i in range(count):
        w = W1[:, i].copy()
        d = Hinv1[i, i]
        g = int(group_of_col[i])
        q = quantize_col(w, scale[:, g], zero[:, g], maxq, sym, clip_ratio)
        Q1[:, i] = q
        err = ((w - q).astype(np.float32) / d).astype(np.float32)
        # rank-1 update of the columns from i on: a rounded product, then a rounded difference
        W1[:, i:] = (W1[:, i:] - (err[:, None] * Hinv1[i, i:][None, :]).astype(np.float32)).astype(np.float32)
        Err1[:, i] = err
    return Q1, Err1


def rotate(x, group_size):
    """fast_hadamard_transform on CPU tensors (flh/nn/quantization.py:129-138): float64 Hadamard of every group of
    `group_size` columns (the whole row when group_size <= 0), divided by sqrt(n), returned as float32."""
    from oracle import fake_quant_port as FQ
    x = np.asarray(x, dtype=np.float64)
    n = group_size if group_size and group_size > 0 and x.shape[-1] % group_size == 0 else x.shape[-1]
    H = FQ.hadamard_matrix(n, dtype=torch.float64).numpy() * np.sqrt(n)          # entries +-1
    y = (x.reshape(-1, n) @ H.T) / np.sqrt(float(n))
    return y.reshape(x.shape).astype(np.float32)


def hessian(batches, group_size):
    """FLHGPTQ.add_batch (flh/nn/gptq.py:124-139) over a list of [tokens, columns] float32 arrays that are ALREADY
    Hadamard-rotated; float32 torch CPU arithmetic."""
    cols = batches[0].shape[1]
    H = torch.zeros((cols, cols), dtype=torch.float32)
    n = 0
    for b in batches:
        inp = torch.from_numpy(np.ascontiguousarray(b, dtype=np.float32)).t()
        tmp = b.shape[0]
        H *= n / (n + tmp)
        n += tmp
        inp = float(np.sqrt(2 / n)) * inp
        H += inp.matmul(inp.t())
    return H.numpy()


def fasterquant(W, H, group_size=128, blocksize=128, percdamp=0.01, actorder=False, sym=True, bits=4, clip_ratio=1.0):
    """FLHGPTQ.fasterquant (flh/nn/gptq.py:141-237) from the rotated weights W and the Hessian H (float32 arrays)."""
    W = W.astype(np.float32).copy()
    H = torch.from_numpy(H.astype(np.float32).copy())
    rows, columns = W.shape
    group_size = group_size if group_size > 0 and columns % group_size == 0 else -1
    maxq = 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead.numpy()] = 0
    W = clip_weight(W, group_size, clip_ratio)
    if group_size > 0:
        parts = [find_params(W[:, i:i + group_size], bits, group_size, sym, clip_ratio) for i in range(0, columns, group_size)]
        scale = np.concatenate([p[0] for p in parts], axis=1)
        zero = np.concatenate([p[1] for p in parts], axis=1)
    else:
        scale, zero = find_params(W, bits, -1, sym, clip_ratio)
    cols = np.arange(columns)
    if actorder:
        perm = torch.argsort(torch.diag(H), descending=True)
        W = W[:, perm.numpy()]
        H = H[perm][:, perm]
        invperm = torch.argsort(perm).numpy()
        cols = perm.numpy()
    group_of_col = cols // group_size if group_size > 0 else np.zeros_like(cols)
    damp = percdamp * torch.mean(torch.diag(H))
    diag = torch.arange(columns)
    H[diag, diag] += damp
    H = torch.linalg.cholesky(H)
    H = torch.cholesky_inverse(H)
    Hinv = torch.linalg.cholesky(H, upper=True)
    Q = np.zeros_like(W)
    for i1 in range(0, columns, blocksize):
        i2 = min(i1 + blocksize, columns)
        Q1, Err1 = block_sweep(W[:, i1:i2], Hinv[i1:i2, i1:i2].numpy(), scale, zero, group_of_col[i1:i2], maxq, sym, clip_ratio)
        Q[:, i1:i2] = Q1
        if i2 < columns:
            W[:, i2:] = (torch.from_numpy(W[:, i2:].copy()) - torch.from_numpy(Err1).matmul(Hinv[i1:i2, i2:])).numpy()
    if actorder:
        Q = Q[:, invperm]
    return Q, scale, zero


def proxy_loss(W, Q, H):
    """tr((W - Q) H (W - Q)^T): the layer-output error GPTQ minimises, in float64."""
    D = (W.astype(np.float64) - Q.astype(np.float64))
    return float(np.einsum("ij,jk,ik->", D, H.astype(np.float64), D))
