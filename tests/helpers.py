"""Seeded synthetic inputs shared by the tests (numpy's frozen RandomState generator)."""
import numpy as np


def rs(seed):
    return np.random.RandomState(seed)


def activations(seed, m, k, outlier_frac=0.001, dtype=np.float16):
    """N(0,1) activations with a fraction of channels scaled x20 (same law as tests/golden/make_golden.py)."""
    r = rs(seed)
    x = r.standard_normal((m, k)).astype(np.float32)
    n_out = max(1, int(round(k * outlier_frac)))
    ch = r.choice(k, n_out, replace=False)
    x[:, ch] *= 20.0
    return x.astype(dtype)


def int4_codes(seed, rows, k, unsigned=False):
    r = rs(seed)
    return r.randint(0, 16, size=(rows, k)) if unsigned else r.randint(-8, 8, size=(rows, k))


def scales(seed, rows, cols, lo=0.005, hi=0.02):
    return rs(seed).uniform(lo, hi, size=(rows, cols)).astype(np.float16)
