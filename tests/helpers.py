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


def token_codes_mismatch(q, s, z, qo, so, zo):
    """Compares a per-token quantiser result (torch tensors) with the oracle's (numpy): returns (rate, max code
    difference, max scale difference in f16 ulps, max zero-point difference), the rate taken over ALL codes of ALL
    rows (rows whose scale or zero-point moved included)."""
    from oracle import oracle as O
    c = O.unpack_i4(q.cpu().numpy(), False).astype(np.int32)
    co = O.unpack_i4(qo, False).astype(np.int32)
    d = np.abs(c - co)
    sd = np.abs(s.cpu().numpy().view(np.uint16).astype(np.int32) - so.view(np.uint16).astype(np.int32))
    zd = np.abs(z.cpu().numpy().astype(np.float32) - zo.astype(np.float32))
    return float((d != 0).mean()), int(d.max()), int(sd.max()), float(zd.max())


def assert_token_tolerance(q, s, z, qo, so, zo, max_rate=1e-3):
    """The stated bound when the transform is not summed in the reference's order: at most 0.1 % of all codes
    differ, by one step; scales within one f16 ulp, zero-points within one."""
    rate, dmax, sd, zd = token_codes_mismatch(q, s, z, qo, so, zo)
    assert dmax <= 1 and sd <= 1 and zd <= 1 and rate <= max_rate, (rate, dmax, sd, zd)
    return rate
