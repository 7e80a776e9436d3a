"""Extract the non-power-of-two Hadamard factor matrices used by get_hadK
(flh/functional/hadamard.py:39-89) into a compact data file.

The matrices are third-party data (N. J. A. Sloane's library of Hadamard
matrices, vendored in the FLH repository).  They are not retyped: this script
imports the FLH module, checks that every matrix is a +-1 Hadamard matrix, and
stores the sign bits (1 = -1) with numpy.packbits, row-major, one array per
order.  Run it with the FLH checkout on the command line:

    python flh_b200/data/make_hadk_tables.py /path/to/FLH
"""
import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import flh.functional.hadamard as H  # noqa: E402

    out = {}
    for k in (12, 20, 28, 36, 40, 52, 60, 108, 140, 156, 172):
        m = getattr(H, f"get_had{k}")().numpy()
        assert m.shape == (k, k) and np.all(np.abs(m) == 1)
        assert np.array_equal(m @ m.T, k * np.eye(k)), f"had{k} is not Hadamard"
        out[f"had{k}"] = np.packbits((m < 0).astype(np.uint8).reshape(-1))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hadk_signs.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("FLH_REFERENCE"):
        raise SystemExit("usage: %s <FLH checkout>   (or set FLH_REFERENCE)" % sys.argv[0])
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["FLH_REFERENCE"])
