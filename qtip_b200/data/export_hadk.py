"""Export the small +-1 Hadamard matrices used for n = K * 2^p layer widths.

The factor matrices (orders 12 ... 172) are data of the upstream project
(lib/utils/matmul_had.py:129 onwards, taken there from N. J. A. Sloane's Hadamard library);
a layer quantized upstream can only be evaluated with exactly these matrices, so they are
exported once, bit-packed (1 = +1, 0 = -1, row-major, numpy packbits order), into hadk.npz
beside this script.  Needs the upstream tree:
    QTIP_REFERENCE_ROOT=/path/to/qtip python qtip_b200/data/export_hadk.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "tests", "golden"))
from _reference_import import load_reference  # noqa: E402


def main():
    mh = load_reference().matmul_had
    out = {}
    for k in (12, 20, 28, 36, 52, 60, 108, 116, 124, 140, 156, 172):
        h = getattr(mh, f"get_had{k}")().numpy()
        assert h.shape == (k, k) and np.all(np.abs(h) == 1)
        assert np.array_equal(h @ h.T, k * np.eye(k)), k
        out[f"had{k}"] = np.packbits((h > 0).astype(np.uint8).reshape(-1))
    np.savez_compressed(os.path.join(HERE, "hadk.npz"), **out)
    print({k: v.size for k, v in out.items()})


if __name__ == "__main__":
    main()
