"""Import the upstream QTIP python sources on CPU so golden vectors can be generated.

Only usable on a machine that has the upstream tree checked out (path in the
QTIP_REFERENCE_ROOT environment variable).  Nothing in the test-suite, the smoke
check or the benchmark imports this module: it is used by make_golden.py (fixture
generation) and by oracle/check_against_reference.py (oracle pinning) only.

Three third-party modules the upstream code imports are missing on a CPU-only
machine and are replaced by minimal stand-ins before the import:
  * qtip_kernels            - only touched inside CUDA op bodies; an empty module is enough
  * glog                    - logging; info/warning mapped to print
  * fast_hadamard_transform - hadamard_transform(x, scale): Sylvester-ordered
                              Walsh-Hadamard transform over the last dim times `scale`
"""
import os
import sys
import types

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch  # noqa: E402


def _fwht_last_dim(x, scale=1.0):
    n = x.shape[-1]
    assert n & (n - 1) == 0, "power of two only"
    y = x.clone().reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        a = y[:, :, 0, :] + y[:, :, 1, :]
        b = y[:, :, 0, :] - y[:, :, 1, :]
        y = torch.stack((a, b), dim=2).reshape(-1, n)
        h *= 2
    return (y * scale).reshape(x.shape)


def load_reference(root=None):
    root = root or os.environ.get("QTIP_REFERENCE_ROOT")
    if not root:
        raise RuntimeError("set QTIP_REFERENCE_ROOT to a checkout of the upstream QTIP repository")
    if not os.path.isdir(os.path.join(root, "lib", "codebook")):
        raise RuntimeError(f"upstream QTIP tree not found at {root}")
    if "qtip_kernels" not in sys.modules:
        sys.modules["qtip_kernels"] = types.ModuleType("qtip_kernels")
    if "glog" not in sys.modules:
        g = types.ModuleType("glog")
        g.info = g.warning = g.error = print
        sys.modules["glog"] = g
    if "fast_hadamard_transform" not in sys.modules:
        f = types.ModuleType("fast_hadamard_transform")
        f.hadamard_transform = _fwht_last_dim
        sys.modules["fast_hadamard_transform"] = f
    if root not in sys.path:
        sys.path.insert(0, root)
    import lib.codebook.bitshift as bitshift
    import lib.utils.kernel_decompress as kernel_decompress
    import lib.utils.matmul_had as matmul_had
    import lib.algo.ldlq as ldlq
    return types.SimpleNamespace(bitshift=bitshift, kernel_decompress=kernel_decompress,
                                 matmul_had=matmul_had, ldlq=ldlq, root=root)
