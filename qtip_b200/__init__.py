"""qtip_b200: B200-native (sm_100a) kernels for the QTIP quantized-linear path.

Python mirrors of the upstream interfaces live in
  qtip_b200.bitshift          BitshiftLinear            (lib/codebook/bitshift.py upstream)
  qtip_b200.quantized_linear  QuantizedLinear           (lib/linear/quantized_linear.py)
  qtip_b200.qtip_kernels      decompress_matvec_16_9_*  (the `qtip_kernels` extension)
  qtip_b200.ops               tensor-level wrappers over the C ABI in include/qtip_b200.h
"""
import sys


def install_as_qtip_kernels():
    """Make `import qtip_kernels` resolve to the shim in this package."""
    from . import qtip_kernels
    sys.modules["qtip_kernels"] = qtip_kernels
    return qtip_kernels
