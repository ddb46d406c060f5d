"""torch.library ops quip_lib::decompress_matvec_qtip_{m}_1_{n}_{K}, the op boundary of
lib/codebook/__init__.py:68-93 upstream (schema `(Tensor compressed, Tensor x, Tensor codebook) -> Tensor`,
fake implementation returning zeros (1, m) fp32, CUDA implementation calling the kernel).

Upstream binds 61 fixed (m, n, K) triples; here any triple can be registered, the upstream table is
registered by `register_upstream_table()`.  If upstream's own lib.codebook has already defined an op
(it does so on import, on top of qtip_b200.qtip_kernels) the existing definition is kept.
"""
import torch

from . import ops

# (m, n, K) of lib/codebook/__init__.py:4-66 upstream, written as shape families x bit rates
UPSTREAM_TABLE = sorted(set(
    [(m, n, 4) for (m, n) in ((1024, 3072), (8192, 3072), (3072, 8192), (3072, 3072))] +
    [(m, n, K) for K in (2, 3, 4) for (m, n) in (
        (53248, 16384), (16384, 53248), (1024, 16384), (16384, 16384), (4096, 14336), (14336, 4096), (1024, 4096),
        (4096, 4096), (4096, 11008), (11008, 4096), (12288, 4096), (22016, 4096), (8192, 8192), (10240, 8192),
        (57344, 8192), (8192, 1024), (8192, 28672), (28672, 8192), (1024, 8192))]))

_registered = set()


def op_name(m, n, K):
    return f"decompress_matvec_qtip_{m}_1_{n}_{K}"


def register(m, n, K):
    """Define quip_lib::decompress_matvec_qtip_{m}_1_{n}_{K} (idempotent).  Returns the op."""
    name = op_name(m, n, K)
    if (m, n, K) not in _registered and not hasattr(torch.ops.quip_lib, name):
        torch.library.define(f"quip_lib::{name}", "(Tensor compressed, Tensor x, Tensor codebook) -> Tensor")

        @torch.library.register_fake(f"quip_lib::{name}")
        def _fake(compressed, x, codebook):
            return torch.zeros(1, m, dtype=torch.float32, device=x.device)

        @torch.library.impl(f"quip_lib::{name}", "cuda")
        def _cuda(compressed, x, codebook):
            out = torch.empty((1, m), dtype=torch.float32, device=x.device)
            ops.decompress_matvec(compressed, x.reshape(1, n).to(torch.float16), codebook, K, m, n, out=out)
            return out
    _registered.add((m, n, K))
    return getattr(torch.ops.quip_lib, name)


def register_upstream_table():
    for (m, n, K) in UPSTREAM_TABLE:
        register(m, n, K)
    return len(UPSTREAM_TABLE)
