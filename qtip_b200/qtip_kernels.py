"""Stand-in for the upstream `qtip_kernels` extension module.

Upstream binds 64 fixed-shape functions decompress_matvec_16_9_{R}_1_{M}_1_{K}(out, compressed, x,
codebook) (qtip-kernels/src/wrapper.cpp:489-564, definitions qtip-kernels/src/qtip_torch.cu:60-671)
and lib/codebook/__init__.py:85-92 calls them by name.  Here any such name resolves, on attribute
access, to a closure over the one shape-generic kernel, so upstream's op registration works
unmodified once this module is importable as `qtip_kernels`:

    import qtip_b200; qtip_b200.install_as_qtip_kernels()   # before `import lib.codebook`

Argument contract (same as upstream): out fp32 (M, 1) written in place on the current stream,
compressed int32 (R*M*K/32,), x fp16 (K, 1), codebook fp16 (1024,).  Violations raise RuntimeError
(upstream: TORCH_CHECK); a failed launch raises instead of terminating the process.
"""
import re

import torch

from . import ops

_NAME = re.compile(r"^decompress_matvec_(\d+)_(\d+)_(\d+)_(\d+)_(\d+)_(\d+)_(\d+)$")
_cache = {}


def _make(L, S, R, V, M, N, K):
    if (L, S, V, N) != (16, 9, 1, 1) or R not in (2, 3, 4) or M % 32 or K % 32:
        raise AttributeError(f"no kernel for L={L} S={S} R={R} V={V} M={M} N={N} K={K}")

    def fn(out, compressed, x, codebook):
        for name, t in (("out", out), ("compressed", compressed), ("x", x), ("codebook", codebook)):
            if not (t.is_cuda and t.is_contiguous()):
                raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
        if out.dim() != 2 or out.dtype != torch.float32 or out.shape[0] != M:
            raise RuntimeError(f"out must be float32 ({M}, 1)")
        if compressed.dim() != 1 or compressed.dtype != torch.int32 or compressed.numel() * 32 != R * M * K:
            raise RuntimeError(f"compressed must be int32 with {R * M * K // 32} elements")
        if x.dim() != 2 or x.dtype != torch.float16 or x.shape[0] != K or x.shape[1] != out.shape[1]:
            raise RuntimeError(f"x must be float16 ({K}, {out.shape[1]})")
        if codebook.dim() != 1 or codebook.dtype != torch.float16 or codebook.numel() != 1 << (S + V):
            raise RuntimeError(f"codebook must be float16 with {1 << (S + V)} elements")
        if out.shape[1] != 1:
            raise RuntimeError("only one right-hand side is supported")
        ops.decompress_matvec(compressed, x.view(1, K), codebook, R, M, K, out=out.view(1, M))

    fn.__name__ = f"decompress_matvec_{L}_{S}_{R}_{V}_{M}_{N}_{K}"
    return fn


def __getattr__(name):
    m = _NAME.match(name)
    if not m:
        raise AttributeError(name)
    if name not in _cache:
        _cache[name] = _make(*map(int, m.groups()))
    return _cache[name]
