"""Seeded synthetic inputs for QTIP layers (stand-ins for released checkpoints).

Distributions follow the quantizer's outputs: packed codes are uniform 16-bit words (every
bit pattern is a valid tail-biting trellis), the HYB LUT is N(0,1) fp16 (512, 2), SU / SV are
+-1 drawn as (randn.sign() + 1e-5).sign() (lib/algo/finetune.py:116-117 upstream), the
activation is N(0,1) fp16.
"""
import numpy as np
import torch


def make_layer(m, n, K, seed, bs=1, code="hyb", device="cpu", as_numpy=None):
    """Returns dict(codes uint16 (m*n/256, 16K), tlut fp16 (512,2) or None, SU fp16 (n), SV fp32 (m),
    x fp16 (bs, n)).  CPU results are numpy arrays unless as_numpy=False; device results are tensors."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(int(seed))
    codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g, device=dev, dtype=torch.int32)
    codes = codes.to(torch.uint16)
    tlut = torch.randn(512, 2, generator=g, device=dev).half() if code == "hyb" else None
    SU = (torch.randn(n, generator=g, device=dev).sign() + 1e-5).sign().half()
    SV = (torch.randn(m, generator=g, device=dev).sign() + 1e-5).sign().float()
    x = torch.randn(bs, n, generator=g, device=dev).half()
    out = dict(codes=codes, tlut=tlut, SU=SU, SV=SV, x=x)
    if as_numpy is None:
        as_numpy = dev.type == "cpu"
    if as_numpy:
        out = {k: (None if v is None else v.cpu().numpy()) for k, v in out.items()}
    return out
