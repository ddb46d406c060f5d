"""QuantizedLinear: the module that owns a QTIP layer's buffers (lib/linear/quantized_linear.py upstream).

Buffer names, shapes and dtypes are upstream's (quantized_linear.py:41-67), so a state dict written by
upstream's hfize step loads unchanged: trellis int16 (m/16*n/16, 16K), SU (n) in the module dtype,
SV fp32 (m), tlut fp16 (2^tlut_bits, V), rcp, tp_rank; had_left / had_right are non-persistent.
"""
import math

import torch
import torch.nn as nn

from . import ops
from .bitshift import BitshiftLinear
from .kernel_check import has_kernel


class QuantizedLinear(nn.Module):

    def __init__(self, in_features, out_features, td_x, td_y, L, K, V, tlut_bits, decode_mode, bias=False,
                 dtype=torch.float16, mode='eval', grad_ckpt=False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.td_x, self.td_y, self.L, self.K, self.V = td_x, td_y, L, K, V
        self.tlut_bits, self.decode_mode, self.dtype = tlut_bits, decode_mode, dtype
        self.register_buffer('rcp', torch.tensor(0))
        self.register_buffer('tp_rank', torch.tensor(8))
        self.register_buffer('trellis', torch.zeros((out_features // td_x) * (in_features // td_y),
                                                    math.ceil((td_x * td_y) * K / 16), dtype=torch.int16))
        if decode_mode in ('lut', 'quantlut', 'quantlut_sym'):
            self.tlut = nn.Parameter(torch.zeros(2**tlut_bits, V, dtype=torch.float16), requires_grad=False)
        else:
            self.tlut = None
        if bias:
            self.register_buffer('bias', torch.ones(out_features))
        else:
            self.bias = None
        self.register_buffer("SU", torch.ones(in_features, dtype=self.dtype))
        self.register_buffer("SV", torch.ones(out_features, dtype=torch.float32))
        self.built_codebook_class = False
        self.mode = mode
        if grad_ckpt:
            raise NotImplementedError("gradient checkpointing belongs to the training path, which is not built")
        self.has_kernel = has_kernel(decode_mode, L, K, V, tlut_bits, td_x, td_y)
        # factor matrices for the full widths, as upstream (quantized_linear.py:70-77); a tensor-parallel
        # chunk width n/tp has the same factor as n for every supported model shape
        had_left, self.K_left = ops.get_hadK(in_features)
        had_right, self.K_right = ops.get_hadK(out_features)
        self.register_buffer('had_left', had_left, persistent=False)
        self.register_buffer('had_right', had_right, persistent=False)

    def forward(self, input):
        if not self.built_codebook_class:
            self.codebook_class = BitshiftLinear(self.td_x, self.td_y, self.L, self.K, self.V, self.tlut_bits,
                                                 self.decode_mode, dtype=self.dtype, tlut=self.tlut,
                                                 has_kernel=self.has_kernel)
            rcp = int(self.rcp.item()) if torch.is_tensor(self.rcp) else int(self.rcp)
            del self.rcp
            self.rcp = rcp
            self.tp = int(self.tp_rank.item())
            if self.mode == 'train-fixW':
                self.codebook_class.cache_hatW(self.trellis, self.had_left, self.had_right, self.K_left,
                                               self.K_right, len(self.SV), len(self.SU), self.rcp, self.tp)
            elif self.mode != 'eval':
                raise NotImplementedError(f"mode {self.mode!r} is not built")
            self.built_codebook_class = True
        result = self.codebook_class(input, self.trellis, self.SU, self.SV, self.had_left, self.had_right,
                                     self.K_left, self.K_right, self.rcp, self.tp, mode=self.mode)
        if self.bias is not None:
            return result + self.bias
        return result

    no_ckpt_forward = forward
