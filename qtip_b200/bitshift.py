"""BitshiftLinear: the inference side of lib/codebook/bitshift.py upstream, on the B200 kernels.

Same constructor and forward signature as upstream's BitshiftLinear (bitshift.py:356-472) so a
QuantizedLinear (or upstream's own) can hold it unchanged.  Only the inference modes are built:
the Viterbi quantizer and the training modes are outside this package.
"""
import math

import torch
from torch import nn

from . import ops

_CODE_OF_MODE = {"quantlut_sym": ops.CODE_HYB, "3inst": ops.CODE_3INST, "1mad": ops.CODE_1MAD}


class BitshiftCodebook(nn.Module):
    """Decode-side state of bitshift_codebook upstream (bitshift.py:83-201): L, K, V, the tunable LUT."""

    def __init__(self, L=16, K=2, V=2, tlut_bits=16, decode_mode='lut', tlut=None):
        super().__init__()
        if decode_mode not in _CODE_OF_MODE:
            raise NotImplementedError(f"decode_mode {decode_mode!r}: only quantlut_sym, 3inst and 1mad are built")
        if L != 16:
            raise NotImplementedError("L must be 16")
        if decode_mode == 'quantlut_sym' and (V != 2 or tlut_bits != 9 or tlut is None):
            raise NotImplementedError("quantlut_sym needs V=2, tlut_bits=9 and a (512, 2) tlut")
        if decode_mode in ('3inst', '1mad') and V != 1:
            raise NotImplementedError("3inst / 1mad need V=1")
        self.L, self.K, self.V, self.tlut_bits, self.decode_mode = L, K, V, tlut_bits, decode_mode
        self.code = _CODE_OF_MODE[decode_mode]
        self.tlut = tlut


class BitshiftLinear(nn.Module):

    def __init__(self, td_x, td_y, L, K, V, tlut_bits, decode_mode, dtype=torch.float16, tlut=None, has_kernel=False):
        super().__init__()
        if td_x != 16 or td_y != 16:
            raise NotImplementedError("16x16 tiles only")
        self.td_x, self.td_y, self.V = td_x, td_y, V
        self.cb = BitshiftCodebook(L, K, V, tlut_bits, decode_mode, tlut=tlut)
        self.internal_dtype = dtype
        self.has_kernel = has_kernel
        self.scale = 32
        self._sv_cache = {}
        self.workspace = None  # optional caller-owned workspace for the fused matvec

    # -- decoders ------------------------------------------------------------------------------
    def get_hatW_kernel(self, trellis, m, n):
        """Kernel-layout codes -> fp16 (m, n)  (bitshift.py:383-387)."""
        return ops.decode_hyb(trellis, self.cb.tlut, self.cb.K, m, n)

    def get_hatW_packed(self, trellis, m, n):
        """Plain-layout codes -> fp16 (m, n); upstream: unpack_trellis + get_hatW (bitshift.py:329-353, 378-381)."""
        return ops.decode_plain(trellis, self.cb.code, self.cb.K, m, n, tlut=self.cb.tlut)

    def decode(self, trellis, m, n):
        return self.get_hatW_kernel(trellis, m, n) if self.has_kernel else self.get_hatW_packed(trellis, m, n)

    def cache_hatW(self, packed_trellis, had_left, had_right, K_left, K_right, m, n, rcp, tp_rank):
        """Dense W with both Hadamard transforms folded in (bitshift.py:389-413): y = x*SU @ hatW.T * SV*32."""
        tp = int(tp_rank)
        hatW = self.decode(packed_trellis, m, n).float() / self.scale
        hl = lambda t: ops.hadamard(t.contiguous(), had_left, K_left)    # noqa: E731
        hr = lambda t: ops.hadamard(t.contiguous(), had_right, K_right)  # noqa: E731
        if rcp == 1:
            w = hr(hl(hatW.reshape(tp * m, n // tp)).reshape(m, n).T).T
        elif rcp == 2:
            w = hr(hl(hatW).T.reshape(tp * n, m // tp)).reshape(n, m).T
        else:
            w = hr(hl(hatW).T).T
        self.hatW = w.contiguous().to(self.internal_dtype)

    # -- forward -------------------------------------------------------------------------------
    def _sv_scaled(self, SV):
        key = (SV.data_ptr(), SV._version, SV.device)
        hit = self._sv_cache.get(key)
        if hit is None:
            self._sv_cache.clear()
            hit = (SV.float() * self.scale).contiguous()
            self._sv_cache[key] = hit
        return hit

    def forward(self, input, trellis, SU, SV, had_left, had_right, K_left, K_right, rcp, tp_rank, mode='eval',
                **kwargs):
        n, m = len(SU), len(SV)
        tp = int(tp_rank)
        x = input.reshape(-1, n)
        bs = x.shape[0]
        if x.dtype not in (torch.float16, torch.float32):
            x = x.float()
        if mode == 'train-fixW':
            y = ((x.float() * SU).to(self.internal_dtype) @ self.hatW.T).float() * self._sv_scaled(SV)
            return y.view(*input.shape[:-1], m).to(input.dtype)
        if mode != 'eval':
            raise NotImplementedError(f"mode {mode!r}: only 'eval' and 'train-fixW' are built")

        # input side: x * SU -> Hadamard^T (per chunk when row-parallel) -> / 32 -> fp16
        seg_n = n // tp if rcp == 1 else n
        xh = ops.rht(x.reshape(-1, seg_n), sign_in=SU, hadk_bits=ops.hadk_bits_for(had_left, x.device),
                     kfac=K_left or 1, transpose=True, scale=1.0 / (math.sqrt(seg_n) * self.scale),
                     out_dtype=torch.float16).reshape(bs, n)

        v1 = self.cb.code in (ops.CODE_3INST, ops.CODE_1MAD)
        if v1 and ops.gemm_plain_supported(m, n, bs):
            # compute codes: the tensor-core kernel decodes eight states per 44-bit window and is the faster one at
            # every batch size it takes (it needs whole 128 x 64 tiles)
            y = ops.decompress_gemm_plain(trellis, xh, self.cb.code, self.cb.K, m, n)
        elif bs <= ops.MAX_MATVEC_BATCH:
            if self.has_kernel:
                y = ops.decompress_matvec(trellis, xh, self.cb.tlut, self.cb.K, m, n, workspace=self.workspace)
            else:
                y = ops.decompress_matvec_plain(trellis, xh, self.cb.code, self.cb.K, m, n, workspace=self.workspace)
        elif self.has_kernel and ops.gemm_supported(m, n, bs):
            # batches 9..128: decode inside the tensor-core GEMM, the dense matrix never exists
            y = ops.decompress_gemm(trellis, xh, self.cb.tlut, self.cb.K, m, n)
        else:
            # anything else: decode once, dense fp16 GEMM (BitshiftLinearKernelAG upstream, bitshift.py:476-489)
            y = (xh @ self.decode(trellis, m, n).T).float()

        # output side: Hadamard (per chunk when column-parallel) -> * SV * 32
        seg_m = m // tp if rcp == 2 else m
        out = ops.rht(y.reshape(-1, seg_m), sign_out=self._sv_scaled(SV), hadk_bits=ops.hadk_bits_for(had_right, x.device),
                      kfac=K_right or 1, transpose=False, scale=1.0 / math.sqrt(seg_m),
                      out_dtype=input.dtype if input.dtype in (torch.float16, torch.float32) else torch.float32)
        return out.reshape(*input.shape[:-1], m).to(input.dtype)
