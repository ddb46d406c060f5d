"""Generate the golden fixtures under tests/golden/ by running the upstream QTIP torch code on CPU.

    QTIP_REFERENCE_ROOT=/path/to/qtip python tests/golden/make_golden.py

Every array saved here is either a seeded input or the output of an upstream function on it:
  decode_kernel.npz  lib/utils/kernel_decompress.py decode_compressed          (HYB, kernel layout)
  decode_plain.npz   lib/codebook/bitshift.py unpack_trellis + get_hatW        (3INST, 1MAD, HYB; plain layout)
  pack_trellis.npz   lib/codebook/bitshift.py pack_trellis on tail-biting and on open trellis walks
  viterbi.npz        lib/codebook/bitshift.py bitshift_codebook.quantize (the tail-biting Viterbi quantizer) on a few sequences
  hadamard.npz       lib/utils/matmul_had.py matmul_hadU / matmul_hadUt
  layer.npz          lib/codebook/bitshift.py BitshiftLinear.forward (has_kernel=False, CPU)
  layer4096.npz      the same forward on the 4096x4096, 2-bit configuration with inputs drawn by
                     qtip_b200/synth.py (only x, y and an input checksum are stored)
The tests never need the upstream tree: they read these files.
"""
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))

from _reference_import import load_reference  # noqa: E402
import qtip_oracle as O  # noqa: E402
from qtip_b200 import synth  # noqa: E402


def main():
    ref = load_reference()
    B, KD, MH = ref.bitshift, ref.kernel_decompress, ref.matmul_had
    g = torch.Generator().manual_seed(20240611)

    tlut = torch.randn(512, 2, generator=g).half()
    tlut[5, 0] = 0.0
    tlut[9, 1] = -0.0

    # ---- HYB kernel layout ----------------------------------------------------------------------
    out = {"tlut": tlut.numpy()}
    lut16 = B.quantlut_sym(tlut, 16, 9)
    for K in (2, 3, 4):
        for (m, n) in ((32, 64), (64, 96)):
            codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
            W = KD.decode_compressed(16, 9, K, 1, m, n, codes.view(torch.int16).reshape(-1), lut16)
            out[f"codes_K{K}_{m}x{n}"] = codes.numpy()
            out[f"W_K{K}_{m}x{n}"] = W.numpy()
    np.savez_compressed(os.path.join(HERE, "decode_kernel.npz"), **out)

    # ---- plain layout, three codes ---------------------------------------------------------------
    out = {"tlut": tlut.numpy()}
    for K in (2, 3, 4):
        for mode, V in (("3inst", 1), ("1mad", 1), ("quantlut_sym", 2)):
            m, n = 32, 64
            codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
            kw = dict(tlut_bits=9, tlut=tlut) if V == 2 else dict(tlut_bits=0)
            bl = B.BitshiftLinear(16, 16, 16, K, V, decode_mode=mode, **kw)
            st = bl.cb.unpack_trellis(codes.view(torch.int16), 256)
            W = bl.get_hatW(st, m, n)
            out[f"codes_{mode}_K{K}"] = codes.numpy()
            out[f"states_{mode}_K{K}"] = st.numpy().astype(np.uint16)
            out[f"W_{mode}_K{K}"] = W.numpy()  # fp32 for 3inst / 1mad, fp16 for HYB
    np.savez_compressed(os.path.join(HERE, "decode_plain.npz"), **out)

    # ---- pack_trellis (own generator: the draws of the other fixtures stay as they were) ---------------
    g2 = torch.Generator().manual_seed(20240612)
    out = {}
    for K in (2, 3, 4):
        for mode, V in (("3inst", 1), ("quantlut_sym", 2)):
            kw = dict(tlut_bits=9, tlut=tlut) if V == 2 else dict(tlut_bits=0)
            cb = B.bitshift_codebook(L=16, K=K, V=V, decode_mode=mode, **kw)
            T, kv = 256 // V, K * V
            codes = torch.randint(0, 65536, (6, 16 * K), generator=g2).to(torch.uint16)
            closed = cb.unpack_trellis(codes.view(torch.int16), 256).to(torch.int64)
            walk = torch.zeros(4, T, dtype=torch.int64)
            walk[:, 0] = torch.randint(0, 65536, (4,), generator=g2)
            for i in range(1, T):
                walk[:, i] = ((walk[:, i - 1] << kv) & 0xFFFF) | torch.randint(0, 1 << kv, (4,), generator=g2)
            states = torch.cat([closed, walk])
            out[f"states_V{V}_K{K}"] = states.numpy().astype(np.uint16)
            out[f"packed_V{V}_K{K}"] = cb.pack_trellis(states).numpy()
    np.savez_compressed(os.path.join(HERE, "pack_trellis.npz"), **out)

    # ---- Viterbi quantizer (own generator) ----------------------------------------------------------------
    g3 = torch.Generator().manual_seed(20240613)
    tlut32 = torch.randn(512, 2, generator=g3)              # the quantizer holds its table in fp32
    out = {"tlut32": tlut32.numpy()}
    for mode, K, V, N in (("quantlut_sym", 2, 2, 6), ("quantlut_sym", 3, 2, 3), ("quantlut_sym", 4, 2, 3),
                          ("3inst", 2, 1, 3), ("1mad", 2, 1, 3), ("3inst", 3, 1, 2), ("1mad", 4, 1, 2)):
        kw = dict(tlut_bits=9, tlut=tlut32) if V == 2 else dict(tlut_bits=0)
        cb = B.bitshift_codebook(L=16, K=K, V=V, decode_mode=mode, **kw)
        X = torch.randn(N, 256, generator=g3)
        X[0, :8] = 0.0                                       # a flat stretch: ties between equally good predecessors
        hatX, st = cb.quantize(X)
        out[f"X_{mode}_K{K}"] = X.half().numpy()
        out[f"states_{mode}_K{K}"] = st.numpy().astype(np.uint16)
        out[f"hatX_{mode}_K{K}"] = hatX.numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "viterbi.npz"), **out)

    # ---- Hadamard ---------------------------------------------------------------------------------
    out = {}
    for n in (128, 896, 2048, 4096, 6656, 11008):
        x = torch.randn(1, n, generator=g)
        out[f"x_{n}"] = x.numpy()
        out[f"y_{n}"] = MH.matmul_hadU(x).numpy()
        out[f"yt_{n}"] = MH.matmul_hadUt(x).numpy()
    np.savez_compressed(os.path.join(HERE, "hadamard.npz"), **out)

    # ---- full layer -------------------------------------------------------------------------------
    out = {"tlut": tlut.numpy()}
    cases = [("hyb", 2, 256, 512, 0, 1), ("hyb", 2, 256, 512, 1, 1), ("hyb", 2, 256, 512, 2, 1),
             ("hyb", 3, 688, 256, 0, 1), ("hyb", 3, 1376, 256, 0, 1), ("hyb", 4, 256, 832, 0, 2),
             ("3inst", 2, 128, 256, 0, 1), ("1mad", 2, 128, 256, 0, 3)]
    for (mode, K, m, n, rcp, bs) in cases:
        V = 2 if mode == "hyb" else 1
        codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
        if V == 2:
            bl = B.BitshiftLinear(16, 16, 16, K, 2, 9, 'quantlut_sym', tlut=tlut, has_kernel=False)
        else:
            bl = B.BitshiftLinear(16, 16, 16, K, 1, 0, mode, has_kernel=False)
            bl.cb.lut = bl.cb.lut.half()  # a model loaded in fp16 holds the code table in fp16
        SU = (torch.randn(n, generator=g).sign() + 1e-5).sign().half()
        SV = (torch.randn(m, generator=g).sign() + 1e-5).sign().float() * (0.5 + torch.rand(m, generator=g))
        tp = 8
        hl, kl = MH.get_hadK(n // tp if rcp == 1 else n)
        hr, kr = MH.get_hadK(m // tp if rcp == 2 else m)
        x = torch.randn(bs, n, generator=g).half()
        y = bl(x, codes.view(torch.int16), SU, SV, hl, hr, kl, kr, rcp, tp)
        tag = f"{mode}_K{K}_{m}x{n}_rcp{rcp}"
        out[f"codes_{tag}"] = codes.numpy()
        out[f"SU_{tag}"] = SU.numpy()
        out[f"SV_{tag}"] = SV.numpy()
        out[f"x_{tag}"] = x.numpy()
        out[f"y_{tag}"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "layer.npz"), **out)

    # ---- 4096 x 4096, 2 bit: upstream forward on the synthetic inputs of qtip_b200/synth.py ----------
    m = n = 4096
    lay = synth.make_layer(m, n, 2, seed=1000)
    bl = B.BitshiftLinear(16, 16, 16, 2, 2, 9, 'quantlut_sym', tlut=torch.from_numpy(lay["tlut"]), has_kernel=False)
    plain = O.kernel_layout_to_plain_words(lay["codes"], m, n, 2)
    # the plain-layout decode places sequence element t at (t//16, t%16); the kernel layout places
    # it at kernel_sequence_permutation()[t].  Decode upstream, then move the elements.
    st = bl.cb.unpack_trellis(torch.from_numpy(plain.view(np.int16)), 256)
    seq = bl.cb.recons(st).transpose(0, 1).transpose(1, 2).reshape(-1, 256)
    tile = torch.zeros_like(seq)
    tile[:, torch.from_numpy(O.kernel_sequence_permutation())] = seq
    hatW = tile.reshape(m // 16, n // 16, 16, 16).transpose(1, 2).reshape(m, n)
    hatW_direct = KD.decode_compressed(16, 9, 2, 1, m, n, torch.from_numpy(lay["codes"].view(np.int16)).reshape(-1),
                                       B.quantlut_sym(torch.from_numpy(lay["tlut"]), 16, 9))
    assert torch.equal(hatW.view(torch.int16), hatW_direct.view(torch.int16))
    x = torch.from_numpy(lay["x"])
    xs = x.float() * torch.from_numpy(lay["SU"]).float()
    xs = MH.matmul_hadUt_cuda(xs, None, 1) / 32
    y = (xs.to(hatW.dtype) @ hatW.T).float()
    y = MH.matmul_hadU_cuda(y, None, 1) * (torch.from_numpy(lay["SV"]) * 32)
    np.savez_compressed(os.path.join(HERE, "layer4096.npz"), x=lay["x"], y=y.numpy(),
                        crc_codes=np.uint32(zlib.crc32(lay["codes"].tobytes())),
                        W_row0=hatW_direct[0].numpy(), W_row4095=hatW_direct[4095].numpy())
    print("done")


if __name__ == "__main__":
    main()
