"""Pin the numpy oracle against the upstream torch implementation (CPU).

Needs a checkout of the upstream QTIP tree (environment variable QTIP_REFERENCE_ROOT); run by hand:
    python oracle/check_against_reference.py
It is not collected by pytest and nothing at run time depends on it; the fixtures under
tests/golden/ carry the same comparisons to machines without the upstream tree.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "tests", "golden"))
sys.path.insert(0, HERE)

from _reference_import import load_reference  # noqa: E402
import qtip_oracle as O  # noqa: E402


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def main():
    ref = load_reference()
    bs_mod, kd, mh = ref.bitshift, ref.kernel_decompress, ref.matmul_had
    g = torch.Generator().manual_seed(1234)
    ok = True

    def check(name, cond):
        nonlocal ok
        print(("PASS " if cond else "FAIL ") + name)
        ok = ok and bool(cond)

    # --- code tables -------------------------------------------------------------------------
    st = torch.arange(1 << 16)
    check("3inst table", np.array_equal(bs_mod.decode_3inst(st).numpy().astype(np.float16).view(np.uint16),
                                        O.decode_3inst_table().view(np.uint16)))
    check("3inst values are fp16-exact", np.array_equal(bs_mod.decode_3inst(st).numpy(),
                                                        O.decode_3inst_table().astype(np.float32)))
    check("1mad table (fp32 bits)", np.array_equal(bs_mod.decode_1mad(st).numpy().view(np.uint32),
                                                   O.decode_1mad_table().view(np.uint32)))
    tlut = torch.randn(512, 2, generator=g).half()
    tlut[3, 0] = 0.0  # exercises -0.0
    check("hyb expanded lut", np.array_equal(bs_mod.quantlut_sym(tlut, 16, 9).numpy().view(np.uint16),
                                             O.hyb_expand_lut(tlut.numpy()).view(np.uint16)))

    # --- kernel layout decode -----------------------------------------------------------------
    for K in (2, 3, 4):
        for (m, n) in ((32, 64), (64, 96), (256, 256)):
            codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
            lut16 = bs_mod.quantlut_sym(tlut, 16, 9)
            want = kd.decode_compressed(16, 9, K, 1, m, n, codes.view(torch.int16).reshape(-1), lut16)
            got = O.decode_kernel_layout(codes.numpy(), m, n, K, tlut.numpy())
            check(f"decode_compressed K={K} {m}x{n}", np.array_equal(want.numpy().view(np.uint16), got.view(np.uint16)))
            # kernel layout == plain layout re-indexed by the sequence permutation
            plain = O.kernel_layout_to_plain_words(codes.numpy(), m, n, K)
            cb = bs_mod.bitshift_codebook(L=16, K=K, V=2, tlut_bits=9, decode_mode='quantlut_sym', tlut=tlut)
            stt = cb.unpack_trellis(torch.from_numpy(plain.view(np.int16)), 256)
            check(f"states plain K={K} {m}x{n}", np.array_equal(stt.numpy().astype(np.uint16),
                                                                 O.states_plain_layout(plain, m, n, K, 2)))
            seq = cb.recons(stt).transpose(0, 1).transpose(1, 2).reshape(-1, 256)  # tiles, 256 (sequence order)
            perm = O.kernel_sequence_permutation()
            tile = torch.zeros_like(seq)
            tile[:, torch.from_numpy(perm)] = seq
            w2 = tile.reshape(m // 16, n // 16, 16, 16).transpose(1, 2).reshape(m, n)
            check(f"kernel==permuted plain K={K} {m}x{n}", np.array_equal(w2.numpy().view(np.uint16), got.view(np.uint16)))
            back = O.plain_words_to_kernel_layout(plain, m, n, K)
            check(f"layout round trip K={K} {m}x{n}", np.array_equal(back.reshape(-1), codes.numpy().reshape(-1)))

    # --- plain layout decode, all codes ----------------------------------------------------------
    for K in (2, 3, 4):
        for mode, V, code in (("3inst", 1, O.CODE_3INST), ("1mad", 1, O.CODE_1MAD), ("quantlut_sym", 2, O.CODE_HYB)):
            m, n = 32, 64
            codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
            kw = dict(tlut_bits=9, tlut=tlut) if V == 2 else dict(tlut_bits=0)
            bl = bs_mod.BitshiftLinear(16, 16, 16, K, V, decode_mode=mode, **kw)
            stt = bl.cb.unpack_trellis(codes.view(torch.int16), 256)
            want = bl.get_hatW(stt, m, n)
            got = O.decode_plain_layout(codes.numpy(), m, n, K, V, code, tlut.numpy())
            check(f"plain decode {mode} K={K}", np.array_equal(want.half().numpy().view(np.uint16), got.view(np.uint16)))

    # --- pack_trellis: upstream on upstream-unpacked states, and on a walk that does not bite its tail ------
    for K in (2, 3, 4):
        for mode, V in (("3inst", 1), ("quantlut_sym", 2)):
            kw = dict(tlut_bits=9, tlut=tlut) if V == 2 else dict(tlut_bits=0)
            cb = bs_mod.bitshift_codebook(L=16, K=K, V=V, decode_mode=mode, **kw)
            codes = torch.randint(0, 65536, (24, 16 * K), generator=g).to(torch.uint16)
            stt = cb.unpack_trellis(codes.view(torch.int16), 256)
            want = cb.pack_trellis(stt)
            check(f"pack_trellis round trip (upstream) {mode} K={K}", torch.equal(want.view(torch.int16), codes.view(torch.int16)))
            check(f"pack_trellis {mode} K={K}", np.array_equal(want.numpy(), O.pack_trellis(stt.numpy(), K, V)))
            # an open walk (last states do not wrap onto the first): the dropped bits are simply lost
            T, kv = 256 // V, K * V
            walk = torch.zeros(5, T, dtype=torch.int64)
            walk[:, 0] = torch.randint(0, 65536, (5,), generator=g)
            for i in range(1, T):
                walk[:, i] = ((walk[:, i - 1] << kv) & 0xFFFF) | torch.randint(0, 1 << kv, (5,), generator=g)
            check(f"pack_trellis open walk {mode} K={K}",
                  np.array_equal(cb.pack_trellis(walk).numpy(), O.pack_trellis(walk.numpy(), K, V)))

    # --- the Viterbi quantizer (tail-biting), C restatement against upstream's quantize() --------------------------
    import c_oracle as C_
    tlut32 = torch.randn(512, 2, generator=g)
    for mode, K, V, code in (("quantlut_sym", 2, 2, O.CODE_HYB), ("quantlut_sym", 4, 2, O.CODE_HYB), ("3inst", 2, 1, O.CODE_3INST),
                             ("1mad", 3, 1, O.CODE_1MAD)):
        kw = dict(tlut_bits=9, tlut=tlut32) if V == 2 else dict(tlut_bits=0)
        cb = bs_mod.bitshift_codebook(L=16, K=K, V=V, decode_mode=mode, **kw)
        X = torch.randn(3, 256, generator=g)
        _, st = cb.quantize(X)
        check(f"recons table {mode}", np.array_equal(cb.recons_state.numpy().reshape(V, -1).view(np.uint32), O.recons_table(code, tlut32.numpy()).view(np.uint32)))
        got, _ = C_.viterbi_quantize(X.half().numpy(), K, V, O.recons_table(code, tlut32.numpy()))
        check(f"viterbi quantize {mode} K={K}", np.array_equal(st.numpy(), got))

    # --- Hadamard ---------------------------------------------------------------------------------
    for n in (128, 4096, 11008, 6656, 14336):
        x = torch.randn(2, n, generator=g)
        hk, kk = mh.get_hadK(n)
        for tr in (False, True):
            want = mh.matmul_hadU(x, transpose=tr)
            got = O.hadamard(x.numpy(), None if hk is None else hk.numpy(), transpose=tr)
            e = rel_l2(got, want.numpy())
            check(f"hadamard n={n} transpose={tr} rel={e:.2e}", e < 2e-6)
            want2 = mh.matmul_hadU_cuda(x, hk, kk, transpose=tr)
            e2 = rel_l2(got, want2.numpy())
            check(f"hadamard(cuda form) n={n} transpose={tr} rel={e2:.2e}", e2 < 2e-6)

    # --- full layer ---------------------------------------------------------------------------------
    for (m, n, rcp) in ((256, 512, 0), (256, 512, 1), (256, 512, 2), (688, 256, 0), (256, 832, 0)):
        K = 2
        codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g).to(torch.uint16)
        bl = bs_mod.BitshiftLinear(16, 16, 16, K, 2, 9, 'quantlut_sym', tlut=tlut, has_kernel=False)
        SU = (torch.randn(n, generator=g).sign() + 1e-5).sign().half()
        SV = (torch.randn(m, generator=g).sign() + 1e-5).sign().float()
        tp = 8
        hl, kl = mh.get_hadK(n // tp if rcp == 1 else n)
        hr, kr = mh.get_hadK(m // tp if rcp == 2 else m)
        x = torch.randn(1, n, generator=g).half()
        want = bl(x, codes.view(torch.int16), SU, SV, hl, hr, kl, kr, rcp, tp)
        W = O.decode_plain_layout(codes.numpy(), m, n, K, 2, O.CODE_HYB, tlut.numpy())
        got = O.layer_forward(x.float().numpy(), W, SU.float().numpy(), SV.numpy(),
                              None if hl is None else hl.numpy(), None if hr is None else hr.numpy(), rcp, tp)
        e = rel_l2(got, want.float().numpy())
        check(f"layer forward {m}x{n} rcp={rcp} rel={e:.2e}", e < 1e-3)

    print("ALL PASS" if ok else "SOME FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
