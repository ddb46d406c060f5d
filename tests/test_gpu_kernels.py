"""GPU parity: every CUDA entry point, called through the C ABI, against the CPU oracles.

Decoders must be bit-exact (uint16 views, including -0.0).  The fused matvec and the layer forward
must agree with the oracle within relative L2 1e-3 (the fp16 budget of the path); the transforms,
being fp32, within 1e-5.
"""
import numpy as np
import pytest
import torch

import c_oracle as C
import qtip_oracle as O
from conftest import rel_l2
from qtip_b200 import ops, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def u16(t):
    if torch.is_tensor(t):
        t = t.cpu().numpy()
    return np.ascontiguousarray(t).view(np.uint16)


# ---- decoders: bit exact ---------------------------------------------------------------------------
@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("shape", ["32x64", "64x96"])
def test_decode_hyb_golden(golden, K, shape):
    g = golden("decode_kernel")
    m, n = map(int, shape.split("x"))
    W = ops.decode_hyb(dev(g[f"codes_K{K}_{shape}"]), dev(g["tlut"]), K, m, n)
    assert np.array_equal(u16(W), u16(g[f"W_K{K}_{shape}"]))


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("m,n", [(256, 256), (4096, 4096), (4096, 11008), (11008, 4096)])
def test_decode_hyb_vs_oracle(K, m, n):
    lay = synth.make_layer(m, n, K, seed=2000 + K)
    W = ops.decode_hyb(dev(lay["codes"]), dev(lay["tlut"]), K, m, n)
    assert np.array_equal(u16(W), u16(C.decode_kernel(lay["codes"], m, n, K, lay["tlut"])))


# ---- producers of the packed formats: bit exact ---------------------------------------------------------
@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("V", [1, 2])
def test_pack_trellis_golden(golden, K, V):
    g = golden("pack_trellis")
    states = torch.from_numpy(g[f"states_V{V}_K{K}"].astype(np.int32)).to(DEV)
    words = ops.pack_trellis(states, K, V)
    assert np.array_equal(u16(words), g[f"packed_V{V}_K{K}"])
    bad = states.clone()
    bad[1, 7] ^= 0x8000          # the top bit overlaps with the previous state only
    with pytest.raises(RuntimeError, match="1 consecutive state pairs"):
        ops.pack_trellis(bad, K, V)
    # check=False packs whatever it is given, like the arithmetic upstream without its assert
    ops.pack_trellis(bad, K, V, check=False)


VITERBI_CASES = [("quantlut_sym", 2, 2), ("quantlut_sym", 3, 2), ("quantlut_sym", 4, 2), ("3inst", 2, 1), ("1mad", 2, 1),
                 ("3inst", 3, 1), ("1mad", 4, 1)]


@pytest.mark.parametrize("mode,K,V", VITERBI_CASES)
def test_viterbi_quantize_golden(golden, mode, K, V):
    """The tail-biting Viterbi quantizer returns the very states upstream's bitshift_codebook.quantize returned."""
    g = golden("viterbi")
    X = torch.from_numpy(g[f"X_{mode}_K{K}"]).to(DEV)
    states = ops.viterbi_quantize(X, mode, K, tlut=torch.from_numpy(g["tlut32"]))
    assert np.array_equal(states.cpu().numpy().astype(np.uint16), g[f"states_{mode}_K{K}"])


@pytest.mark.parametrize("mode,K,V,N", [("quantlut_sym", 2, 2, 300), ("quantlut_sym", 3, 2, 40), ("quantlut_sym", 4, 2, 40),
                                        ("3inst", 2, 1, 24), ("1mad", 3, 1, 24), ("3inst", 4, 1, 24)])
def test_viterbi_quantize_vs_oracle(mode, K, V, N):
    """More sequences than CTAs can hold at once (the grid-stride loop), scaled inputs, against the C restatement of
    upstream's formulation (full cost vector per step); bit-exact states and final costs."""
    rng = np.random.default_rng(40 + K + V)
    code = ops.CODE_IDS[mode]
    tlut32 = (rng.standard_normal((512, 2)) * 0.97).astype(np.float32)
    X = (rng.standard_normal((N, 256)) * rng.uniform(0.2, 3.0, size=(N, 1))).astype(np.float16)
    X[1] = 0                                                    # all candidates tie on a constant sequence
    want, want_cost = C.viterbi_quantize(X, K, V, O.recons_table(code, tlut32))
    got, cost = ops.viterbi_quantize(torch.from_numpy(X).to(DEV), mode, K, tlut=torch.from_numpy(tlut32), return_cost=True)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(cost.cpu().numpy().view(np.uint32), want_cost.view(np.uint32))


@pytest.mark.parametrize("mode,K,T,N", [("quantlut_sym", 2, 8, 3), ("quantlut_sym", 4, 16, 1), ("3inst", 2, 8, 2), ("1mad", 3, 64, 1),
                                        ("quantlut_sym", 3, 1024, 2)])
def test_viterbi_quantize_short_and_long_sequences(mode, K, T, N):
    """Sequence lengths other than a 16x16 tile - the shortest the tail-biting construction allows (16 stream bits), a single
    sequence, the longest the kernel takes (1024) - against the C restatement."""
    rng = np.random.default_rng(T + K)
    code = ops.CODE_IDS[mode]
    V = 2 if mode == "quantlut_sym" else 1
    tlut32 = rng.standard_normal((512, 2)).astype(np.float32)
    X = rng.standard_normal((N, T)).astype(np.float16)
    want, want_cost = C.viterbi_quantize(X, K, V, O.recons_table(code, tlut32))
    got, cost = ops.viterbi_quantize(torch.from_numpy(X).to(DEV), mode, K, tlut=torch.from_numpy(tlut32), return_cost=True)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(cost.cpu().numpy().view(np.uint32), want_cost.view(np.uint32))


def test_producers_smallest_shapes():
    """One tile / one block: pack_trellis on a single tile, the layout shuffles on a single 32 x 32 block."""
    rng = np.random.default_rng(3)
    for K in (2, 3, 4):
        plain = rng.integers(0, 65536, size=(4, 16 * K), dtype=np.uint16)
        kern = ops.plain_to_kernel_layout(dev(plain), K, 32, 32)
        assert np.array_equal(u16(kern).reshape(-1), O.plain_words_to_kernel_layout(plain, 32, 32, K).reshape(-1))
        for V in (1, 2):
            st = O.states_plain_layout(plain[:1], 16, 16, K, V)
            words = ops.pack_trellis(torch.from_numpy(st.astype(np.int32)).to(DEV), K, V)
            assert np.array_equal(u16(words), plain[:1])


def test_viterbi_quantize_to_decoder():
    """The quantizer's tail on the GPU, end to end: sequences -> Viterbi states -> pack_trellis -> kernel layout -> fused
    decoder.  4096 sequences (a 1024 x 1024 matrix of 16x16 tiles); the table is fp16-representable so that the decoder
    (fp16 table) reproduces the quantizer's reconstruction exactly.  Checks that every walk bites its tail (pack_trellis
    counts violations), that the decoded matrix is the reconstruction the quantizer minimised over, and that the
    reported cost is its squared error."""
    K, m, n = 2, 1024, 1024
    rng = np.random.default_rng(9)
    tl16 = rng.standard_normal((512, 2)).astype(np.float16)
    W = rng.standard_normal((m, n)).astype(np.float32)
    # 16x16 tiles as sequences, row-major inside the tile (lib/algo/finetune.py:188-194 hands these rows to the quantizer)
    seqs = W.reshape(m // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(-1, 256)
    Xd = torch.from_numpy(seqs).to(DEV)
    states, cost = ops.viterbi_quantize(Xd, "quantlut_sym", K, tlut=torch.from_numpy(tl16.astype(np.float32)), return_cost=True)
    words = ops.pack_trellis(states, K, 2)                  # raises if a walk does not overlap / bite its tail
    assert np.array_equal(O.states_plain_layout(u16(words), m, n, K, 2), states.cpu().numpy().astype(np.uint16))
    hat = ops.decode_plain(words, "quantlut_sym", K, m, n, tlut=dev(tl16)).float().cpu().numpy()
    x16 = seqs.astype(np.float16).astype(np.float64).reshape(m // 16, n // 16, 16, 16).transpose(0, 2, 1, 3).reshape(m, n)
    err_tiles = ((hat.astype(np.float64) - x16) ** 2).reshape(m // 16, 16, n // 16, 16).sum(axis=(1, 3)).reshape(-1)
    assert np.allclose(cost.cpu().numpy(), err_tiles, rtol=1e-5)
    # 2 bits per weight on N(0,1) data: the trellis code gets close to the rate-distortion bound (0.0625); a scalar
    # quantizer is at 0.118
    assert 0.06 < err_tiles.sum() / (m * n) < 0.085
    # a handful of sequences against the oracle
    want, _ = C.viterbi_quantize(seqs[:16].astype(np.float16), K, 2, O.recons_table(O.CODE_HYB, tl16.astype(np.float32)))
    assert np.array_equal(states[:16].cpu().numpy(), want)
    # the same codes through the kernel layout and the fused decoder
    kern = ops.plain_to_kernel_layout(words, K, m, n)
    Wk = ops.decode_hyb(kern, dev(tl16), K, m, n)
    assert np.array_equal(u16(Wk), u16(C.decode_kernel(u16(kern), m, n, K, tl16)))


@pytest.mark.parametrize("K,V,m,n", [(2, 2, 4096, 4096), (3, 2, 1024, 2048), (4, 2, 256, 512), (2, 1, 2048, 1024), (4, 1, 512, 512)])
def test_pack_trellis_round_trip(K, V, m, n):
    """pack(unpack(words)) == words on uniform code words (every 256*K-bit stream is a tail-biting walk), and against
    the numpy restatement on a sample of the tiles."""
    rng = np.random.default_rng(77 + K + V)
    codes = rng.integers(0, 65536, size=(m * n // 256, 16 * K), dtype=np.uint16)
    states = O.states_plain_layout(codes, m, n, K, V)
    words = ops.pack_trellis(torch.from_numpy(states.astype(np.int32)).to(DEV), K, V)
    assert np.array_equal(u16(words), codes)
    assert np.array_equal(O.pack_trellis(states[:64], K, V), codes[:64])


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("m,n", [(32, 64), (64, 96), (4096, 4096), (4096, 11008)])
def test_layout_shuffle_vs_oracle(K, m, n):
    rng = np.random.default_rng(5 + K)
    plain = rng.integers(0, 65536, size=(m * n // 256, 16 * K), dtype=np.uint16)
    kern = ops.plain_to_kernel_layout(dev(plain), K, m, n)
    assert np.array_equal(u16(kern).reshape(-1), O.plain_words_to_kernel_layout(plain, m, n, K).reshape(-1))
    back = ops.kernel_to_plain_layout(kern, K, m, n)
    assert np.array_equal(u16(back), plain)
    assert np.array_equal(u16(ops.kernel_to_plain_layout(dev(plain), K, m, n)).reshape(-1),
                          O.kernel_layout_to_plain_words(plain, m, n, K).reshape(-1))


def test_quantizer_tail_to_decoder():
    """States -> pack_trellis -> kernel layout -> the fused decoder gives the plain-layout decode of the same states with
    the elements moved by the kernel's sequence permutation (what lib/algo/finetune.py:188-201 hands to the kernels)."""
    K, m, n = 2, 256, 512
    lay = synth.make_layer(m, n, K, seed=31)
    plain = O.kernel_layout_to_plain_words(lay["codes"], m, n, K)
    states = O.states_plain_layout(plain, m, n, K, 2)
    words = ops.pack_trellis(torch.from_numpy(states.astype(np.int32)).to(DEV), K, 2)
    kern = ops.plain_to_kernel_layout(words, K, m, n)
    assert np.array_equal(u16(kern).reshape(-1), lay["codes"].reshape(-1))
    W = ops.decode_hyb(kern, dev(lay["tlut"]), K, m, n)
    assert np.array_equal(u16(W), u16(C.decode_kernel(lay["codes"], m, n, K, lay["tlut"])))


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("mode", ["3inst", "1mad", "quantlut_sym"])
def test_decode_plain_golden(golden, K, mode):
    g = golden("decode_plain")
    W = ops.decode_plain(dev(g[f"codes_{mode}_K{K}"]), mode, K, 32, 64, tlut=dev(g["tlut"]))
    # 3INST values are fp16-exact; 1MAD is upstream's fp32 value rounded once to fp16
    assert np.array_equal(u16(W), u16(g[f"W_{mode}_K{K}"].astype(np.float16)))


@pytest.mark.parametrize("code,V", [(O.CODE_3INST, 1), (O.CODE_1MAD, 1), (O.CODE_HYB, 2)])
@pytest.mark.parametrize("K,m,n", [(2, 64, 96), (3, 256, 256), (4, 64, 96), (2, 8192, 8192)])
def test_decode_plain_vs_oracle(code, V, K, m, n):
    lay = synth.make_layer(m, n, K, seed=2100 + K)
    W = ops.decode_plain(dev(lay["codes"]), code, K, m, n, tlut=dev(lay["tlut"]))
    want = C.decode_plain(lay["codes"], m, n, K, V, O.state_table(code, lay["tlut"]))
    assert np.array_equal(u16(W), u16(want))


def test_state_functions_all_65536_states():
    """Every state value through both compute codes and the HYB hash: a stream whose windows enumerate
    all 16-bit states (K=4, V=1 / V=2 tiles filled with a counter pattern would not cover them), so
    instead decode random tiles until every state was seen at least once."""
    K, m, n = 4, 512, 512
    lay = synth.make_layer(m, n, K, seed=5)
    st = O.states_plain_layout(lay["codes"], m, n, K, 1)
    assert np.unique(st).size > 64000
    for code in (O.CODE_3INST, O.CODE_1MAD):
        W = ops.decode_plain(dev(lay["codes"]), code, K, m, n)
        assert np.array_equal(u16(W), u16(O.decode_plain_layout(lay["codes"], m, n, K, 1, code)))


# ---- fused matvec ----------------------------------------------------------------------------------
def test_known_answer():
    """qtip-kernels/src/test.cu:22-58 upstream: zero codes, LUT 1.0, x 1.0 => every output is exactly n."""
    for (m, n) in ((8192, 8192), (64, 256)):
        codes = torch.zeros(m * n // 256, 32, dtype=torch.int16, device=DEV)
        tlut = torch.ones(512, 2, dtype=torch.float16, device=DEV)
        x = torch.ones(1, n, dtype=torch.float16, device=DEV)
        y = ops.decompress_matvec(codes, x, tlut, 2, m, n)
        assert torch.all(y == n)


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("m,n,bs", [(32, 64, 1), (64, 96, 1), (256, 256, 1), (4096, 4096, 1), (4096, 11008, 1),
                                    (11008, 4096, 1), (1024, 8192, 1), (4096, 4096, 4), (512, 1024, 8)])
def test_matvec_hyb(K, m, n, bs):
    lay = synth.make_layer(m, n, K, seed=3000 + K, bs=bs)
    out = torch.full((bs, m), float("nan"), device=DEV)  # the op overwrites, it must not accumulate
    y = ops.decompress_matvec(dev(lay["codes"]), dev(lay["x"]), dev(lay["tlut"]), K, m, n, out=out)
    want = C.matvec_kernel(lay["codes"], m, n, K, lay["tlut"], lay["x"])
    assert rel_l2(y.cpu().numpy(), want) < 1e-3
    assert rel_l2(y.cpu().numpy(), want) < 2e-6  # fp32 accumulation of exact fp16 products: only summation order differs
    y2 = ops.decompress_matvec(dev(lay["codes"]), dev(lay["x"]), dev(lay["tlut"]), K, m, n)
    assert torch.equal(y, y2), "result must be deterministic run to run"


def test_matvec_hyb_upstream_test_inputs():
    """Inputs shaped like prepare_arguments of qtip-kernels/test_decompress_matvec.py:251-272 upstream
    (codebook and x ~ N(0,1)/16 clamped to [-1,1]); acceptance as there: allclose(atol=1e-5, rtol=1e-2) in fp16."""
    g = torch.Generator().manual_seed(42)
    for K in (2, 3, 4):
        for (m, n) in ((256, 256), (8192, 1024), (1024, 8192)):
            cb = (torch.randn(1024, generator=g).half() / 16).clamp(-1, 1)
            codes = torch.randint(-2**31, 2**31, (K * m * n // 32,), generator=g, dtype=torch.int64).to(torch.int32)
            x = (torch.randn(n, 1, generator=g).half() / 16).clamp(-1, 1)
            y = ops.decompress_matvec(codes.to(DEV), x.to(DEV).view(1, n), cb.to(DEV), K, m, n)
            W = C.decode_kernel(codes.numpy(), m, n, K, cb.numpy())
            ref = torch.from_numpy(C.matvec_dense(W, x.numpy().reshape(1, n)))
            assert torch.allclose(y.cpu().half(), ref.half(), atol=1e-5, rtol=0.01)


@pytest.mark.parametrize("code", [O.CODE_3INST, O.CODE_1MAD])
@pytest.mark.parametrize("K,m,n,bs", [(2, 32, 64, 1), (2, 256, 256, 1), (3, 64, 96, 2), (4, 128, 256, 8),
                                      (2, 8192, 8192, 1), (2, 8192, 8192, 4)])
def test_matvec_plain(code, K, m, n, bs):
    lay = synth.make_layer(m, n, K, seed=3100 + K, bs=bs, code="none")
    y = ops.decompress_matvec_plain(dev(lay["codes"]), dev(lay["x"]), code, K, m, n)
    W = C.decode_plain(lay["codes"], m, n, K, 1, O.state_table(code))
    want = C.matvec_dense(W, lay["x"])
    assert rel_l2(y.cpu().numpy(), want) < 1e-3
    assert rel_l2(y.cpu().numpy(), want) < 2e-6


# ---- Hadamard -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [128, 896, 2048, 4096, 6656, 11008])
def test_hadamard_golden(golden, n):
    g = golden("hadamard")
    hk, k = ops.get_hadK(n)
    x = dev(g[f"x_{n}"])
    hk = None if hk is None else hk.to(DEV)
    assert rel_l2(ops.hadamard(x, hk, k).cpu().numpy(), g[f"y_{n}"]) < 1e-5
    assert rel_l2(ops.hadamard(x, hk, k, transpose=True).cpu().numpy(), g[f"yt_{n}"]) < 1e-5


@pytest.mark.parametrize("n", [2, 64, 8192, 14336, 16384, 28672, 53248])
def test_rht_vs_oracle(n):
    rng = np.random.default_rng(n)
    rows = 3
    x = rng.standard_normal((rows, n)).astype(np.float32)
    su = np.sign(rng.standard_normal(n)).astype(np.float16)
    sv = (np.sign(rng.standard_normal(n)) * (0.5 + rng.random(n))).astype(np.float32)
    hk, k = ops.get_hadK(n)
    bits = None if hk is None else ops.pack_hadk(hk.to(DEV))
    hkn = None if hk is None else hk.numpy()
    # input side: fp32 in, fp16 out, sign in, transposed factor
    got = ops.rht(dev(x), sign_in=dev(su), hadk_bits=bits, kfac=k, transpose=True, scale=1 / np.sqrt(n) / 32,
                  out_dtype=torch.float16)
    want = O.hadamard(x * su.astype(np.float32), hkn, transpose=True) / 32
    assert rel_l2(got.float().cpu().numpy(), want) < 6e-4  # fp16 output rounding
    # output side: fp32 in, fp32 out, sign out
    got = ops.rht(dev(x), sign_out=dev(sv), hadk_bits=bits, kfac=k, scale=1 / np.sqrt(n))
    want = O.hadamard(x, hkn) * sv
    assert rel_l2(got.cpu().numpy(), want) < 1e-5
    # fp16 in
    xh = x.astype(np.float16)
    got = ops.rht(dev(xh), hadk_bits=bits, kfac=k, scale=1 / np.sqrt(n), out_dtype=torch.float32)
    assert rel_l2(got.cpu().numpy(), O.hadamard(xh.astype(np.float32), hkn)) < 1e-5


def test_rht_chunked_signs():
    """Per-chunk transforms of the tensor-parallel layouts: rows cycle through the chunks of the sign vector."""
    rng = np.random.default_rng(0)
    bs, tp, seg = 2, 8, 832  # 832 = 52 * 16
    x = rng.standard_normal((bs, tp * seg)).astype(np.float32)
    su = np.sign(rng.standard_normal(tp * seg)).astype(np.float32)
    hk, k = ops.get_hadK(seg)
    got = ops.rht(dev(x).reshape(bs * tp, seg), sign_in=dev(su), hadk_bits=ops.pack_hadk(hk.to(DEV)), kfac=k,
                  transpose=True, scale=1 / np.sqrt(seg)).reshape(bs, tp * seg)
    want = O.hadamard((x * su).reshape(bs * tp, seg), hk.numpy(), transpose=True).reshape(bs, tp * seg)
    assert rel_l2(got.cpu().numpy(), want) < 1e-5


# ---- tcgen05 decompress-GEMM ---------------------------------------------------------------------------------
@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("m,n,bs", [(128, 64, 16), (256, 256, 9), (1024, 2048, 32), (8192, 8192, 16), (4096, 11008, 64),
                                    (11008, 4096, 33), (1024, 2048, 65), (4096, 4096, 128), (8192, 8192, 100)])
def test_decompress_gemm(K, m, n, bs):
    """Tensor-core path against the dense product of the (bit-exact) decoded matrix, fp32 accumulation."""
    lay = synth.make_layer(m, n, K, seed=3300 + K, bs=bs)
    codes, x, tl = dev(lay["codes"]), dev(lay["x"]), dev(lay["tlut"])
    y = ops.decompress_gemm(codes, x, tl, K, m, n)
    W = ops.decode_hyb(codes, tl, K, m, n)
    want = x.float() @ W.float().T
    torch.cuda.synchronize()
    assert ops.gemm_status(DEV) == 0, "a bounded barrier wait inside the kernel gave up"
    assert rel_l2(y.cpu().numpy(), want.cpu().numpy()) < 1e-3
    assert rel_l2(y.cpu().numpy(), want.cpu().numpy()) < 1e-5
    y2 = ops.decompress_gemm(codes, x, tl, K, m, n)
    assert torch.equal(y, y2)


@pytest.mark.gpu
@pytest.mark.parametrize("code", [O.CODE_3INST, O.CODE_1MAD])
@pytest.mark.parametrize("K,m,n,bs", [(2, 128, 64, 16), (2, 1024, 2048, 32), (3, 256, 256, 9), (4, 512, 1024, 64),
                                      (2, 8192, 8192, 16), (2, 1024, 2048, 128), (3, 512, 1024, 72)])
def test_decompress_gemm_plain_vs_oracle(code, K, m, n, bs):
    """Compute codes (V = 1, plain layout) on the tensor-core path against the CPU oracle: bit-exact decode
    (C.decode_plain with the oracle's state table) + dense product with fp32 accumulation."""
    lay = synth.make_layer(m, n, K, seed=3500 + K, bs=bs, code="none")
    y = ops.decompress_gemm_plain(dev(lay["codes"]), dev(lay["x"]), code, K, m, n)
    torch.cuda.synchronize()
    want = C.matvec_dense(C.decode_plain(lay["codes"], m, n, K, 1, O.state_table(code)), lay["x"])
    assert ops.gemm_status(DEV) == 0, "a bounded barrier wait inside the kernel gave up"
    assert rel_l2(y.cpu().numpy(), want) < 1e-5
    assert torch.equal(y, ops.decompress_gemm_plain(dev(lay["codes"]), dev(lay["x"]), code, K, m, n))


@pytest.mark.gpu
@pytest.mark.parametrize("K,m,n,bs", [(2, 1024, 2048, 16), (4, 256, 256, 40), (3, 1024, 1024, 128), (2, 256, 512, 90)])
def test_decompress_gemm_vs_oracle(K, m, n, bs):
    """The tensor-core path directly against the CPU oracle (decode of the kernel layout + dense product), with no
    CUDA kernel of this library on the reference side."""
    lay = synth.make_layer(m, n, K, seed=3400 + K, bs=bs)
    y = ops.decompress_gemm(dev(lay["codes"]), dev(lay["x"]), dev(lay["tlut"]), K, m, n)
    torch.cuda.synchronize()
    want = C.matvec_dense(C.decode_kernel(lay["codes"], m, n, K, lay["tlut"]), lay["x"])
    assert ops.gemm_status(DEV) == 0
    assert rel_l2(y.cpu().numpy(), want) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("ctx", [1, 7, 200, 257, 2048, 2049, 5000])
@pytest.mark.parametrize("heads", [(8, 8), (16, 2)])
def test_attn_decode_matches_fp32_softmax(ctx, heads):
    """Single-query attention over a cache of `ctx` rows against an fp32 torch reference (tolerance:
    fp16 rounding of the output, 2e-3 absolute on values of order 1)."""
    n_heads, n_kv = heads
    hd = 128
    g = torch.Generator(device="cuda").manual_seed(ctx * 31 + n_heads)
    q = torch.randn(n_heads, hd, generator=g, device="cuda").half()
    ck = torch.randn(ctx + 3, n_kv * hd, generator=g, device="cuda").half()
    cv = torch.randn(ctx + 3, n_kv * hd, generator=g, device="cuda").half()
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    out = torch.empty(n_heads, hd, dtype=torch.float16, device="cuda")
    ops.attn_decode(out, q, ck, cv, pos, n_heads, n_kv, hd)
    rep = n_heads // n_kv
    k = ck[:ctx].float().view(ctx, n_kv, hd).repeat_interleave(rep, dim=1)     # (ctx, heads, hd)
    v = cv[:ctx].float().view(ctx, n_kv, hd).repeat_interleave(rep, dim=1)
    s = torch.einsum("hd,thd->ht", q.float(), k) / hd ** 0.5
    ref = torch.einsum("ht,thd->hd", torch.softmax(s, dim=-1), v)
    torch.testing.assert_close(out.float(), ref, atol=2e-3, rtol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(4096, 32000), (512, 1001), (16384, 2048)])
def test_lm_head_matches_torch(shape):
    """Final RMSNorm + fp16 head against torch (fp32 accumulation; tolerance 1e-3 relative L2)."""
    hidden, vocab = shape
    g = torch.Generator(device="cuda").manual_seed(hidden + vocab)
    res = torch.randn(hidden, generator=g, device="cuda").half()
    delta = (0.3 * torch.randn(hidden, generator=g, device="cuda")).half()
    w_norm = (1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).half()
    W = (0.02 * torch.randn(vocab, hidden, generator=g, device="cuda")).half()
    logits = torch.zeros(vocab, device="cuda")
    ops.lm_head(logits, res, delta, w_norm, W, 1e-5)
    h = (res + delta).float()
    h = (h * torch.rsqrt(h.pow(2).mean() + 1e-5)).half() * w_norm
    want = h.float() @ W.float().T
    assert rel_l2(logits.cpu().numpy(), want.cpu().numpy()) < 1e-3


@pytest.mark.gpu
def test_embed_and_sampler():
    """Embedding lookup is a copy; the sampler returns one of the top-k logits, is reproducible for a seed and a
    position, follows softmax(top / temperature) over many positions, and advances the position."""
    vocab, hidden, k = 5000, 256, 5
    g = torch.Generator(device="cuda").manual_seed(5)
    embed = torch.randn(vocab, hidden, generator=g, device="cuda").half()
    tok = torch.tensor([1234], dtype=torch.int64, device="cuda")
    res = torch.zeros(hidden, dtype=torch.float16, device="cuda")
    delta = torch.ones(hidden, dtype=torch.float16, device="cuda")
    ops.embed_token(res, delta, embed, tok)
    assert torch.equal(res, embed[1234]) and torch.count_nonzero(delta) == 0

    logits = torch.randn(vocab, generator=g, device="cuda")
    top = torch.topk(logits, k)
    n_draws = 4000
    out = torch.full((n_draws + 2,), -1, dtype=torch.int64, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(n_draws):
        ops.sample_top_k(tok, out, pos, logits, temperature=0.6, top_k=k, seed=77)
    torch.cuda.synchronize()
    assert int(pos) == n_draws and int(out[0]) == -1 and int(tok) == int(out[n_draws])
    drawn = out[1:n_draws + 1]
    assert bool(torch.isin(drawn, top.indices).all())
    want = torch.softmax(top.values / 0.6, dim=0)
    freq = torch.stack([(drawn == i).float().mean() for i in top.indices])
    assert torch.allclose(freq, want, atol=0.03)
    # same seed and positions -> same tokens
    out2 = torch.full_like(out, -1)
    pos.zero_()
    for _ in range(50):
        ops.sample_top_k(tok, out2, pos, logits, temperature=0.6, top_k=k, seed=77)
    assert torch.equal(out2[1:51], out[1:51])
