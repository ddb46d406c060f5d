"""CPU: the numpy and C restatements against the golden vectors produced by the upstream torch code."""
import numpy as np
import pytest

import c_oracle as C
import qtip_oracle as O
from conftest import rel_l2
from qtip_b200 import ops, synth


def u16(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("shape", ["32x64", "64x96"])
def test_decode_kernel_layout_golden(golden, K, shape):
    g = golden("decode_kernel")
    m, n = map(int, shape.split("x"))
    want = u16(g[f"W_K{K}_{shape}"])
    assert np.array_equal(u16(O.decode_kernel_layout(g[f"codes_K{K}_{shape}"], m, n, K, g["tlut"])), want)
    assert np.array_equal(u16(C.decode_kernel(g[f"codes_K{K}_{shape}"], m, n, K, g["tlut"])), want)


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("mode,V,code", [("3inst", 1, O.CODE_3INST), ("1mad", 1, O.CODE_1MAD),
                                         ("quantlut_sym", 2, O.CODE_HYB)])
def test_decode_plain_layout_golden(golden, K, mode, V, code):
    g = golden("decode_plain")
    codes = g[f"codes_{mode}_K{K}"]
    assert np.array_equal(O.states_plain_layout(codes, 32, 64, K, V), g[f"states_{mode}_K{K}"])
    want = g[f"W_{mode}_K{K}"]
    got = O.decode_plain_layout(codes, 32, 64, K, V, code, g["tlut"])
    if mode == "1mad":
        # upstream keeps 1MAD weights in fp32; the fp16 decoders round that value once (nearest even)
        assert want.dtype == np.float32
        table32 = O.decode_1mad_table()
        st = O.states_plain_layout(codes, 32, 64, K, 1)
        w32 = table32[st].reshape(2, 4, 16, 16).transpose(0, 2, 1, 3).reshape(32, 64)
        assert np.array_equal(w32.view(np.uint32), want.view(np.uint32))
    want16 = want.astype(np.float16)
    if mode == "3inst":
        assert np.array_equal(want16.astype(np.float32), want)  # 3INST values are exact in fp16
    assert np.array_equal(u16(got), u16(want16))
    table = O.state_table(code, g["tlut"])
    assert np.array_equal(u16(C.decode_plain(codes, 32, 64, K, V, table)), u16(want16))


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("V", [1, 2])
def test_pack_trellis_golden(golden, K, V):
    g = golden("pack_trellis")
    states = g[f"states_V{V}_K{K}"]
    assert np.array_equal(O.pack_trellis(states, K, V), g[f"packed_V{V}_K{K}"])
    # the first six walks of the fixture bite their tail: unpacking the words gives the states back
    back = O.states_plain_layout(g[f"packed_V{V}_K{K}"][:6], 16, 96, K, V)
    assert np.array_equal(back, states[:6])
    bad = states.copy()
    bad[1, 7] ^= 0x8000
    with pytest.raises(ValueError):
        O.pack_trellis(bad, K, V)


VITERBI_CASES = [("quantlut_sym", 2, 2), ("quantlut_sym", 3, 2), ("quantlut_sym", 4, 2), ("3inst", 2, 1), ("1mad", 2, 1),
                 ("3inst", 3, 1), ("1mad", 4, 1)]


@pytest.mark.parametrize("mode,K,V", VITERBI_CASES)
def test_viterbi_quantize_golden(golden, mode, K, V):
    """The C restatement of the tail-biting Viterbi quantizer returns the states upstream's quantize() returned."""
    g = golden("viterbi")
    code = {"quantlut_sym": O.CODE_HYB, "3inst": O.CODE_3INST, "1mad": O.CODE_1MAD}[mode]
    recons = O.recons_table(code, g["tlut32"])
    X = g[f"X_{mode}_K{K}"]
    states, cost = C.viterbi_quantize(X, K, V, recons)
    assert np.array_equal(states.astype(np.uint16), g[f"states_{mode}_K{K}"])
    # upstream's hatX is the reconstruction of those states, and the reported cost is its squared error
    hat = recons[:, states].transpose(1, 2, 0).reshape(X.shape)
    assert np.array_equal(hat, g[f"hatX_{mode}_K{K}"])
    err = ((hat.astype(np.float64) - X.astype(np.float64)) ** 2).sum(axis=1)
    assert np.allclose(cost, err, rtol=1e-5)
    # the walks bite their tail: packing raises on a broken overlap, unpacking the words gives the states back
    words = O.pack_trellis(states, K, V)
    assert np.array_equal(O.states_plain_layout(words, 16, 16 * len(X), K, V), states.astype(np.uint16))


def test_c_tables_match_numpy():
    assert np.array_equal(u16(C.code_table(1)), u16(O.decode_3inst_table()))
    assert np.array_equal(u16(C.code_table(2)), u16(O.decode_1mad_table().astype(np.float16)))
    tl = np.random.default_rng(1).standard_normal((512, 2)).astype(np.float16)
    assert np.array_equal(u16(C.hyb_expand_lut(tl)), u16(O.hyb_expand_lut(tl)))


@pytest.mark.parametrize("n", [128, 896, 2048, 4096, 6656, 11008])
def test_hadamard_golden(golden, n):
    g = golden("hadamard")
    hk, k = ops.get_hadK(n)
    hk = None if hk is None else hk.numpy()
    x = g[f"x_{n}"]
    for tr, key in ((False, "y"), (True, "yt")):
        want = g[f"{key}_{n}"]
        assert rel_l2(O.hadamard(x, hk, transpose=tr), want) < 2e-6
        assert rel_l2(C.hadamard(x, hk, transpose=tr), want) < 2e-6


def test_hadamard_factor_table():
    assert [O.had_factor(n) for n in (4096, 11008, 8192, 28672, 16384, 53248, 2048, 6656, 128, 14336)] == \
        [1, 172, 1, 28, 1, 52, 1, 52, 1, 28]
    for n in (4096, 11008, 53248, 6656, 896):
        assert ops.had_factor(n) == O.had_factor(n)
    for k in (12, 20, 28, 36, 52, 60, 108, 116, 124, 140, 156, 172):
        h = ops.get_hadK(k * 2)[0].numpy()
        assert np.array_equal(h @ h.T, k * np.eye(k))


LAYER_CASES = [("hyb", 2, 256, 512, 0), ("hyb", 2, 256, 512, 1), ("hyb", 2, 256, 512, 2), ("hyb", 3, 688, 256, 0), ("hyb", 3, 1376, 256, 0),
               ("hyb", 4, 256, 832, 0), ("3inst", 2, 128, 256, 0), ("1mad", 2, 128, 256, 0)]


@pytest.mark.parametrize("mode,K,m,n,rcp", LAYER_CASES)
def test_layer_forward_golden(golden, mode, K, m, n, rcp):
    """Upstream BitshiftLinear.forward (plain layout, CPU, fp16 matmul) vs the restatement; the budget
    is the fp16 rounding of upstream's CPU matmul output (about 3e-4 relative L2)."""
    g = golden("layer")
    tag = f"{mode}_K{K}_{m}x{n}_rcp{rcp}"
    codes, SU, SV, x, want = (g[f"{k}_{tag}"] for k in ("codes", "SU", "SV", "x", "y"))
    tp = 8
    hl = ops.get_hadK(n // tp if rcp == 1 else n)[0]
    hr = ops.get_hadK(m // tp if rcp == 2 else m)[0]
    hl, hr = (None if h is None else h.numpy() for h in (hl, hr))
    code = O.CODE_NAMES[mode]
    W = O.decode_plain_layout(codes, m, n, K, 2 if mode == "hyb" else 1, code, g["tlut"])
    got = O.layer_forward(x.astype(np.float32), W, SU.astype(np.float32), SV, hl, hr, rcp, tp)
    assert rel_l2(got, want.astype(np.float32)) < 1e-3
    if mode == "hyb" and m % 32 == 0 and n % 32 == 0:
        # the C forward consumes kernel-layout codes: move the plain tiles' sequence order over
        kc = O.plain_words_to_kernel_layout(codes, m, n, K)
        Wk = O.decode_kernel_layout(kc, m, n, K, g["tlut"])
        got_c = C.layer_forward(x.astype(np.float32), kc, m, n, K, g["tlut"], SU.astype(np.float32), SV, hl, hr, rcp, tp)
        want_c = O.layer_forward(x.astype(np.float32), Wk, SU.astype(np.float32), SV, hl, hr, rcp, tp)
        assert rel_l2(got_c, want_c) < 1e-5


def test_layer4096_golden(golden):
    """4096x4096, 2 bit, HYB, batch 1 (upstream's own CPU-runnable case): upstream forward vs both restatements."""
    g = golden("layer4096")
    import zlib
    lay = synth.make_layer(4096, 4096, 2, seed=1000)
    assert np.uint32(zlib.crc32(lay["codes"].tobytes())) == g["crc_codes"], "synthetic generator drifted"
    W = C.decode_kernel(lay["codes"], 4096, 4096, 2, lay["tlut"])
    assert np.array_equal(u16(W[0]), u16(g["W_row0"])) and np.array_equal(u16(W[4095]), u16(g["W_row4095"]))
    y = C.layer_forward(lay["x"].astype(np.float32), lay["codes"], 4096, 4096, 2, lay["tlut"],
                        lay["SU"].astype(np.float32), lay["SV"])
    assert rel_l2(y, g["y"]) < 1e-3
    y2 = O.layer_forward(lay["x"].astype(np.float32), W, lay["SU"].astype(np.float32), lay["SV"])
    assert rel_l2(y, y2) < 1e-5


def test_known_answer_all_zero_codes():
    """qtip-kernels/src/test.cu:22-58 upstream: zero codes, LUT all 1.0, x all 1.0 => every output equals n."""
    m, n = 64, 256
    codes = np.zeros((m * n // 256, 32), dtype=np.uint16)
    tlut = np.ones((512, 2), dtype=np.float16)
    x = np.ones((1, n), dtype=np.float16)
    assert np.all(C.matvec_kernel(codes, m, n, 2, tlut, x) == n)
    assert np.all(O.matvec_fp16(O.decode_kernel_layout(codes, m, n, 2, tlut), x) == n)


@pytest.mark.parametrize("K", [2, 3, 4])
def test_layout_round_trip(K):
    rng = np.random.default_rng(K)
    m, n = 64, 96
    codes = rng.integers(0, 65536, (m * n // 256, 16 * K), dtype=np.uint16)
    plain = O.kernel_layout_to_plain_words(codes, m, n, K)
    assert np.array_equal(O.plain_words_to_kernel_layout(plain, m, n, K), codes)
    # same weights, sequence order differs by the fragment permutation
    tl = rng.standard_normal((512, 2)).astype(np.float16)
    Wk = O.decode_kernel_layout(codes, m, n, K, tl)
    Wp = O.decode_plain_layout(plain, m, n, K, 2, O.CODE_HYB, tl)
    perm = O.kernel_sequence_permutation()
    tiles_p = Wp.reshape(m // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(-1, 256)
    tiles_k = Wk.reshape(m // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(-1, 256)
    assert np.array_equal(u16(tiles_k[:, perm]), u16(tiles_p))


def test_c_matvec_matches_dense():
    lay = synth.make_layer(128, 256, 3, seed=7, bs=3)
    W = C.decode_kernel(lay["codes"], 128, 256, 3, lay["tlut"])
    a = C.matvec_kernel(lay["codes"], 128, 256, 3, lay["tlut"], lay["x"])
    b = C.matvec_dense(W, lay["x"])
    assert rel_l2(a, b) < 1e-5


def test_cpu_decode_step_fused_matrices_equal_separate_linears():
    """The CPU decode step of the benchmark's reference arm with q||k||v as ONE matrix (per-chunk output transforms, upstream's
    rcp = 2 layout) gives what three separate linears over the same rows, table and signs give."""
    import llama_oracle as LO
    rng = np.random.default_rng(12)
    hadk = lambda n: None  # noqa: E731  (powers of two only here)
    m, n, K = 3 * 256, 512, 2
    fused = LO._Lin(rng, m, n, K, hadk, chunks=3)
    x = rng.standard_normal(n).astype(np.float32)
    y = fused(x)
    rows = m // 3
    per = fused.codes.reshape(-1).size // 3
    for c in range(3):
        part = C.layer_forward(x, fused.codes.reshape(-1)[c * per:(c + 1) * per], rows, n, K, fused.tlut, fused.SU,
                               fused.SV[c * rows:(c + 1) * rows], None, None)
        assert np.array_equal(LO._f16(part.reshape(-1)), y[c * rows:(c + 1) * rows])
    # and a whole step runs with fused matrices (tiny shape)
    model = LO.OracleLlama(hadk, n_layers=2, hidden=256, n_heads=2, n_kv_heads=2, head_dim=128, mlp=512, vocab=64,
                           max_positions=8, weight_sets=2, fuse_qkv=True)
    model.fill_cache(3)
    tok = model.step(5)
    assert 0 <= tok < 64 and model.pos == 4
