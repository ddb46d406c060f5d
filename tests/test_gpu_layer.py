"""GPU parity of the module-level interfaces: BitshiftLinear.forward, QuantizedLinear, the qtip_kernels shim."""
import numpy as np
import pytest
import torch

import c_oracle as C
import qtip_oracle as O
from conftest import rel_l2
from qtip_b200 import ops, qtip_kernels, synth
from qtip_b200.bitshift import BitshiftLinear
from qtip_b200.quantized_linear import QuantizedLinear

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LAYER_CASES = [("hyb", 2, 256, 512, 0), ("hyb", 2, 256, 512, 1), ("hyb", 2, 256, 512, 2), ("hyb", 3, 1376, 256, 0),
               ("hyb", 4, 256, 832, 0), ("3inst", 2, 128, 256, 0), ("1mad", 2, 128, 256, 0)]


def t16(a):
    return torch.from_numpy(a.view(np.int16)).to(DEV)


@pytest.mark.parametrize("mode,K,m,n,rcp", LAYER_CASES)
def test_bitshift_linear_forward_golden(golden, mode, K, m, n, rcp):
    """Outputs of upstream BitshiftLinear.forward (CPU, plain layout) are the reference.  HYB layers run here
    through the fused kernel on the same weights moved to the kernel layout (a pure byte shuffle plus the
    fragment permutation of the tile elements, so the decoded matrix differs only by that permutation:
    compare against the oracle on the kernel-layout matrix, and against upstream through the plain path)."""
    g = golden("layer")
    tag = f"{mode}_K{K}_{m}x{n}_rcp{rcp}"
    codes, SU, SV, x, want = (g[f"{k}_{tag}"] for k in ("codes", "SU", "SV", "x", "y"))
    tp = 8
    hl, kl = ops.get_hadK(n // tp if rcp == 1 else n)
    hr, kr = ops.get_hadK(m // tp if rcp == 2 else m)
    hl, hr = (None if h is None else h.to(DEV) for h in (hl, hr))
    tl = torch.from_numpy(g["tlut"]).to(DEV)
    V = 2 if mode == "hyb" else 1
    dm = "quantlut_sym" if mode == "hyb" else mode
    # plain layout on the GPU == upstream's path
    bl = BitshiftLinear(16, 16, 16, K, V, 9 if V == 2 else 0, dm, tlut=tl if V == 2 else None, has_kernel=False)
    xs = torch.from_numpy(x).to(DEV)
    if V == 1:
        y = bl(xs, t16(codes), torch.from_numpy(SU).to(DEV), torch.from_numpy(SV).to(DEV), hl, hr, kl, kr, rcp, tp)
        assert y.dtype == xs.dtype and y.shape == (x.shape[0], m)
        assert rel_l2(y.float().cpu().numpy(), want.astype(np.float32)) < 1e-3
        return
    # HYB: decode of the plain layout is bit exact with upstream's matrix ...
    Wp = bl.decode(t16(codes), m, n)
    assert np.array_equal(Wp.cpu().numpy().view(np.uint16),
                          O.decode_plain_layout(codes, m, n, K, 2, O.CODE_HYB, g["tlut"]).view(np.uint16))
    # ... and the whole forward through the dense path matches upstream's output
    bl.cb.K = K
    xh = ops.rht(xs.reshape(-1, n // tp if rcp == 1 else n), sign_in=torch.from_numpy(SU).to(DEV),
                 hadk_bits=ops.hadk_bits_for(hl, DEV), kfac=kl, transpose=True,
                 scale=1 / (np.sqrt(n // tp if rcp == 1 else n) * 32), out_dtype=torch.float16).reshape(-1, n)
    yy = (xh @ Wp.T).float()
    out = ops.rht(yy.reshape(-1, m // tp if rcp == 2 else m), sign_out=torch.from_numpy(SV).to(DEV) * 32,
                  hadk_bits=ops.hadk_bits_for(hr, DEV), kfac=kr, scale=1 / np.sqrt(m // tp if rcp == 2 else m))
    assert rel_l2(out.reshape(-1, m).cpu().numpy(), want.astype(np.float32)) < 1e-3
    # fused kernel on kernel-layout codes vs the oracle's forward on the same codes
    if m % 32 == 0 and n % 32 == 0:
        kc = O.plain_words_to_kernel_layout(codes, m, n, K)
        blk = BitshiftLinear(16, 16, 16, K, 2, 9, "quantlut_sym", tlut=tl, has_kernel=True)
        y = blk(xs, t16(kc), torch.from_numpy(SU).to(DEV), torch.from_numpy(SV).to(DEV), hl, hr, kl, kr, rcp, tp)
        want_k = C.layer_forward(x.astype(np.float32), kc, m, n, K, g["tlut"], SU.astype(np.float32), SV,
                                 None if hl is None else hl.cpu().numpy(), None if hr is None else hr.cpu().numpy(), rcp, tp)
        assert y.dtype == torch.float16
        assert rel_l2(y.float().cpu().numpy(), want_k) < 1e-3


def test_layer4096_vs_upstream_output(golden):
    """4096x4096, 2 bit, HYB, batch 1 (upstream's own CPU-runnable case): upstream's CPU forward output is the fixture."""
    g = golden("layer4096")
    lay = synth.make_layer(4096, 4096, 2, seed=1000)
    q = QuantizedLinear(4096, 4096, 16, 16, 16, 2, 2, 9, "quantlut_sym").to(DEV)
    q.trellis.copy_(t16(lay["codes"]))
    q.tlut.copy_(torch.from_numpy(lay["tlut"]))
    q.SU.copy_(torch.from_numpy(lay["SU"]))
    q.SV.copy_(torch.from_numpy(lay["SV"]))
    y = q(torch.from_numpy(lay["x"]).to(DEV))
    assert y.shape == (1, 4096) and y.dtype == torch.float16
    assert rel_l2(y.float().cpu().numpy(), g["y"]) < 1e-3


@pytest.mark.parametrize("K", [2, 3, 4])
@pytest.mark.parametrize("m,n", [(4096, 11008), (11008, 4096)])
def test_quantized_linear_llama_shapes(K, m, n):
    lay = synth.make_layer(m, n, K, seed=4000 + K)
    q = QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, "quantlut_sym").to(DEV)
    q.trellis.copy_(t16(lay["codes"]))
    q.tlut.copy_(torch.from_numpy(lay["tlut"]))
    q.SU.copy_(torch.from_numpy(lay["SU"]))
    q.SV.copy_(torch.from_numpy(lay["SV"]))
    y = q(torch.from_numpy(lay["x"]).to(DEV))
    hl = None if q.had_left is None else q.had_left.cpu().numpy()
    hr = None if q.had_right is None else q.had_right.cpu().numpy()
    want = C.layer_forward(lay["x"].astype(np.float32), lay["codes"], m, n, K, lay["tlut"],
                           lay["SU"].astype(np.float32), lay["SV"], hl, hr)
    assert rel_l2(y.float().cpu().numpy(), want) < 1e-3


def test_batched_forward_uses_dense_path():
    m, n, K, bs = 512, 1024, 2, 16
    lay = synth.make_layer(m, n, K, seed=77, bs=bs)
    q = QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, "quantlut_sym").to(DEV)
    q.trellis.copy_(t16(lay["codes"]))
    q.tlut.copy_(torch.from_numpy(lay["tlut"]))
    q.SU.copy_(torch.from_numpy(lay["SU"]))
    q.SV.copy_(torch.from_numpy(lay["SV"]))
    y = q(torch.from_numpy(lay["x"]).to(DEV))
    want = C.layer_forward(lay["x"].astype(np.float32), lay["codes"], m, n, K, lay["tlut"],
                           lay["SU"].astype(np.float32), lay["SV"])
    assert rel_l2(y.float().cpu().numpy(), want) < 1e-3


def test_legacy_entry_point_and_graph_capture():
    """The upstream call sequence of lib/codebook/__init__.py:85-92, replayed from a CUDA graph."""
    m, n, K = 4096, 4096, 2
    lay = synth.make_layer(m, n, K, seed=9)
    fn = getattr(qtip_kernels, f"decompress_matvec_16_9_{K}_1_{m}_1_{n}")
    compressed = t16(lay["codes"]).reshape(-1).view(torch.int32)
    x = torch.from_numpy(lay["x"]).to(DEV).T.contiguous()        # (n, 1) fp16
    codebook = torch.from_numpy(lay["tlut"]).to(DEV).reshape(-1)
    out = torch.zeros((m, 1), dtype=torch.float32, device=DEV)
    fn(out, compressed, x, codebook)
    want = C.matvec_kernel(lay["codes"], m, n, K, lay["tlut"], lay["x"])
    assert rel_l2(out.T.cpu().numpy(), want) < 2e-6
    first = out.clone()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    ws = torch.zeros(ops._lib.load().qtip_matvec_workspace_bytes(m, n, 1), dtype=torch.uint8, device=DEV)
    gph = torch.cuda.CUDAGraph()
    out2 = torch.zeros((1, m), dtype=torch.float32, device=DEV)
    with torch.cuda.stream(s):
        ops.decompress_matvec(compressed, x.view(1, n), codebook, K, m, n, out=out2, workspace=ws)  # warm-up
        torch.cuda.current_stream().synchronize()
        with torch.cuda.graph(gph, stream=s):
            ops.decompress_matvec(compressed, x.view(1, n), codebook, K, m, n, out=out2, workspace=ws)
    out2.zero_()
    gph.replay()
    gph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out2.view(-1), first.view(-1))
    with pytest.raises(RuntimeError):
        fn(out, compressed, x.float(), codebook)


@pytest.mark.parametrize("m,n,K", [(4096, 4096, 2), (11008, 4096, 3), (4096, 11008, 4)])
def test_quip_lib_op_on_the_shim(m, n, K):
    """The torch.library op of lib/codebook/__init__.py:68-92 upstream, dispatched on the GPU to this package installed as
    `qtip_kernels`.  With QTIP_REFERENCE_ROOT pointing at a checkout the upstream file itself is imported, unmodified;
    otherwise an op with the same schema and the same call into `qtip_kernels` is registered here."""
    import os
    import sys
    import qtip_b200
    qtip_b200.install_as_qtip_kernels()
    root = os.environ.get("QTIP_REFERENCE_ROOT")
    name = f"decompress_matvec_qtip_{m}_1_{n}_{K}"
    if root and os.path.isdir(os.path.join(root, "lib", "codebook")):
        if root not in sys.path:
            sys.path.insert(0, root)
        import lib.codebook  # noqa: F401  (registers quip_lib::*)
        op = getattr(torch.ops.quip_lib, name)
    else:
        import qtip_kernels as qk            # resolves to the shim
        ns = "qtip_b200_shim_test"
        if not hasattr(getattr(torch.ops, ns), name):
            torch.library.define(f"{ns}::{name}", "(Tensor compressed, Tensor x, Tensor codebook) -> Tensor")

            @torch.library.impl(f"{ns}::{name}", "cuda")
            def _impl(compressed, x, codebook):
                out = torch.zeros((m, 1), dtype=torch.float32, device=x.device)
                getattr(qk, f"decompress_matvec_16_9_{K}_1_{m}_1_{n}")(out, compressed.reshape(-1).view(torch.int32),
                                                                       x.to(torch.float16).T, codebook.reshape(-1))
                return out.T
        op = getattr(getattr(torch.ops, ns), name)
    lay = synth.make_layer(m, n, K, seed=19)
    y = op(t16(lay["codes"]), torch.from_numpy(lay["x"]).to(DEV), torch.from_numpy(lay["tlut"]).to(DEV))
    assert tuple(y.shape) == (1, m) and y.dtype == torch.float32
    want = C.matvec_kernel(lay["codes"], m, n, K, lay["tlut"], lay["x"])
    assert rel_l2(y.cpu().numpy(), want) < 2e-6


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_tensor_parallel_shards_equal_unsharded_layer(tp):
    """Sum (row-parallel) / concatenation (column-parallel) of the per-rank results equals the unsharded
    BitshiftLinear.forward with the matching rcp - all ranks emulated one after the other on one GPU."""
    import math
    from qtip_b200 import tp as tpmod
    K = 2
    tl = None
    # ---- row-parallel: rcp = 1
    m, n = 512, 6656                       # 6656 = 52 * 128; chunks keep the factor 52 down to tp = 8
    lay = synth.make_layer(m, n, K, seed=500 + tp)
    codes, SU, SV = t16(lay["codes"]), torch.from_numpy(lay["SU"]).to(DEV), torch.from_numpy(lay["SV"]).to(DEV)
    tl = torch.from_numpy(lay["tlut"]).to(DEV)
    x = torch.from_numpy(lay["x"]).to(DEV)
    hl, kl = ops.get_hadK(n // tp)
    hr, kr = ops.get_hadK(m)
    hl = None if hl is None else hl.to(DEV)
    bl = BitshiftLinear(16, 16, 16, K, 2, 9, "quantlut_sym", tlut=tl, has_kernel=True)
    want = bl(x, codes, SU, SV, hl, None, kl, kr, 1, tp).float()
    total = torch.zeros(1, m, device=DEV)
    for r in range(tp):
        c_r, su_r, sv_r, n_r = tpmod.shard_row_parallel(codes, SU, SV, m, n, K, r, tp)
        xh = ops.rht(x[:, r * n_r:(r + 1) * n_r].contiguous(), sign_in=su_r.contiguous(), hadk_bits=ops.hadk_bits_for(hl, DEV),
                     kfac=kl, transpose=True, scale=1 / (math.sqrt(n_r) * 32), out_dtype=torch.float16)
        total += ops.decompress_matvec(c_r, xh, tl, K, m, n_r)
    got = ops.rht(total, sign_out=SV * 32, scale=1 / math.sqrt(m), out_dtype=torch.float16).float()
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 1e-3
    # ---- column-parallel: rcp = 2
    m, n = 6656, 512
    lay = synth.make_layer(m, n, K, seed=600 + tp)
    codes, SU, SV = t16(lay["codes"]), torch.from_numpy(lay["SU"]).to(DEV), torch.from_numpy(lay["SV"]).to(DEV)
    tl = torch.from_numpy(lay["tlut"]).to(DEV)
    x = torch.from_numpy(lay["x"]).to(DEV)
    hr, kr = ops.get_hadK(m // tp)
    hr = None if hr is None else hr.to(DEV)
    bl = BitshiftLinear(16, 16, 16, K, 2, 9, "quantlut_sym", tlut=tl, has_kernel=True)
    want = bl(x, codes, SU, SV, None, hr, 1, kr, 2, tp).float()
    xh = ops.rht(x, sign_in=SU, transpose=True, scale=1 / (math.sqrt(n) * 32), out_dtype=torch.float16)
    outs = []
    for r in range(tp):
        c_r, su_r, sv_r, m_r = tpmod.shard_column_parallel(codes, SU, SV, m, n, K, r, tp)
        y = ops.decompress_matvec(c_r.contiguous(), xh, tl, K, m_r, n)
        outs.append(ops.rht(y, sign_out=sv_r.contiguous() * 32, hadk_bits=ops.hadk_bits_for(hr, DEV), kfac=kr,
                            scale=1 / math.sqrt(m_r), out_dtype=torch.float16))
    got = torch.cat(outs, dim=1).float()
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 1e-3


@pytest.mark.parametrize("K", [2, 3, 4])
def test_linear_fused_matches_three_kernel_path(K):
    """qtip_linear_fused (input transform, matvec, output transform in one launch, three linears batched)
    against the separate RHT / matvec / RHT launches."""
    import math
    from qtip_b200 import _lib
    m = n = 4096
    lays = [synth.make_layer(m, n, K, seed=700 + 10 * K + i) for i in range(3)]
    g = torch.Generator().manual_seed(K)
    raw = torch.randn(n, generator=g).half().to(DEV)
    res = torch.randn(n, generator=g).half().to(DEV)
    w = (1 + 0.1 * torch.randn(n, generator=g)).half().to(DEV)
    need = _lib.load().qtip_matvec_workspace_bytes(m, n, 1)
    descs, want, res_want = [], [], None
    res_out = torch.zeros(n, dtype=torch.float16, device=DEV)
    for i, lay in enumerate(lays):
        codes, tl = t16(lay["codes"]), torch.from_numpy(lay["tlut"]).to(DEV)
        SU, SV = torch.from_numpy(lay["SU"]).to(DEV), torch.from_numpy(lay["SV"]).to(DEV) * 32
        xh = torch.zeros(1, n, dtype=torch.float16, device=DEV)
        r2 = torch.zeros(n, dtype=torch.float16, device=DEV)
        ops.rht_fused(raw, 1, n, xh, residual=res, residual_out=r2, norm_weight=w, eps=1e-5, sign_in=SU, transpose=True,
                      scale=1 / (math.sqrt(n) * 32))
        y = ops.decompress_matvec(codes, xh, tl, K, m, n)
        want.append(ops.rht(y, sign_out=SV, scale=1 / math.sqrt(m), out_dtype=torch.float16))
        res_want = r2
        descs.append(dict(y=torch.zeros(m, device=DEV), codes=codes, tlut=tl, workspace=torch.zeros(need, dtype=torch.uint8, device=DEV),
                          in_raw=raw, residual=res, residual_out=res_out if i == 0 else None, norm_weight=w, sign_in=SU,
                          in_scale=1 / (math.sqrt(n) * 32), eps=1e-5, out=torch.zeros(m, dtype=torch.float16, device=DEV),
                          sign_out=SV, out_scale=1 / math.sqrt(m)))
    for _ in range(2):   # twice: the workspace counters must be left ready for the next call
        for d in descs:
            d["out"].zero_()
        ops.linear_fused(descs, K, m, n, 1)
        torch.cuda.synchronize()
        assert torch.equal(res_out, res_want)
        for d, wv in zip(descs, want):
            assert rel_l2(d["out"].float().cpu().numpy(), wv.float().cpu().numpy()) < 1e-3
    # no fusion, two linears in one launch == two single launches
    xs = [torch.from_numpy(l["x"]).to(DEV) for l in lays[:2]]
    plain = [dict(y=torch.zeros(m, device=DEV), codes=d["codes"], tlut=d["tlut"], workspace=d["workspace"], x=x)
             for d, x in zip(descs, xs)]
    ops.linear_fused(plain, K, m, n, 1)
    for d, x in zip(plain, xs):
        assert torch.equal(d["y"].view(1, m), ops.decompress_matvec(d["codes"], x, d["tlut"], K, m, n))


@pytest.mark.parametrize("n", [4096, 8192])
def test_linear_fused_deferred_producer_side(n):
    """in_y: the producer's output side (sign * H(y) * scale, rounded to fp16) computed inside the consumer's
    prologue must equal handing the consumer the materialised fp16 tensor."""
    import math
    from qtip_b200 import _lib
    K, m = 2, 4096
    lay = synth.make_layer(m, n, K, seed=900 + n)
    g = torch.Generator().manual_seed(n)
    y_prev = torch.randn(n, generator=g).to(DEV)                       # raw fp32 result of some producer linear
    sv_prev = (torch.randn(n, generator=g).sign() * 0.37).to(DEV)
    res = torch.randn(n, generator=g).half().to(DEV)
    w = (1 + 0.1 * torch.randn(n, generator=g)).half().to(DEV)
    codes, tl = t16(lay["codes"]), torch.from_numpy(lay["tlut"]).to(DEV)
    SU = torch.from_numpy(lay["SU"]).to(DEV)
    need = _lib.load().qtip_matvec_workspace_bytes(m, n, 1)
    delta = ops.rht(y_prev.view(1, n), sign_out=sv_prev, scale=1 / math.sqrt(n), out_dtype=torch.float16).view(n)
    common = dict(codes=codes, tlut=tl, residual=res, norm_weight=w, sign_in=SU, in_scale=1 / (math.sqrt(n) * 32), eps=1e-5)
    a = dict(common, y=torch.zeros(m, device=DEV), workspace=torch.zeros(need, dtype=torch.uint8, device=DEV),
             in_raw=delta, residual_out=torch.zeros(n, dtype=torch.float16, device=DEV))
    b = dict(common, y=torch.zeros(m, device=DEV), workspace=torch.zeros(need, dtype=torch.uint8, device=DEV),
             in_y=y_prev, in_y_sign=sv_prev, in_y_scale=1 / math.sqrt(n),
             residual_out=torch.zeros(n, dtype=torch.float16, device=DEV))
    ops.linear_fused([a], K, m, n, 1)
    for _ in range(2):
        ops.linear_fused([b], K, m, n, 1)
        torch.cuda.synchronize()
        # the two transforms sum in different orders: fp16 roundings of the intermediate may differ in the last bit
        assert rel_l2(b["residual_out"].float().cpu().numpy(), a["residual_out"].float().cpu().numpy()) < 1e-3
        assert rel_l2(b["y"].cpu().numpy(), a["y"].cpu().numpy()) < 2e-3


@pytest.mark.parametrize("heads", [(32, 32), (32, 8), (64, 8)])
def test_rope_kv_append_fused_matches_separate_launches(heads):
    """qtip_rope_kv_append_fused == output-side RHT of q/k/v + qtip_rope_kv_append."""
    import math
    n_heads, n_kv = heads
    hd, pos_v, maxpos = 128, 5, 8
    H, KV = n_heads * hd, n_kv * hd
    g = torch.Generator().manual_seed(n_heads * 100 + n_kv)
    y = [torch.randn(w, generator=g).to(DEV) for w in (H, KV, KV)]
    sv = [(torch.randn(w, generator=g).sign() * 0.5).to(DEV) for w in (H, KV, KV)]
    pos = torch.tensor([pos_v], dtype=torch.int32, device=DEV)
    q, k, v = [ops.rht(t.view(1, -1), sign_out=s_, scale=1 / math.sqrt(t.numel()), out_dtype=torch.float16).view(-1)
               for t, s_ in zip(y, sv)]
    ck, cv = [torch.zeros(maxpos, KV, dtype=torch.float16, device=DEV) for _ in range(2)]
    ops.rope_kv_append(q, k, v, ck, cv, pos, n_heads, n_kv, hd, 10000.0)
    q2 = torch.zeros(H, dtype=torch.float16, device=DEV)
    ck2, cv2 = [torch.zeros(maxpos, KV, dtype=torch.float16, device=DEV) for _ in range(2)]
    ops.rope_kv_append_fused(q2, y[0], y[1], y[2], sv[0], sv[1], sv[2], 1 / math.sqrt(H), 1 / math.sqrt(KV), ck2, cv2, pos,
                             n_heads, n_kv, hd, 10000.0)
    torch.cuda.synchronize()
    for got, want in ((q2, q), (ck2, ck), (cv2, cv)):
        assert rel_l2(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1e-3
    assert torch.count_nonzero(ck2[:pos_v]) == 0 and torch.count_nonzero(ck2[pos_v + 1:]) == 0


@pytest.mark.parametrize("n", [11008, 5504, 1376, 3328])
def test_mlp_mid_matches_two_rht_launches(n):
    """qtip_mlp_mid (tensor-core Hadamard factor, one cluster launch) against the output-side RHT of gate and up
    followed by the SwiGLU + input-side RHT of down_proj.  Widths: 172*64, 172*32, 172*8 (unsupported row length:
    must be refused), 52*64."""
    import math
    g = torch.Generator().manual_seed(n)
    y_g, y_u = [(torch.randn(n, generator=g) * 3).to(DEV) for _ in range(2)]
    sv_g, sv_u = [(torch.randn(n, generator=g).sign() * 1.7).to(DEV) for _ in range(2)]
    su = torch.randn(n, generator=g).sign().half().to(DEV)
    out = torch.zeros(n, dtype=torch.float16, device=DEV)
    if not ops.mlp_mid_supported(n):
        assert n == 1376
        with pytest.raises(RuntimeError):
            ops.mlp_mid(out, y_g, y_u, sv_g, sv_u, su, n, 1 / math.sqrt(n), 1 / (32 * math.sqrt(n)))
        return
    hadK, kfac = ops.get_hadK(n)
    bits = ops.hadk_bits_for(hadK, torch.device(DEV))
    gu = torch.zeros(2, n, dtype=torch.float16, device=DEV)
    ops.rht_fused(torch.stack([y_g, y_u]), 2, n, gu, sign_out=torch.cat([sv_g, sv_u]), hadk_bits=bits, kfac=kfac,
                  scale=1 / math.sqrt(n))
    want = torch.zeros(n, dtype=torch.float16, device=DEV)
    ops.rht_fused(gu[1], 1, n, want, gate=gu[0], sign_in=su, hadk_bits=bits, kfac=kfac, transpose=True,
                  scale=1 / (32 * math.sqrt(n)))
    for _ in range(2):
        out.zero_()
        ops.mlp_mid(out, y_g, y_u, sv_g, sv_u, su, n, 1 / math.sqrt(n), 1 / (32 * math.sqrt(n)))
        torch.cuda.synchronize()
        # fp16 roundings of g, u may fall on the other side in a few places (different summation order)
        assert rel_l2(out.float().cpu().numpy(), want.float().cpu().numpy()) < 2e-3


@pytest.mark.parametrize("heads", [(32, 32), (32, 8), (4, 4), (8, 1)])
@pytest.mark.parametrize("pos_v", [0, 1, 37, 300])
def test_attn_decode_fused_matches_separate_launches(heads, pos_v):
    """qtip_attn_decode_fused == output-side RHT of q/k/v + rotary / cache append + attention."""
    import math
    n_heads, n_kv = heads
    hd, maxpos = 128, 304
    H, KV = n_heads * hd, n_kv * hd
    g = torch.Generator().manual_seed(n_heads * 1000 + n_kv * 10 + pos_v)
    y = [torch.randn(w, generator=g).to(DEV) for w in (H, KV, KV)]
    sv = [(torch.randn(w, generator=g).sign() * 0.5).to(DEV) for w in (H, KV, KV)]
    pos = torch.tensor([pos_v], dtype=torch.int32, device=DEV)
    ck = (0.5 * torch.randn(maxpos, KV, generator=g)).half().to(DEV)
    cv = (0.5 * torch.randn(maxpos, KV, generator=g)).half().to(DEV)
    ck2, cv2 = ck.clone(), cv.clone()
    q, k, v = [ops.rht(t.view(1, -1), sign_out=s_, scale=1 / math.sqrt(t.numel()), out_dtype=torch.float16).view(-1)
               for t, s_ in zip(y, sv)]
    ops.rope_kv_append(q, k, v, ck, cv, pos, n_heads, n_kv, hd, 10000.0)
    want = torch.zeros(n_heads, hd, dtype=torch.float16, device=DEV)
    ops.attn_decode(want, q, ck, cv, pos, n_heads, n_kv, hd)
    got = torch.zeros(n_heads, hd, dtype=torch.float16, device=DEV)
    ops.attn_decode_fused(got, y[0], y[1], y[2], sv[0], sv[1], sv[2], 1 / math.sqrt(H), 1 / math.sqrt(KV), ck2, cv2, pos,
                          n_heads, n_kv, hd, 10000.0)
    torch.cuda.synchronize()
    assert rel_l2(got.float().cpu().numpy(), want.float().cpu().numpy()) < 2e-3
    # the cache rows: the new one equal up to fp16 rounding of the transform, every other untouched
    assert rel_l2(ck2[pos_v].float().cpu().numpy(), ck[pos_v].float().cpu().numpy()) < 1e-3
    assert rel_l2(cv2[pos_v].float().cpu().numpy(), cv[pos_v].float().cpu().numpy()) < 1e-3
    keep = torch.ones(maxpos, dtype=torch.bool, device=DEV)
    keep[pos_v] = False
    assert torch.equal(ck2[keep], ck[keep]) and torch.equal(cv2[keep], cv[keep])


def test_linear_fused_peer_sum_and_signal():
    """Tensor parallelism without an all-reduce launch, emulated on one GPU: the producer stores its result as
    stamped values and advances the sequence counter; the consumer adds two stamped vectors once their stamps are
    current; a vector that nobody refreshes makes the (bounded) wait give up with a status instead of hanging."""
    import math
    from qtip_b200 import _lib
    K, m, n = 2, 4096, 4096
    lay = synth.make_layer(m, n, K, seed=4242)
    g = torch.Generator().manual_seed(11)
    codes, tl = t16(lay["codes"]), torch.from_numpy(lay["tlut"]).to(DEV)
    need = _lib.load().qtip_matvec_workspace_bytes(m, n, 1)
    ws = lambda: torch.zeros(need, dtype=torch.uint8, device=DEV)   # noqa: E731

    def stamped(vec, stamp):
        pairs = torch.empty(vec.numel(), 2, dtype=torch.int32, device=DEV)
        pairs[:, 0] = vec.view(torch.int32)
        pairs[:, 1] = stamp
        return pairs

    # producer side: plain linear + two stamped copies
    sig_seq = torch.tensor([6], dtype=torch.int32, device=DEV)
    copies = [torch.zeros(m, 2, dtype=torch.int32, device=DEV) for _ in range(2)]
    x = torch.from_numpy(lay["x"]).to(DEV)
    prod = dict(y=torch.zeros(m, device=DEV), codes=codes, tlut=tl, workspace=ws(), x=x, signal_seq=sig_seq.data_ptr(),
                signal_y=[c.data_ptr() for c in copies])
    for it in (7, 8):
        ops.linear_fused([prod], K, m, n, 1)
        torch.cuda.synchronize()
        assert int(sig_seq) == it
        # the plain launch runs 16 decoding warps, this one 32: same products, another summation order
        plain = ops.decompress_matvec(codes, x, tl, K, m, n)
        assert rel_l2(prod["y"].view(1, m).cpu().numpy(), plain.cpu().numpy()) < 2e-6
        for c in copies:
            assert torch.equal(c, stamped(prod["y"], it))

    # consumer side
    parts = [torch.randn(n, generator=g).to(DEV) for _ in range(2)]
    sv_prev = (torch.randn(n, generator=g).sign() * 0.4).to(DEV)
    res = torch.randn(n, generator=g).half().to(DEV)
    w = (1 + 0.1 * torch.randn(n, generator=g)).half().to(DEV)
    SU = torch.from_numpy(lay["SU"]).to(DEV)
    common = dict(codes=codes, tlut=tl, residual=res, norm_weight=w, sign_in=SU, in_scale=1 / (math.sqrt(n) * 32), eps=1e-5,
                  in_y_sign=sv_prev, in_y_scale=1 / math.sqrt(n))
    want = dict(common, y=torch.zeros(m, device=DEV), workspace=ws(), in_y=parts[0] + parts[1])
    ops.linear_fused([want], K, m, n, 1)
    seq = torch.tensor([5], dtype=torch.int32, device=DEV)
    vecs = [stamped(parts[0], 5), stamped(parts[1], 5)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = dict(common, y=torch.zeros(m, device=DEV), workspace=ws(), peer_y=[v.data_ptr() for v in vecs],
               peer_seq=seq.data_ptr(), peer_status=status.data_ptr())
    ops.linear_fused([got], K, m, n, 1)
    torch.cuda.synchronize()
    assert int(status) == 0 and torch.equal(got["y"], want["y"])
    # one value with an old stamp: the wait runs out after 2000 re-reads, the kernel still terminates
    vecs[1][1234, 1] = 4
    got["peer_max_polls"] = 2000
    ops.linear_fused([got], K, m, n, 1)
    torch.cuda.synchronize()
    assert int(status) == 1
    # a launch AFTER a recorded run-out does not wait again: every stamp stale (a lost GPU), default limits, and the
    # launch still returns at once (the 200 ms time bound is never reached) with the status word left set
    for v in vecs:
        v[:, 1] = 3
    got.pop("peer_max_polls")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ops.linear_fused([got], K, m, n, 1)
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 50.0, "a launch after a recorded time-out polled again"
    assert int(status) != 0


def test_quip_lib_op_under_graph_capture():
    """The torch op boundary (lib/codebook/__init__.py:68-93 upstream): eager call and CUDA-graph replay."""
    from qtip_b200 import codebook_ops
    m, n, K = 4096, 4096, 3
    lay = synth.make_layer(m, n, K, seed=21)
    op = codebook_ops.register(m, n, K)
    trellis, tl = t16(lay["codes"]), torch.from_numpy(lay["tlut"]).to(DEV)
    x = torch.from_numpy(lay["x"]).to(DEV).float()
    y = op(trellis, x, tl)
    want = C.matvec_kernel(lay["codes"], m, n, K, lay["tlut"], lay["x"])
    assert y.shape == (1, m) and rel_l2(y.cpu().numpy(), want) < 2e-6
    ops.matvec_workspace(m, n, 1, DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        op(trellis, x, tl)
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            y2 = op(trellis, x, tl)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y2, y)


def test_cache_hatw_dense_path_matches_fused_path():
    """train-fixW (dense manifest, lib/codebook/bitshift.py:389-413 upstream) against the fused eval path."""
    m, n, K = 1376, 512, 2
    lay = synth.make_layer(m, n, K, seed=33, bs=3)
    q = QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, "quantlut_sym").to(DEV)
    qd = QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, "quantlut_sym", mode="train-fixW").to(DEV)
    for mod in (q, qd):
        mod.trellis.copy_(t16(lay["codes"])); mod.tlut.copy_(torch.from_numpy(lay["tlut"]))
        mod.SU.copy_(torch.from_numpy(lay["SU"])); mod.SV.copy_(torch.from_numpy(lay["SV"]))
    x = torch.from_numpy(lay["x"]).to(DEV)
    assert rel_l2(qd(x).float().cpu().numpy(), q(x).float().cpu().numpy()) < 3e-3
