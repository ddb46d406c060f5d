"""Per-layer sweep of the fused decode-matvec (and the other kernels) on synthetic weights.

    python -m qtip_b200.microbench                       # Llama-2-7B shapes, K = 2, 3, 4, batch 1
    python -m qtip_b200.microbench --shapes 8192x8192,28672x8192 --bits 2 --batch 1,4,8
    python -m qtip_b200.microbench --shapes 8192x8192 --bits 2 --batch 16,64         # tcgen05 decompress-GEMM
    python -m qtip_b200.microbench --mlp-mid 11008 --rht 11008                        # transform kernels
    python -m qtip_b200.microbench --shapes 4096x11008 --bits 2 --plain-launches 8   # for a profiler

Timing method (the one of qtip-kernels/test_decompress_matvec.py:69-91 upstream, scaled up): the
launches of one measurement walk over enough distinct weight sets to exceed the 126 MB L2, are
captured in one CUDA graph, and the graph is replayed between two CUDA events.  GB/s counts the
algorithmic bytes m*n*K/8 + 2*bs*(m+n).  Shapes are written out_features x in_features.
"""
import argparse
import json

import torch

from . import _lib, ops, synth

LLAMA7B = "4096x4096,11008x4096,4096x11008"
_PLAIN_MATVEC = False   # --plain-matvec: time qtip_decompress_matvec_plain instead of the tensor-core kernel (batch <= 8)


def _sets(m, n, K, bs, code, device, min_bytes=400e6, max_sets=48):
    per = m * n * K // 8
    nset = int(min(max_sets, max(3, min_bytes // per)))
    return [synth.make_layer(m, n, K, seed=i, bs=bs, code=code, device=device) for i in range(nset)]


def _launch(lay, code, K, m, n, out, ws):
    if code == "hyb" and lay["x"].shape[0] > ops.MAX_MATVEC_BATCH:
        ops.decompress_gemm(lay["codes"], lay["x"], lay["tlut"], K, m, n, out=out)      # tcgen05 path, batches 9..128
    elif code == "hyb":
        ops.decompress_matvec(lay["codes"], lay["x"], lay["tlut"], K, m, n, out=out, workspace=ws)
    elif ops.gemm_plain_supported(m, n, lay["x"].shape[0]) and not _PLAIN_MATVEC:
        ops.decompress_gemm_plain(lay["codes"], lay["x"], code, K, m, n, out=out)      # compute codes on the tcgen05 path
    else:
        ops.decompress_matvec_plain(lay["codes"], lay["x"], code, K, m, n, out=out, workspace=ws)


def time_matvec(m, n, K, bs=1, code="hyb", device="cuda:0", replays=20):
    lays = _sets(m, n, K, bs, code, device)
    ws = torch.zeros(_lib.load().qtip_matvec_workspace_bytes(m, n, min(bs, ops.MAX_MATVEC_BATCH)), dtype=torch.uint8, device=device)
    out = torch.empty(bs, m, device=device)
    stream = torch.cuda.Stream(device=device)
    stream.wait_stream(torch.cuda.current_stream(device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        _launch(lays[0], code, K, m, n, out, ws)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for lay in lays:
                _launch(lay, code, K, m, n, out, ws)
    torch.cuda.current_stream(device).wait_stream(stream)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / (replays * len(lays))
    byts = m * n * K / 8 + 2 * bs * (m + n)
    return dict(code=code, K=K, m=m, n=n, bs=bs, us=us, gbs=byts / us / 1e3, weight_sets=len(lays))


def plain_launches(m, n, K, bs, code, count, device="cuda:0"):
    """`count` ordinary stream launches over rotating weight sets (what a profiler should capture)."""
    lays = _sets(m, n, K, bs, code, device, min_bytes=160e6, max_sets=14)
    ws = torch.zeros(_lib.load().qtip_matvec_workspace_bytes(m, n, min(bs, ops.MAX_MATVEC_BATCH)), dtype=torch.uint8, device=device)
    out = torch.empty(bs, m, device=device)
    for i in range(count):
        _launch(lays[i % len(lays)], code, K, m, n, out, ws)
    torch.cuda.synchronize(device)


def time_rht(n, rows=1, device="cuda:0", replays=20, launches=32, plain=0, mid=False):
    """Input-side transform (fp16 in, SwiGLU gate, signs, fp16 out) of `rows` rows of width n; mid=True times
    qtip_mlp_mid (gate/up output side + SwiGLU + down input side) instead."""
    import math
    k = ops.had_factor(n)
    bits = None if k == 1 else ops.pack_hadk(ops.get_hadK(n)[0].to(device))
    x = torch.randn(rows, n, device=device).half()
    gate = torch.randn(rows, n, device=device).half()
    su = torch.ones(n, device=device, dtype=torch.float16)
    out = torch.empty(rows, n, device=device, dtype=torch.float16)
    y_g, y_u, sv = (torch.randn(n, device=device) for _ in range(3))

    def launch():
        if mid:
            ops.mlp_mid(out, y_g, y_u, sv, sv, su, n, 1 / math.sqrt(n), 1 / math.sqrt(n))
        else:
            ops.rht_fused(x, rows, n, out, gate=gate, sign_in=su, hadk_bits=bits, kfac=k, transpose=True, scale=1 / math.sqrt(n))

    if plain:
        for _ in range(plain):
            launch()
        torch.cuda.synchronize(device)
        return None
    stream = torch.cuda.Stream(device=device)
    stream.wait_stream(torch.cuda.current_stream(device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        launch()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                launch()
    torch.cuda.current_stream(device).wait_stream(stream)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) * 1e3 / (replays * launches)


def time_viterbi(N):
    """Sequences per second of qtip_viterbi_quantize (CUDA events around one call after a warm-up call)."""
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(11)
    X = torch.randn(N, 256, generator=g, device=dev).half()
    tlut = torch.randn(512, 2, generator=g, device=dev)
    for mode, Ks in (("quantlut_sym", (2, 3, 4)), ("3inst", (2, 3, 4)), ("1mad", (2,))):
        for K in Ks:
            ops.viterbi_quantize(X[:256], mode, K, tlut=tlut)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _, cost = ops.viterbi_quantize(X, mode, K, tlut=tlut, return_cost=True)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            V = 2 if mode == "quantlut_sym" else 1
            evals = 2.0 * N * (256 // V) * 65536          # candidate evaluations: two passes, 2^16 per step
            print(f"viterbi {mode} K={K}: {N} sequences in {ms:8.2f} ms = {N / ms * 1e3:9.0f} sequences/s, "
                  f"{evals / ms / 1e9:6.2f} T candidate evaluations/s, mean squared error {float(cost.sum()) / (N * 256):.4f}",
                  flush=True)


def pipe_rates():
    """The ceiling of the decode kernels: what the integer pipes, the shared-memory gather and the legacy MMA issue per clock."""
    import ctypes
    from . import _lib
    lib = _lib.load()
    n = lib.qtip_pipe_rate_count()
    for threads in (1024, 512):
        buf = (ctypes.c_double * n)()
        _lib.check(lib.qtip_measure_pipe_rates(buf, n, threads), "qtip_measure_pipe_rates")
        for i in range(n):
            name = lib.qtip_pipe_rate_name(i).decode()
            unit = "state" if "per state" in name else "warp-instruction"
            print(f"{threads // 32:2d} warps/SM  {name:55s} {buf[i]:6.2f} cycles per {unit} per sub-partition", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mlp-mid", default="", help="comma-separated widths: time qtip_mlp_mid")
    ap.add_argument("--rht", default="", help="comma-separated widths: time the transform kernel instead of the matvec")
    ap.add_argument("--shapes", default=LLAMA7B)
    ap.add_argument("--bits", default="2,3,4")
    ap.add_argument("--batch", default="1")
    ap.add_argument("--code", default="hyb", choices=["hyb", "3inst", "1mad"])
    ap.add_argument("--plain-launches", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--viterbi", type=int, default=0, metavar="N",
                    help="time the tail-biting Viterbi quantizer on N sequences of 256 values for every code / bitrate")
    ap.add_argument("--pipes", action="store_true",
                    help="issue rates of the instruction classes the decoders are made of (cycles per warp-instruction per "
                         "SM sub-partition), with 32 and 16 warps per SM")
    ap.add_argument("--plain-matvec", action="store_true",
                    help="compute codes, batch <= 8: time the mma.sync matvec instead of the tcgen05 kernel")
    args = ap.parse_args()
    if args.pipes:
        pipe_rates()
        return
    if args.viterbi:
        time_viterbi(args.viterbi)
        return
    global _PLAIN_MATVEC
    _PLAIN_MATVEC = args.plain_matvec
    peak = None
    try:
        import os
        peak = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                           "MEASURED_PEAKS.json")))["hbm_gbs"]
    except (OSError, KeyError):
        pass
    if args.mlp_mid:
        for n in (int(v) for v in args.mlp_mid.split(",")):
            us = time_rht(n, plain=args.plain_launches, mid=True)
            if us is not None:
                print(f"mlp_mid n={n} (factor {ops.had_factor(n)}): {us:7.2f} us per launch (back-to-back launches in one graph)", flush=True)
        if not args.rht:
            return
    if args.rht:
        for n in (int(v) for v in args.rht.split(",")):
            us = time_rht(n, plain=args.plain_launches)
            if us is not None:
                print(f"rht n={n} (factor {ops.had_factor(n)}): {us:7.2f} us per launch (back-to-back launches in one graph)", flush=True)
        return
    rows = []
    for K in (int(b) for b in args.bits.split(",")):
        for shape in args.shapes.split(","):
            m, n = (int(v) for v in shape.split("x"))
            for bs in (int(b) for b in args.batch.split(",")):
                if args.plain_launches:
                    plain_launches(m, n, K, bs, args.code, args.plain_launches)
                    continue
                r = time_matvec(m, n, K, bs, args.code)
                rows.append(r)
                frac = f"  {100 * r['gbs'] / peak:5.1f}% of measured HBM peak" if peak else ""
                if not args.json:
                    print(f"{args.code} K={K} {m}x{n} bs={bs}: {r['us']:8.2f} us  {r['gbs']:7.0f} GB/s{frac}", flush=True)
    if args.json:
        print(json.dumps(rows))


if __name__ == "__main__":
    main()
