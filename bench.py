#!/usr/bin/env python
"""Benchmark: batch-1 decode tokens/s of a random-init Llama-2-7B-shaped model whose linears are all
2-bit HYB QTIP layers (128-token prompt, then timed decode steps from one CUDA graph), plus the
roofline of the dominant kernel (the fused decode-matvec) and a CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl qtip_b200|reference]

One JSON line on stdout (rank 0).  A "step" is one decoded token.  Under torchrun (N > 1) each rank
drives one GPU.  `--impl reference` times the CPU port of the upstream path (oracle/) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# The CPU legs use every host core whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1): set before any
# OpenMP / BLAS runtime is loaded.
if "--impl" in sys.argv and "reference" in sys.argv:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

METRIC = "bs=1 decode tok/s (Llama-2-7B-shape, 2-bit HYB)"
PROMPT_TOKENS = 128
PUBLISHED_TOK_S = 188.0  # upstream README.md:31-38, Llama-2-7B 2-bit on an RTX 6000 Ada (fused q/k/v and up/gate)
# DRAM bytes (read + write) of one decode-matvec launch per layer shape, from an ncu capture of the same kernel
# instantiation on plain launches over rotating weights (dram__bytes_read.sum + dram__bytes_write.sum)
NCU_TRAFFIC_BYTES = {(4096, 4096): 4536405, (11008, 4096): 11697152, (4096, 11008): 11798443, (12288, 4096): 13007189,
                     (22016, 4096): 22975915}
WORKLOADS = {
    "llama2-7b": dict(name="Llama-2-7B", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=32, head_dim=128, mlp=11008,
                      vocab=32000, rope_theta=10000.0),
    "llama3-405b": dict(name="Llama-3.1-405B", n_layers=126, hidden=16384, n_heads=128, n_kv_heads=8, head_dim=128,
                        mlp=53248, vocab=128256, rope_theta=500000.0),
}


def workload_config(workload, prompt, world, fused=False):
    w = WORKLOADS[workload]
    cfg = {"workload": (f"{w['name']} shape ({w['n_layers']} layers, hidden {w['hidden']}, {w['n_heads']} heads, MLP {w['mlp']}, "
                        f"vocab {w['vocab']}), every linear 2-bit HYB QTIP (L=16, Q=9, V=2, 16x16 tiles), "
                        f"batch 1, {prompt}-token prompt, CUDA-graph decode"),
           "l2": "each step streams all packed codes (1.6 GB for the 7B shape) and the lm_head, far larger than L2",
           "parallelism": f"tp{world}"}
    if fused:
        cfg["fused_matrices"] = "q||k||v and gate||up as one matrix each"
    return cfg


def use_fused_matrices(args):
    """q||k||v and gate||up as ONE packed matrix each - the layers upstream's published decode speed was measured with -
    is the default where it applies: the 7B shape (equal q / k / v widths) on one GPU at batch 1.  Both arms follow it."""
    return (not args.separate_qkv and args.workload == "llama2-7b" and args.gpus == 1 and args.batch == 1
            and int(os.environ.get("WORLD_SIZE", "1")) == 1)


def metric_name(workload):
    return METRIC if workload == "llama2-7b" else METRIC.replace("Llama-2-7B", "Llama-3.1-405B")


def llama7b_linears():
    """(m, n) of the seven linears of a decoder layer: q, k, v, o, gate, up, down."""
    return [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]


def algorithmic_bytes(m, n, K, bs=1):
    """Packed codes read once plus fp16 activations in and out (per layer call)."""
    return m * n * K // 8 + 2 * bs * (m + n)


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------
# CPU port of the upstream path (oracle/): the reference arm, and (through it) the reported CPU baseline
# ---------------------------------------------------------------------------------------------------------
def _hadk_loader():
    """Hadamard factor matrices from the package's data file, without importing torch."""
    import numpy as np
    cache = {}
    factors = (172, 156, 140, 124, 116, 108, 60, 52, 36, 28, 20, 12)

    def hadk(n):
        for k in factors:
            if n % k == 0 and ((n // k) & (n // k - 1)) == 0:
                if k not in cache:
                    with np.load(os.path.join(ROOT, "qtip_b200", "data", "hadk.npz")) as z:
                        cache[k] = (np.unpackbits(z[f"had{k}"])[:k * k].reshape(k, k).astype(np.float32) * 2 - 1)
                return cache[k]
        return None
    return hadk


def run_reference(args):
    """The upstream decode step on the host cores (C restatement of the QTIP linears with OpenMP, numpy for the rest):
    every step is one full token - all layers, attention over the prompt-long KV cache, lm_head, sampling."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import c_oracle as C
    from llama_oracle import OracleLlama
    threads = C.use_all_cores()
    w = dict(WORKLOADS[args.workload])
    w.pop("name")
    layers_timed, scale = w["n_layers"], 1.0
    sample = ("every step is one full decoded token on the host: all decoder layers (RMSNorm, q/k/v/o/gate/up/down through the "
              "C restatement of BitshiftLinear.forward, rotary embedding, attention over the KV cache, SwiGLU), final norm, "
              "fp16 lm_head, top-k sampling; the KV cache is pre-filled with synthetic keys/values for the prompt positions "
              "instead of running the prompt; layers cycle through 4 distinct weight sets")
    if args.workload == "llama3-405b":
        layers_timed, scale = 2, w["n_layers"] / 2.0
        sample = f"2 of the {w['n_layers']} decoder layers per step, time scaled by {scale:g}; " + sample
        w["n_layers"] = layers_timed
    steps, warmup = args.steps, args.warmup
    fused = use_fused_matrices(args)
    model = OracleLlama(_hadk_loader(), max_positions=args.prompt + warmup + steps + 8,
                        weight_sets=4 if args.workload == "llama2-7b" else 1, fuse_qkv=fused, **w)
    model.fill_cache(args.prompt)
    tok, per_step = 1, []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        tok = model.step(tok)
        if i >= warmup:
            per_step.append((time.perf_counter() - t0) * scale)
    ms = statistics.mean(per_step) * 1e3
    value = 1e3 / ms
    out = {"impl": "reference", "metric": metric_name(args.workload), "value": value, "unit": "tok/s", "n_gpus": args.gpus,
           "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
           "dtype": "f16", "data": "synthetic", "config": workload_config(args.workload, args.prompt, args.gpus, fused),
           "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def cpu_baseline_subprocess(args, steps=4, warmup=1):
    """The reference arm in a fresh process (no CUDA context, no second OpenMP runtime in the way), a few steps."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(steps), "--warmup", str(warmup),
           "--prompt", str(args.prompt), "--workload", args.workload] + (["--separate-qkv"] if args.separate_qkv else [])
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "OMP_NUM_THREADS")}
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
        cb = json.loads(line)["cpu_baseline"]
        cb["sample"] = f"{steps} steps after {warmup} warm-up; " + cb["sample"]
        return cb
    except Exception as e:   # the baseline is reported context, never a reason to lose the GPU line
        return {"value": None, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {e!r}"}


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
def measure_matvec_roofline(model, torch, reps=5):
    """Average duration of one fused decode-matvec launch: all 7 x n_layers launches of a token, every one on
    its own weights (1.6 GB in total, far beyond L2), captured in one graph and timed with CUDA events."""
    from qtip_b200 import ops
    s = model.shape
    dev = model.device
    names = model.linear_names
    widths = {d for L in model.layers[:1] for name in names for d in (L[name].m, L[name].n)}
    xh = {n: torch.randn(n, device=dev).half() for n in widths}
    ys = {m: torch.zeros(m, dtype=torch.float32, device=dev) for m in widths}

    def all_matvecs():
        for L in model.layers:
            for name in names:
                lin = L[name]
                ops.decompress_matvec(lin.codes, xh[lin.n], lin.tlut, lin.K, lin.m, lin.n, out=ys[lin.m].view(1, -1),
                                      workspace=model.workspace)

    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(stream):
        all_matvecs()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            all_matvecs()
    torch.cuda.current_stream(dev).wait_stream(stream)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    launches = len(names) * s.n_layers
    us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
    byts = sum(algorithmic_bytes(L[name].m, L[name].n, s.K) for L in model.layers[:1] for name in names) / len(names)
    return us, byts, launches


def measure_issue_ceiling(torch, K, sm_mhz):
    """What the SM's pipes allow the decode kernel at most, measured live: the per-state decode sequence (funnel shift,
    multiply-add hash, mask, multiply-add address, lane-private shared load) as a pure loop on every SM, in cycles per
    state per sub-partition; 16 states per 128*K-byte block on 4 sub-partitions -> GB/s over all SMs at the sampled clock."""
    import ctypes
    from qtip_b200 import _lib
    lib = _lib.load()
    n = lib.qtip_pipe_rate_count()
    buf = (ctypes.c_double * n)()
    if lib.qtip_measure_pipe_rates(buf, n, 1024) != 0:
        return None
    names = [lib.qtip_pipe_rate_name(i).decode() for i in range(n)]
    cyc = next(buf[i] for i, nm in enumerate(names) if nm.startswith("decode sequence per state (shf"))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    gbs = 128 * K / (16 * cyc / 4) * sms * sm_mhz * 1e6 / 1e9
    return {"cycles_per_state_per_subpartition": cyc, "gbs": gbs,
            "what": "upper bound of any kernel that decodes one trellis state per table lookup: the decode instructions alone, "
                    "no MMA, reduction or loop control (integer multiply-add, logic and shift instructions issue at one per "
                    "two cycles per sub-partition on this part)"}


def measure_layer_e2e(torch, K=2, m=4096, n=4096, reps=200):
    """One QTIP linear through the module the reference defines (QuantizedLinear.forward) with HOST buffers: per call
    the activation goes pinned host -> device, the layer runs (transform in, decode-matvec, transform out), the
    result comes back to pinned host memory and the stream is synchronised.  Returns (us per call, h2d, d2h bytes)."""
    from qtip_b200 import synth
    from qtip_b200.quantized_linear import QuantizedLinear
    dev = torch.device("cuda", torch.cuda.current_device())
    lay = synth.make_layer(m, n, K, seed=77, device=dev)
    q = QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, "quantlut_sym").to(dev)
    q.trellis.copy_(lay["codes"].view(torch.int16)); q.tlut.copy_(lay["tlut"]); q.SU.copy_(lay["SU"]); q.SV.copy_(lay["SV"])
    hx = torch.randn(1, n).half().pin_memory()
    hy = torch.empty(1, m, dtype=torch.float16).pin_memory()
    dx = torch.empty(1, n, dtype=torch.float16, device=dev)
    for _ in range(5):
        dx.copy_(hx, non_blocking=True); hy.copy_(q(dx), non_blocking=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        dx.copy_(hx, non_blocking=True)
        hy.copy_(q(dx), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    return (time.perf_counter() - t0) * 1e6 / reps, hx.numel() * 2, hy.numel() * 2


def measure_decoder_gbs(torch, K=2, m=4096, n=11008):
    """qtip_decode_hyb (packed codes -> dense fp16 matrix): GB/s over the bytes it must move, K*m*n/8 in + 2*m*n out."""
    from qtip_b200 import ops, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    lays = [synth.make_layer(m, n, K, seed=900 + i, device=dev) for i in range(8)]
    W = torch.empty(m, n, dtype=torch.float16, device=dev)
    for lay in lays:
        ops.decode_hyb(lay["codes"], lay["tlut"], K, m, n, out=W)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(4):
        for lay in lays:
            ops.decode_hyb(lay["codes"], lay["tlut"], K, m, n, out=W)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 32
    return (K * m * n / 8 + 2 * m * n) / us / 1e3, us


def run_gpu_batch(args, model, torch, dist, world, rank, dev):
    """--batch B: B sequences decoded in lockstep (QtipLlama.step_batch, one CUDA graph per step).  The KV caches are
    brought to the prompt length by decoding (every sequence samples its own tokens)."""
    B, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
    model.enable_batch(B)
    model.b_token.copy_(torch.arange(B, device=dev) * 7 + 3)
    model.capture_batch()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with ClockSampler(int(dev.split(":")[1])) as clocks:
        model.steps_done = 0
        model.generate_batch(args.prompt + warmup)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.generate_batch(steps)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        h_tok = torch.zeros(B, dtype=torch.int64).pin_memory()
        h_out = torch.zeros(B, dtype=torch.int64).pin_memory()
        h_tok.copy_(model.b_token.cpu())
        barrier()
        model._reserve(steps)
        t0 = time.perf_counter()
        for _ in range(steps):
            model.b_token.copy_(h_tok, non_blocking=True)
            model.b_graph.replay()
            h_out.copy_(model.b_token, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            h_tok.copy_(h_out)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    model.check_status()
    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    if rank == 0:
        cfg = workload_config(args.workload, args.prompt, world)
        cfg["workload"] = cfg["workload"].replace("batch 1", f"batch {B} (sequences in lockstep)")
        out = {"metric": metric_name(args.workload).replace("bs=1", f"bs={B}"), "value": B * steps / (ms / 1e3), "unit": "tok/s",
               "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
               "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
               "config": cfg, "roofline": None, "cpu_baseline": None,
               "e2e": {"value": B * steps / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
               "gpu_launches": model.n_launches_per_batch_step * steps, "clocks": clocks.summary()}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        model.release_graph()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from qtip_b200.llama import LLAMA2_7B, LLAMA3_405B, QtipLlama
    shape = LLAMA3_405B if args.workload == "llama3-405b" else LLAMA2_7B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))

    steps, warmup = args.steps, max(args.warmup, 3)
    torch.cuda.manual_seed(1234)  # (the sampler itself is keyed by the model seed and the position: same draws on every rank)
    # N > 1: the one sequence is decoded tensor-parallel over the N GPUs (column/row-parallel shards, per-GPU
    # Hadamard transforms; the partial results of o_proj / down_proj are summed through peer-mapped memory)
    model = QtipLlama(shape, max_positions=args.prompt + 2 * (warmup + steps) + 16, device=dev, seed=3000,
                      tp_rank=rank, tp_size=world, group=dist.group.WORLD if world > 1 else None, fuse_qkv=args.fuse_qkv)
    if args.batch > 1:
        return run_gpu_batch(args, model, torch, dist, world, rank, dev)
    model.capture()
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, shape.vocab, (args.prompt,), generator=g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def prefill():
        model.reset()
        model.feed(prompt)
        model.generate(warmup)

    h_tok = torch.zeros(1, dtype=torch.int64).pin_memory()
    h_out = torch.zeros(1, dtype=torch.int64).pin_memory()
    with ClockSampler(local) as clocks:       # sampled over both timed regions and their warm-ups (>= 1 s)
        # ---- device-timed decode: K graph replays, tokens stay on the device --------------------------------
        prefill()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.generate(steps)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)

        # ---- end to end: every step the token goes host -> device (pinned) and the sampled token comes back ----
        prefill()
        h_tok.copy_(model.token.cpu())
        barrier()
        model._reserve(steps)
        t0 = time.perf_counter()
        for _ in range(steps):
            model.token.copy_(h_tok, non_blocking=True)
            model.graph.replay()
            h_out.copy_(model.token, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            h_tok[0] = h_out[0]
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        if clocks.proc is not None and len(clocks.rows) < 12:
            time.sleep(1.0 - min(1.0, 0.05 * len(clocks.rows)))     # short runs: let the sampler cover a full second
    model.check_status()

    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()

    if model.peers is not None and int(model.peers.status) != 0:
        raise RuntimeError("a wait for a peer GPU's values ran out during the run: the numbers are invalid")
    out = None
    if rank == 0:
        us, byts, launches = measure_matvec_roofline(model, torch)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = byts / us / 1e3  # GB/s
        seven_b = args.workload == "llama2-7b"
        shapes = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)] if args.fuse_qkv else llama7b_linears()
        traffic = [NCU_TRAFFIC_BYTES.get(s) for s in shapes]
        traffic = None if world > 1 or not seven_b or any(t is None for t in traffic) else sum(traffic) / len(traffic)
        extra = {}
        if world == 1 and seven_b:
            layer_us, h2d, d2h = measure_layer_e2e(torch)
            dec_gbs, dec_us = measure_decoder_gbs(torch)
            extra = {"e2e_layer": {"what": "QuantizedLinear.forward 4096x4096 K=2 with pinned host input and output",
                                   "us_per_call": layer_us, "h2d_bytes_per_call": h2d, "d2h_bytes_per_call": d2h},
                     "decode_hyb": {"shape": "4096x11008 K=2", "gbs": dec_gbs, "us": dec_us,
                                    "bytes": "K*m*n/8 read + 2*m*n written"}}
        out = {
            "metric": metric_name(args.workload),
            "value": steps / (ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": steps / (ms / 1e3) / PUBLISHED_TOK_S if seven_b else None,
            "dtype": "f16", "data": "synthetic",
            "config": workload_config(args.workload, args.prompt, world, args.fuse_qkv),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "kernel": "matvec_hyb_kernel<K=2, staged x, 32 warps> (the instantiation every "
                         "launch of the decode graph uses), timed on this model's own weight sets, one launch per linear",
                         "us_per_launch": us, "algorithmic_bytes_per_launch": byts,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650 GB/s"},
            "cpu_baseline": cpu_baseline_subprocess(args) if world == 1 else None,
            "e2e": {"value": steps / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 8,
                    "d2h_bytes_per_step": 8},
            "gpu_launches": model.n_launches_per_step * steps,
            "clocks": clocks.summary(),
        }
        out.update(extra)
        if world == 1:
            ceil = measure_issue_ceiling(torch, 2, float(out["clocks"].get("sm_mhz") or 1965.0))
            if ceil is not None:
                ceil["frac_of_hbm_peak"] = ceil["gbs"] / peak
                ceil["achieved_over_ceiling"] = achieved / ceil["gbs"]
                out["roofline"]["issue_ceiling"] = ceil
    if out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        model.release_graph()  # graphs that captured NCCL kernels must go before the communicator
        torch.cuda.synchronize()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=PROMPT_TOKENS, help="prompt length (128 in the benchmark configuration)")
    ap.add_argument("--workload", default="llama2-7b", choices=["llama2-7b", "llama3-405b"],
                    help="llama3-405b: the 126-layer shape of the tensor-parallel configuration (256-token prompt)")
    ap.add_argument("--impl", default="qtip_b200", choices=["qtip_b200", "reference"])
    ap.add_argument("--batch", type=int, default=1,
                    help="sequences decoded in lockstep (<= 8; the batch rides in the matvec launches); value counts all of them")
    ap.add_argument("--separate-qkv", action="store_true",
                    help="keep q, k, v and gate, up as separate matrices (three / two problems in one launch).  The default on "
                         "one GPU at batch 1 is q||k||v and gate||up as ONE matrix each (12288x4096, 22016x4096 at the 7B shape), "
                         "the layout upstream's published 188 tok/s was measured with; tensor-parallel and batched runs "
                         "always use separate matrices")
    args = ap.parse_args()
    args.fuse_qkv = use_fused_matrices(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
