"""Batch-1 decode loop of a Llama-architecture model whose linears are all QTIP layers.

This is the measurement harness for end-to-end decode speed: a random-init model of a given shape
(`LlamaShape`), a static KV cache, and one CUDA graph per decode step, replayed once per token
(upstream: eval/interactive_gen.py:42-85 with model/llama.py; the graph capture follows the pattern
of lib/utils/graph_wrapper.py:16-47 instead of torch.compile).  Inside the graph a decoder layer of the
Llama-2-7B shape is 6 launches of this library's kernels:
    q,k,v in one launch      (deferred output side of the previous down_proj, residual add, RMSNorm, input side)
    attention                (output side of q/k/v, rotary embedding, KV append, single-query attention)
    o_proj                   (input side fused; its output side is deferred into the next launch)
    gate,up in one launch    (deferred output side of o_proj, residual add, RMSNorm, input side)
    MLP middle               (output side of gate/up, SwiGLU product, input side of down_proj: 11008 = 172*64)
    down_proj                (its output side is deferred into the next layer's q,k,v launch)
plus three per token (embedding lookup, final norm + fp16 lm_head, sampler).  With tensor parallelism the partial
results of o_proj / down_proj are summed inside the consuming launch through peer-mapped memory (qtip_b200/tp.py).
Shapes the fused kernels do not cover (widths that are not 4096 / 8192, head counts that are not powers of two,
factor widths with short rows) fall back to separate transform / rotary / attention launches.
"""
import math
import os
import sys
from dataclasses import dataclass

import torch

from . import ops
from . import tp as tp_mod


@dataclass
class LlamaShape:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    mlp: int = 11008
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    K: int = 2  # bits per weight of every linear


LLAMA2_7B = LlamaShape()
LLAMA3_405B = LlamaShape(n_layers=126, hidden=16384, n_heads=128, n_kv_heads=8, head_dim=128, mlp=53248, vocab=128256,
                         rms_eps=1e-5, rope_theta=500000.0, K=2)


class _Linear:
    """Buffers of one (shard of a) QTIP linear - the state of QuantizedLinear upstream
    (lib/linear/quantized_linear.py:41-67).  m, n are the LOCAL sizes; `split` says which side is sharded
    ("col": rows of the full matrix, "row": columns, None: not sharded).  Codes and LUT come from the local
    generator, the sign vectors from the shared one (all ranks draw the full vectors and keep their slice)."""

    def __init__(self, m, n, K, g_local, g_shared, device, split=None, rank=0, tp=1, shard_full=False):
        self.m, self.n, self.K = m, n, K
        n_full = n * tp if split == "row" else n
        m_full = m * tp if split == "col" else m
        if shard_full:
            # the FULL matrix from the shared generator (same on every rank, and the same as a tp = 1 model draws),
            # then this rank's shard of it: the ranks together hold exactly one unsharded model
            full = torch.randint(0, 65536, (m_full * n_full // 256, 16 * K), generator=g_shared, device=device,
                                 dtype=torch.int32).to(torch.int16)
            if split == "col":
                full = tp_mod.shard_column_parallel(full, None, torch.zeros(m_full), m_full, n_full, K, rank, tp)[0]
            elif split == "row":
                full = tp_mod.shard_row_parallel(full, torch.zeros(n_full), None, m_full, n_full, K, rank, tp)[0]
            self.codes = full.contiguous()
        else:
            self.codes = torch.randint(0, 65536, (m * n // 256, 16 * K), generator=g_local, device=device,
                                       dtype=torch.int32).to(torch.int16)
        self.tlut = torch.randn(512, 2, generator=g_shared, device=device).half()
        SU = (torch.randn(n_full, generator=g_shared, device=device).sign() + 1e-5).sign().half()
        # SV carries the weight scale; keep the layer's output variance about that of its input
        SV = (torch.randn(m_full, generator=g_shared, device=device).sign() + 1e-5).sign().float() / math.sqrt(n_full)
        self.SU = SU[rank * n:(rank + 1) * n].contiguous() if split == "row" else SU
        self.SV = SV[rank * m:(rank + 1) * m].contiguous() if split == "col" else SV
        self.SV32 = (self.SV * 32).contiguous()


class _LinearView:
    """Sign / scale slices of one chunk (q, k, v, gate or up) of a fused matrix."""


class QtipLlama:

    def __init__(self, shape=LLAMA2_7B, max_positions=512, device="cuda:0", seed=3000, tp_rank=0, tp_size=1,
                 group=None, full_model_shards=False, fuse_qkv=False):
        """tp_size > 1: this process holds rank tp_rank's shards (qtip_b200.tp) and `group` is the
        torch.distributed group of the tp_size ranks (one all-reduce after o_proj and after down_proj).
        full_model_shards: every rank draws the full matrices (from the shared generator) and keeps its shard, so
        that the ranks together hold the one model a tp_size = 1 instance with the same seed holds; the default
        draws each rank's shard directly (same distribution, much faster for large shapes).
        fuse_qkv: q||k||v and gate||up are ONE QTIP matrix each (out_features H + 2*KV and 2*MLP: 12288 x 4096 and
        22016 x 4096 at the 7B shape, the layers upstream's published decode speed was measured with, README.md:31,
        48-51): one packed matrix, one LUT, one SU, and the output-side transform per q / k / v (gate / up) chunk,
        i.e. upstream's rcp = 2 layout with 3 (2) chunks (lib/codebook/bitshift.py:465-469).  Single GPU only."""
        self.shape, self.device, self.max_positions = shape, torch.device(device), max_positions
        self.tp, self.rank, self.group = tp_size, tp_rank, group
        s, dev, tp = shape, self.device, tp_size
        g = torch.Generator(device=dev).manual_seed(seed)                              # shared across ranks
        gl = torch.Generator(device=dev).manual_seed(seed + 7919 * (tp_rank + 1))      # this rank's shards
        assert s.n_heads % tp == 0 and s.n_kv_heads % tp == 0 and s.mlp % tp == 0
        H, KV, MLP = s.n_heads * s.head_dim // tp, s.n_kv_heads * s.head_dim // tp, s.mlp // tp   # LOCAL widths
        self.H, self.KV, self.MLP = H, KV, MLP
        self.n_heads, self.n_kv_heads = s.n_heads // tp, s.n_kv_heads // tp
        assert s.n_heads * s.head_dim == s.hidden
        for d in (s.hidden, H, KV, MLP):
            assert d % 32 == 0, f"width {d} is not a multiple of 32"
        assert s.head_dim == 128, "the decode attention kernel is built for head_dim 128"
        col = dict(split="col" if tp > 1 else None, rank=tp_rank, tp=tp, shard_full=full_model_shards)
        row = dict(split="row" if tp > 1 else None, rank=tp_rank, tp=tp, shard_full=full_model_shards)
        self.fuse_qkv = bool(fuse_qkv)
        assert not (self.fuse_qkv and tp > 1), "fused q||k||v / gate||up matrices are built for a single GPU"
        self.linear_names = ("qkv", "o", "gu", "down") if self.fuse_qkv else ("q", "k", "v", "o", "gate", "up", "down")
        self.layers = []
        for _ in range(s.n_layers):
            if self.fuse_qkv:
                L = dict(qkv=_Linear(H + 2 * KV, s.hidden, s.K, gl, g, dev), o=_Linear(s.hidden, H, s.K, gl, g, dev),
                         gu=_Linear(2 * MLP, s.hidden, s.K, gl, g, dev), down=_Linear(s.hidden, MLP, s.K, gl, g, dev))
                # the chunks of the fused matrices as the rest of the step sees them: sign / scale slices only
                for name, lin, lo, hi in (("q", L["qkv"], 0, H), ("k", L["qkv"], H, H + KV), ("v", L["qkv"], H + KV, H + 2 * KV),
                                          ("gate", L["gu"], 0, MLP), ("up", L["gu"], MLP, 2 * MLP)):
                    view = _LinearView()
                    view.SU, view.SV, view.SV32 = lin.SU, lin.SV[lo:hi], lin.SV32[lo:hi]
                    L[name] = view
            else:
                L = dict(q=_Linear(H, s.hidden, s.K, gl, g, dev, **col), k=_Linear(KV, s.hidden, s.K, gl, g, dev, **col),
                         v=_Linear(KV, s.hidden, s.K, gl, g, dev, **col), o=_Linear(s.hidden, H, s.K, gl, g, dev, **row),
                         gate=_Linear(MLP, s.hidden, s.K, gl, g, dev, **col), up=_Linear(MLP, s.hidden, s.K, gl, g, dev, **col),
                         down=_Linear(s.hidden, MLP, s.K, gl, g, dev, **row))
            L["ln1"] = (1 + 0.02 * torch.randn(s.hidden, generator=g, device=dev)).half()
            L["ln2"] = (1 + 0.02 * torch.randn(s.hidden, generator=g, device=dev)).half()
            # sign vectors of launches that share one input, concatenated
            if not self.fuse_qkv:
                L["SU_qkv"] = torch.cat([L["q"].SU, L["k"].SU, L["v"].SU]).contiguous()
                L["SU_gu"] = torch.cat([L["gate"].SU, L["up"].SU]).contiguous()
            L["SV_gu"] = torch.cat([L["gate"].SV32, L["up"].SV32]).contiguous()
            self.layers.append(L)
        self.embed = (0.02 * torch.randn(s.vocab, s.hidden, generator=g, device=dev)).half()
        self.lm_head = (0.02 * torch.randn(s.vocab, s.hidden, generator=g, device=dev)).half()
        self.ln_f = (1 + 0.02 * torch.randn(s.hidden, generator=g, device=dev)).half()
        self.cache_k = torch.zeros(s.n_layers, max_positions, KV, dtype=torch.float16, device=dev)
        self.cache_v = torch.zeros_like(self.cache_k)
        # Hadamard factors: full hidden width, and the local chunks of the split sides
        self.kf_h = ops.had_factor(s.hidden)
        self.kf_hl = ops.had_factor(H)
        self.kf_m = ops.had_factor(MLP)
        self.kf_kv = ops.had_factor(KV)
        self.bits = {}
        for k in {self.kf_h, self.kf_hl, self.kf_m, self.kf_kv}:
            self.bits[k] = None if k == 1 else ops.pack_hadk(ops.get_hadK(k * 2)[0].to(dev))
        # activations (static, so the step can be captured)
        f16 = dict(dtype=torch.float16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.res = [torch.zeros(s.hidden, **f16), torch.zeros(s.hidden, **f16)]  # residual stream, ping-pong
        self.delta = torch.zeros(s.hidden, **f16)   # output of the last linear, not yet added to the stream
        self.xh_qkv = torch.zeros(3, s.hidden, **f16)   # RHT-in outputs (fp16 activations of the matvecs)
        self.xh_gu = torch.zeros(2, s.hidden, **f16)
        self.xh_o = torch.zeros(H, **f16)
        self.xh_d = torch.zeros(MLP, **f16)
        self.y_qkv = torch.zeros(H + 2 * KV, **f32)
        self.qkv = torch.zeros(H + 2 * KV, **f16)
        self.attn = torch.zeros(H, **f16)
        self.y_h = torch.zeros(s.hidden, **f32)
        self.y_gu = torch.zeros(2 * MLP, **f32)
        self.gu = torch.zeros(2 * MLP, **f16)
        self.logits = torch.zeros(1, s.vocab, **f32)
        self.sample_seed = seed
        self.out_tokens = torch.zeros(max_positions + 1, dtype=torch.int64, device=dev)
        # set by a kernel that found the position / token outside its buffer (the kernel then skipped its work)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.steps_done = 0   # host-side count of positions consumed since reset()
        need = max(ops._lib.load().qtip_matvec_workspace_bytes(m, n, 1)
                   for (m, n) in ((H, s.hidden), (MLP, s.hidden), (s.hidden, MLP), (s.hidden, H), (KV, s.hidden),
                                  (H + 2 * KV, s.hidden), (2 * MLP, s.hidden)))
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        self.workspaces = [self.workspace] + [torch.zeros(need, dtype=torch.uint8, device=dev) for _ in range(2)]
        pow2 = lambda d: d & (d - 1) == 0  # noqa: E731
        # which transforms can ride inside the matvec launch (powers of two only; see qtip_linear_fused)
        fin = lambda d: pow2(d) and d <= 8192   # the in-kernel input transform needs its fp32 scratch in shared memory  # noqa: E731
        self.fuse_in_h, self.fuse_in_hl, self.fuse_in_m = fin(s.hidden), fin(H), fin(MLP)
        fout = lambda d: pow2(d) and d <= 16384  # noqa: E731
        self.fuse_out_h, self.fuse_out_hl, self.fuse_out_kv, self.fuse_out_m = fout(s.hidden), fout(H), fout(KV), fout(MLP)
        # deferred output sides: the Hadamard transform + sign of o_proj / down_proj runs in the prologue of the
        # NEXT launch (which needs the register transform: 4096 or 8192 wide), that of q/k/v in the rotary kernel
        self.defer_h = self.fuse_in_h and s.hidden in (4096, 8192)
        # tp > 1: the partial results of o_proj / down_proj stay where they are; the next launch on every GPU waits
        # for all GPUs' flags and adds the partial vectors through peer-mapped memory (no all-reduce launch)
        self.peers = None
        if tp > 1 and self.defer_h and os.environ.get("QTIP_TP_PEER", "1") != "0":
            # every rank must take the same path: agree on whether the peer-mapped buffers could be set up
            import torch.distributed as dist
            try:
                peers = tp_mod.PeerBuffers(s.hidden, tp_rank, tp_size, group, dev)
            except Exception as e:   # no symmetric memory on this system: all-reduce launches instead
                print(f"qtip_b200: peer-mapped buffers unavailable ({e!r}); using NCCL all-reduce", file=sys.stderr)
                peers = None
            ok = torch.tensor([1 if peers is not None else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            self.peers = peers if int(ok) == 1 else None
        self.defer_qkv = self.fuse_in_h and all(w in (1024, 2048, 4096, 8192, 16384) for w in (H, KV))
        # ... or, with power-of-two head counts, inside the attention kernel itself (no rotary launch at all)
        self.attn_fused = self.fuse_in_h and s.head_dim == 128 and pow2(self.n_heads) and pow2(self.n_kv_heads)
        # gate/up output side + SwiGLU + down input side as one cluster launch (widths with a Hadamard factor)
        self.mid_fused = (not self.fuse_out_m) and (not self.fuse_in_m) and ops.mlp_mid_supported(MLP)
        self.mid_table = ops.mlp_mid_table(MLP, dev, self.bits[self.kf_m]) if self.mid_fused else None
        if self.fuse_qkv:
            assert self.fuse_in_h and (self.attn_fused or self.defer_qkv), \
                "fused q||k||v / gate||up matrices need the in-kernel input transform and a deferred q/k/v output side"
        if self.peers is not None:
            import torch.distributed as dist
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)           # start the flag protocol with every rank ready
        self.graph = None
        self.n_launches_per_step = None   # counted while the step runs (library launches only)

    # -- one linear: the three launches ------------------------------------------------------------
    def _matvec(self, lin, xh, y):
        ops.decompress_matvec(lin.codes, xh, lin.tlut, lin.K, lin.m, lin.n, out=y.view(1, lin.m), workspace=self.workspace)

    def _all_reduce(self, t):
        if self.tp > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)

    def _linears(self, lins, xs_or_raw, ys, n, m, *, fused_in=None, outs=None, sign_outs=None, out_scale=1.0, extra=None):
        """One launch for the same-shape linears `lins`.  fused_in: dict(in_raw, residual, residual_out, norm_weight,
        gate, sign_ins, in_scale) or None (then xs_or_raw holds the transformed fp16 inputs).  outs: fused output side."""
        descs = []
        for i, lin in enumerate(lins):
            d = dict(y=ys[i], codes=lin.codes, tlut=lin.tlut, workspace=self.workspaces[i])
            if fused_in is None:
                d["x"] = xs_or_raw[i]
            else:
                d.update(in_raw=fused_in.get("in_raw"), in_y=fused_in.get("in_y"), in_y_sign=fused_in.get("in_y_sign"),
                         in_y_scale=fused_in.get("in_y_scale", 1.0),
                         residual=fused_in.get("residual"), norm_weight=fused_in.get("norm_weight"),
                         gate=fused_in.get("gate"), sign_in=fused_in["sign_ins"][i], in_scale=fused_in["in_scale"],
                         eps=self.shape.rms_eps)
                if i == 0:
                    d["residual_out"] = fused_in.get("residual_out")
            if outs is not None:
                d.update(out=outs[i], sign_out=sign_outs[i], out_scale=out_scale)
            if fused_in is not None and "peer" in fused_in:
                d.update(fused_in["peer"])
            if extra:
                d.update(extra)
            descs.append(d)
        ops.linear_fused(descs, lins[0].K, m, n, 1)

    def step(self):
        """One decode step on the static buffers: token -> next_token, pos += 1.  Capturable."""
        s = self.shape
        H, KV, MLP = self.H, self.KV, self.MLP
        res_a, res_b = self.res
        ops.embed_token(res_a, self.delta, self.embed, self.token, status=self.status)
        inv_h, inv_hl, inv_m, inv_kv = (1 / math.sqrt(d) for d in (s.hidden, H, MLP, KV))
        bits = self.bits
        tp1 = self.tp == 1
        y_q, y_k, y_v = self.y_qkv[:H], self.y_qkv[H:H + KV], self.y_qkv[H + KV:]
        q, k, v = self.qkv[:H], self.qkv[H:H + KV], self.qkv[H + KV:]
        delta_src = dict(in_raw=self.delta)      # where the pending residual update comes from
        last = len(self.layers) - 1
        for li, L in enumerate(self.layers):
            # ---- attention block: res_b = res_a + delta ; h = RMSNorm(res_b) ; q,k,v (column-parallel)
            if self.fuse_in_h and (self.attn_fused or self.defer_qkv or (self.fuse_out_hl and self.fuse_out_kv)):
                dq = self.defer_qkv or self.attn_fused
                fin = dict(delta_src, residual=res_a, residual_out=res_b, norm_weight=L["ln1"], in_scale=inv_h / 32)
                if self.fuse_qkv:
                    assert dq, "the fused q||k||v matrix needs its output side inside the attention / rotary launch"
                    self._linears([L["qkv"]], None, [self.y_qkv], s.hidden, H + 2 * KV,
                                  fused_in=dict(fin, sign_ins=[L["qkv"].SU]))
                elif H == KV:
                    self._linears([L["q"], L["k"], L["v"]], None, [y_q, y_k, y_v], s.hidden, H,
                                  fused_in=dict(fin, sign_ins=[L["q"].SU, L["k"].SU, L["v"].SU]), outs=None if dq else [q, k, v],
                                  sign_outs=[L["q"].SV32, L["k"].SV32, L["v"].SV32], out_scale=inv_hl)
                else:
                    self._linears([L["q"]], None, [y_q], s.hidden, H, fused_in=dict(fin, sign_ins=[L["q"].SU]),
                                  outs=None if dq else [q], sign_outs=[L["q"].SV32], out_scale=inv_hl)
                    fin2 = dict(in_raw=res_b, norm_weight=L["ln1"], in_scale=inv_h / 32, sign_ins=[L["k"].SU, L["v"].SU])
                    self._linears([L["k"], L["v"]], None, [y_k, y_v], s.hidden, KV, fused_in=fin2, outs=None if dq else [k, v],
                                  sign_outs=[L["k"].SV32, L["v"].SV32], out_scale=inv_kv)
            else:
                dq = False
                assert "in_raw" in delta_src
                xh = self.xh_qkv
                ops.rht_fused(self.delta, 3, s.hidden, xh, in_row_stride=0, residual=res_a, residual_out=res_b,
                              norm_weight=L["ln1"], eps=s.rms_eps, sign_in=L["SU_qkv"], hadk_bits=bits[self.kf_h],
                              kfac=self.kf_h, transpose=True, scale=inv_h / 32)
                self._matvec(L["q"], xh[0], y_q)
                self._matvec(L["k"], xh[1], y_k)
                self._matvec(L["v"], xh[2], y_v)
                ops.rht_fused(y_q, 1, H, q, sign_out=L["q"].SV32, hadk_bits=bits[self.kf_hl], kfac=self.kf_hl, scale=inv_hl)
                sv = L.get("SV_kv")
                if sv is None:
                    sv = L["SV_kv"] = torch.cat([L["k"].SV32, L["v"].SV32]).contiguous()
                ops.rht_fused(self.y_qkv[H:], 2, KV, self.qkv[H:], sign_out=sv, hadk_bits=bits[self.kf_kv],
                              kfac=self.kf_kv, scale=inv_kv)
            if dq and self.attn_fused:
                ops.attn_decode_fused(self.attn, y_q, y_k, y_v, L["q"].SV32, L["k"].SV32, L["v"].SV32, inv_hl, inv_kv,
                                      self.cache_k[li], self.cache_v[li], self.pos, self.n_heads, self.n_kv_heads,
                                      s.head_dim, s.rope_theta, status=self.status)
            elif dq:
                ops.rope_kv_append_fused(q, y_q, y_k, y_v, L["q"].SV32, L["k"].SV32, L["v"].SV32, inv_hl, inv_kv,
                                         self.cache_k[li], self.cache_v[li], self.pos, self.n_heads, self.n_kv_heads,
                                         s.head_dim, s.rope_theta, status=self.status)
            else:
                ops.rope_kv_append(q, k, v, self.cache_k[li], self.cache_v[li], self.pos, self.n_heads, self.n_kv_heads,
                                   s.head_dim, s.rope_theta, status=self.status)
            if not (dq and self.attn_fused):
                ops.attn_decode(self.attn, q, self.cache_k[li], self.cache_v[li], self.pos, self.n_heads, self.n_kv_heads,
                                s.head_dim, status=self.status)
            # ---- o_proj (row-parallel: local chunk in, full-length partial out, all-reduce, transform)
            defer = self.defer_h
            use_peers = defer and self.peers is not None
            fuse_out = tp1 and self.fuse_out_h and not defer
            y_o = self.y_h
            sig = self.peers.signal(0) if use_peers else None
            if self.fuse_in_hl:
                self._linears([L["o"]], None, [y_o], H, s.hidden,
                              fused_in=dict(in_raw=self.attn, sign_ins=[L["o"].SU], in_scale=inv_hl / 32),
                              outs=[self.delta] if fuse_out else None, sign_outs=[L["o"].SV32], out_scale=inv_h, extra=sig)
            else:
                ops.rht_fused(self.attn, 1, H, self.xh_o, sign_in=L["o"].SU, hadk_bits=bits[self.kf_hl], kfac=self.kf_hl,
                              transpose=True, scale=inv_hl / 32)
                self._linears([L["o"]], [self.xh_o], [y_o], H, s.hidden, outs=[self.delta] if fuse_out else None,
                              sign_outs=[L["o"].SV32], out_scale=inv_h, extra=sig)
            if use_peers:
                delta_src = dict(peer=self.peers.consume(0), in_y_sign=L["o"].SV32, in_y_scale=inv_h)
            elif defer:
                self._all_reduce(self.y_h)
                delta_src = dict(in_y=self.y_h, in_y_sign=L["o"].SV32, in_y_scale=inv_h)
            else:
                delta_src = dict(in_raw=self.delta)
                if not fuse_out:
                    self._all_reduce(self.y_h)
                    ops.rht_fused(self.y_h, 1, s.hidden, self.delta, sign_out=L["o"].SV32, hadk_bits=bits[self.kf_h],
                                  kfac=self.kf_h, scale=inv_h)
            # ---- MLP block: res_a = res_b + delta ; h = RMSNorm(res_a) ; gate, up (column-parallel)
            y_g, y_u = self.y_gu[:MLP], self.y_gu[MLP:]
            if self.fuse_in_h:
                fin = dict(delta_src, residual=res_b, residual_out=res_a, norm_weight=L["ln2"], in_scale=inv_h / 32,
                           sign_ins=[L["gate"].SU, L["up"].SU])
                fo = self.fuse_out_m and not self.fuse_qkv
                if self.fuse_qkv:
                    self._linears([L["gu"]], None, [self.y_gu], s.hidden, 2 * MLP, fused_in=dict(fin, sign_ins=[L["gu"].SU]))
                else:
                    self._linears([L["gate"], L["up"]], None, [y_g, y_u], s.hidden, MLP, fused_in=fin,
                                  outs=[self.gu[:MLP], self.gu[MLP:]] if fo else None,
                                  sign_outs=[L["gate"].SV32, L["up"].SV32], out_scale=inv_m)
            else:
                fo = False
                xg = self.xh_gu
                ops.rht_fused(self.delta, 2, s.hidden, xg, in_row_stride=0, residual=res_b, residual_out=res_a,
                              norm_weight=L["ln2"], eps=s.rms_eps, sign_in=L["SU_gu"], hadk_bits=bits[self.kf_h],
                              kfac=self.kf_h, transpose=True, scale=inv_h / 32)
                self._matvec(L["gate"], xg[0], y_g)
                self._matvec(L["up"], xg[1], y_u)
            mid = self.mid_fused and not fo
            if mid:
                ops.mlp_mid(self.xh_d, y_g, y_u, L["gate"].SV32, L["up"].SV32, L["down"].SU, MLP, inv_m, inv_m / 32,
                            table=self.mid_table)
            elif not fo:
                ops.rht_fused(self.y_gu, 2, MLP, self.gu, sign_out=L["SV_gu"], hadk_bits=bits[self.kf_m],
                              kfac=self.kf_m, scale=inv_m)
            # ---- down_proj (row-parallel), input silu(gate) * up
            defer = self.defer_h and li != last       # the last layer's result is read by the final norm
            use_peers = defer and self.peers is not None
            fuse_out = tp1 and self.fuse_out_h and not defer
            y_d = self.y_h
            sig = self.peers.signal(1) if use_peers else None
            if self.fuse_in_m:
                self._linears([L["down"]], None, [y_d], MLP, s.hidden,
                              fused_in=dict(in_raw=self.gu[MLP:], gate=self.gu[:MLP], sign_ins=[L["down"].SU], in_scale=inv_m / 32),
                              outs=[self.delta] if fuse_out else None, sign_outs=[L["down"].SV32], out_scale=inv_h, extra=sig)
            else:
                xd = self.xh_d
                if not mid:
                    ops.rht_fused(self.gu[MLP:], 1, MLP, xd, gate=self.gu[:MLP], sign_in=L["down"].SU,
                                  hadk_bits=bits[self.kf_m], kfac=self.kf_m, transpose=True, scale=inv_m / 32)
                self._linears([L["down"]], [xd], [y_d], MLP, s.hidden, outs=[self.delta] if fuse_out else None,
                              sign_outs=[L["down"].SV32], out_scale=inv_h, extra=sig)
            if use_peers:
                delta_src = dict(peer=self.peers.consume(1), in_y_sign=L["down"].SV32, in_y_scale=inv_h)
            elif defer:
                self._all_reduce(self.y_h)
                delta_src = dict(in_y=self.y_h, in_y_sign=L["down"].SV32, in_y_scale=inv_h)
            else:
                delta_src = dict(in_raw=self.delta)
                if not fuse_out:
                    self._all_reduce(self.y_h)
                    ops.rht_fused(self.y_h, 1, s.hidden, self.delta, sign_out=L["down"].SV32, hadk_bits=bits[self.kf_h],
                                  kfac=self.kf_h, scale=inv_h)
        # ---- final norm + lm_head (fp16 weights, HBM-bound GEMV), sampler: token, out_tokens[pos + 1], pos += 1
        ops.lm_head(self.logits, res_a, self.delta, self.ln_f, self.lm_head, s.rms_eps)
        ops.sample_top_k(self.token, self.out_tokens, self.pos, self.logits, temperature=0.6, top_k=5, seed=self.sample_seed,
                         status=self.status)

    # -- batched decode: B sequences in lockstep ------------------------------------------------------
    def enable_batch(self, B):
        """Buffers for decoding B (<= 8) independent sequences per step (step_batch).  The batch rides in the matvec
        launches (the packed matrices are streamed once for all B rows); the transforms run as row-batched launches of
        the transform kernel, rotary embedding / attention / sampling per sequence.  Works for every shape and for
        tensor parallelism (NCCL all-reduce after o_proj and down_proj)."""
        assert 1 <= B <= ops.MAX_MATVEC_BATCH and not self.fuse_qkv
        s, dev, H, KV, MLP = self.shape, self.device, self.H, self.KV, self.MLP
        f16 = dict(dtype=torch.float16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.B = B
        self.b_token = torch.zeros(B, dtype=torch.int64, device=dev)
        self.b_pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.b_res = [torch.zeros(B, s.hidden, **f16), torch.zeros(B, s.hidden, **f16)]
        self.b_delta = torch.zeros(B, s.hidden, **f16)
        self.b_xh = torch.zeros(B, max(s.hidden, MLP, H), **f16)
        self.b_y = torch.zeros(B, max(s.hidden, MLP, H), **f32)
        self.b_q, self.b_k, self.b_v = torch.zeros(B, H, **f16), torch.zeros(B, KV, **f16), torch.zeros(B, KV, **f16)
        self.b_attn = torch.zeros(B, H, **f16)
        self.b_g, self.b_u = torch.zeros(B, MLP, **f16), torch.zeros(B, MLP, **f16)
        self.b_cache_k = torch.zeros(B, s.n_layers, self.max_positions, KV, **f16)
        self.b_cache_v = torch.zeros_like(self.b_cache_k)
        self.b_logits = torch.zeros(B, s.vocab, **f32)
        self.b_out_tokens = torch.zeros(B, self.max_positions + 1, dtype=torch.int64, device=dev)
        need = max(ops._lib.load().qtip_matvec_workspace_bytes(m, n, B)
                   for (m, n) in ((H, s.hidden), (MLP, s.hidden), (s.hidden, MLP), (s.hidden, H), (KV, s.hidden)))
        self.b_workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        self.b_graph = None

    def _b_linear(self, lin, src, *, residual=None, residual_out=None, norm=None, gate=None, kf_in, kf_out,
                  out, all_reduce=False):
        """One QTIP linear on B rows: transform in (optionally residual add / RMSNorm / SwiGLU), matvec, transform out."""
        B, n, m = self.B, lin.n, lin.m
        xh, y = self.b_xh.view(-1)[:B * n].view(B, n), self.b_y.view(-1)[:B * m].view(B, m)
        ops.rht_fused(src, B, n, xh, residual=residual, residual_out=residual_out, norm_weight=norm, eps=self.shape.rms_eps,
                      gate=gate, sign_in=lin.SU, hadk_bits=self.bits[kf_in], kfac=kf_in, transpose=True,
                      scale=1 / math.sqrt(n) / 32)
        ops.decompress_matvec(lin.codes, xh, lin.tlut, lin.K, m, n, out=y, workspace=self.b_workspace)
        if all_reduce:
            self._all_reduce(y)
        ops.rht_fused(y, B, m, out, sign_out=lin.SV32, hadk_bits=self.bits[kf_out], kfac=kf_out, scale=1 / math.sqrt(m))

    def step_batch(self):
        """One decode step of B sequences on the static batch buffers: b_token -> next tokens, b_pos += 1."""
        s, B = self.shape, self.B
        ra, rb = self.b_res
        torch.index_select(self.embed, 0, self.b_token, out=ra)
        self.b_delta.zero_()
        for li, L in enumerate(self.layers):
            # res_b = res_a + delta ; h = RMSNorm(res_b) ; q, k, v
            self._b_linear(L["q"], self.b_delta, residual=ra, residual_out=rb, norm=L["ln1"], kf_in=self.kf_h,
                           kf_out=self.kf_hl, out=self.b_q)
            self._b_linear(L["k"], rb, norm=L["ln1"], kf_in=self.kf_h, kf_out=self.kf_kv, out=self.b_k)
            self._b_linear(L["v"], rb, norm=L["ln1"], kf_in=self.kf_h, kf_out=self.kf_kv, out=self.b_v)
            for b in range(B):
                ck, cv, pos = self.b_cache_k[b, li], self.b_cache_v[b, li], self.b_pos[b:b + 1]
                ops.rope_kv_append(self.b_q[b], self.b_k[b], self.b_v[b], ck, cv, pos, self.n_heads, self.n_kv_heads,
                                   s.head_dim, s.rope_theta, status=self.status)
                ops.attn_decode(self.b_attn[b], self.b_q[b], ck, cv, pos, self.n_heads, self.n_kv_heads, s.head_dim,
                                status=self.status)
            self._b_linear(L["o"], self.b_attn, kf_in=self.kf_hl, kf_out=self.kf_h, out=self.b_delta, all_reduce=True)
            # res_a = res_b + delta ; h = RMSNorm(res_a) ; gate, up ; down(silu(gate) * up)
            self._b_linear(L["gate"], self.b_delta, residual=rb, residual_out=ra, norm=L["ln2"], kf_in=self.kf_h,
                           kf_out=self.kf_m, out=self.b_g)
            self._b_linear(L["up"], ra, norm=L["ln2"], kf_in=self.kf_h, kf_out=self.kf_m, out=self.b_u)
            self._b_linear(L["down"], self.b_u, gate=self.b_g, kf_in=self.kf_m, kf_out=self.kf_h, out=self.b_delta,
                           all_reduce=True)
        # final norm + unquantized lm_head for the whole batch (fp16 GEMM: not part of the QTIP path), then the sampler
        x32 = (ra + self.b_delta).float()
        hn = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + s.rms_eps)).half() * self.ln_f
        self.b_logits.copy_(torch.matmul(hn, self.lm_head.T))
        for b in range(B):
            ops.sample_top_k(self.b_token[b:b + 1], self.b_out_tokens[b], self.b_pos[b:b + 1], self.b_logits[b:b + 1],
                             temperature=0.6, top_k=5, seed=self.sample_seed + b, status=self.status)

    def capture_batch(self):
        tok, pos = self.b_token.clone(), self.b_pos.clone()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.step_batch()
            self.b_token.copy_(tok); self.b_pos.copy_(pos)
            before = ops.launch_count
            self.step_batch()
            self.n_launches_per_batch_step = ops.launch_count - before
            self.b_token.copy_(tok); self.b_pos.copy_(pos)
            stream.synchronize()
            self.b_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.b_graph, stream=stream):
                self.step_batch()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.b_token.copy_(tok); self.b_pos.copy_(pos)
        torch.cuda.synchronize(self.device)

    def generate_batch(self, n_tokens):
        self._reserve(n_tokens)
        run = self.b_graph.replay if self.b_graph is not None else self.step_batch
        for _ in range(n_tokens):
            run()

    # -- driving ----------------------------------------------------------------------------------
    def capture(self):
        """Capture step() into a CUDA graph (two eager warm-up steps first; state is restored)."""
        tok, pos = self.token.clone(), self.pos.clone()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.step()
            self.token.copy_(tok); self.pos.copy_(pos)
            before = ops.launch_count
            self.step()
            self.n_launches_per_step = ops.launch_count - before
            self.token.copy_(tok); self.pos.copy_(pos)
            stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self.step()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.token.copy_(tok); self.pos.copy_(pos)
        torch.cuda.synchronize(self.device)

    def release_graph(self):
        """Destroy the captured graph.  With tensor parallelism this must happen before the process group is
        destroyed: NCCL does not tear a communicator down while a CUDA graph that captured its kernels is alive
        (destroy_process_group blocks forever otherwise)."""
        if self.graph is not None:
            torch.cuda.synchronize(self.device)
            self.graph.reset()
            self.graph = None
        if getattr(self, "b_graph", None) is not None:
            torch.cuda.synchronize(self.device)
            self.b_graph.reset()
            self.b_graph = None

    def reset(self):
        self.pos.zero_()
        self.cache_k.zero_(); self.cache_v.zero_()
        self.steps_done = 0

    def _reserve(self, n_steps):
        """Refuse on the host what the KV cache cannot hold (the kernels would skip the step and set `status`)."""
        if self.steps_done + n_steps > self.max_positions:
            raise RuntimeError(f"{self.steps_done} positions used, {n_steps} more requested: the KV cache holds "
                               f"{self.max_positions}")
        self.steps_done += n_steps

    def check_status(self):
        """Raise if a kernel reported an index outside its buffer (synchronises)."""
        st = int(self.status.item())
        if st:
            raise RuntimeError(f"decode-loop status {st}: 1 = position outside the KV cache, 2 = token outside the "
                               "embedding table, 4 = token log full")

    def feed(self, token_ids):
        """Run the given tokens through the model one position at a time (fills the KV cache); the
        sampled continuation of the last one is left in self.token."""
        ids = token_ids.tolist()
        self._reserve(len(ids))
        run = self.graph.replay if self.graph is not None else self.step
        for t in ids:
            if not 0 <= int(t) < self.shape.vocab:
                raise RuntimeError(f"token {t} outside the vocabulary of {self.shape.vocab}")
            self.token.fill_(int(t))
            run()

    def generate(self, n_tokens):
        self._reserve(n_tokens)
        run = self.graph.replay if self.graph is not None else self.step
        for _ in range(n_tokens):
            run()
