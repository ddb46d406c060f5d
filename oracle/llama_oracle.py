"""CPU decode step of a Llama-architecture model whose linears are QTIP layers, on the C restatement.

TEST INFRASTRUCTURE / CPU BASELINE ONLY (imported by bench.py's reference arm and CPU-baseline leg, never by
the product).  One `step` is what the upstream decode loop does per token (eval/interactive_gen.py:42-48 with
model/llama.py): embedding, per layer RMSNorm -> q/k/v (BitshiftLinear.forward, lib/codebook/bitshift.py:415-472)
-> rotary embedding -> attention over the KV cache -> o_proj -> residual -> RMSNorm -> gate/up -> SwiGLU -> down_proj
-> residual, final norm, lm_head, temperature / top-k sampling.  The linears run in qo_layer_forward (OpenMP, all
host threads); the rest is numpy in the precision of the fp16 torch modules.

Weights are seeded synthetic stand-ins (uniform 16-bit code words, N(0,1) LUT, +-1 sign vectors, N(0, 0.02)
embedding / lm_head).  To bound host memory and set-up time the decoder layers cycle through `weight_sets` distinct
sets of layer weights (default 4 = 200 MB of codes at the 7B shape, far beyond the CPU caches); the arithmetic per
step is that of the full depth.
"""
import math

import numpy as np

import c_oracle as C


def _f16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


class _Lin:
    def __init__(self, rng, m, n, K, hadk, chunks=1):
        """chunks > 1: a fused matrix (q||k||v, gate||up): one packed matrix and one table, the output-side transform
        per chunk of m/chunks rows - upstream's rcp = 2 layout (lib/codebook/bitshift.py:465-469)."""
        self.m, self.n, self.K, self.chunks = m, n, K, chunks
        self.codes = rng.integers(0, 65536, size=(m * n // 256, 16 * K), dtype=np.uint16)
        self.tlut = rng.standard_normal((512, 2)).astype(np.float16)
        self.SU = np.where(rng.standard_normal(n) >= 0, 1.0, -1.0).astype(np.float32)
        self.SV = (np.where(rng.standard_normal(m) >= 0, 1.0, -1.0) / math.sqrt(n)).astype(np.float32)
        self.hl, self.hr = hadk(n), hadk(m // chunks)

    def __call__(self, v):
        y = C.layer_forward(v, self.codes, self.m, self.n, self.K, self.tlut, self.SU, self.SV, self.hl, self.hr,
                            rcp=2 if self.chunks > 1 else 0, tp=self.chunks)
        return _f16(y.reshape(-1))


class OracleLlama:
    def __init__(self, hadk, n_layers=32, hidden=4096, n_heads=32, n_kv_heads=32, head_dim=128, mlp=11008, vocab=32000,
                 K=2, rms_eps=1e-5, rope_theta=10000.0, max_positions=512, weight_sets=4, seed=3000, fuse_qkv=False):
        """hadk(n) -> the Hadamard factor matrix of width n (fp32 numpy) or None for a power of two.
        fuse_qkv: q||k||v and gate||up as one packed matrix each (needs n_heads == n_kv_heads), upstream's fused layers."""
        rng = np.random.default_rng(seed)
        self.n_layers, self.hidden, self.n_heads, self.n_kv, self.hd = n_layers, hidden, n_heads, n_kv_heads, head_dim
        self.eps, self.theta, self.vocab = rms_eps, rope_theta, vocab
        H, KV = n_heads * head_dim, n_kv_heads * head_dim
        self.fuse_qkv = bool(fuse_qkv)
        assert not self.fuse_qkv or H == KV, "the fused q||k||v matrix is built for equal q / k / v widths"
        self.H, self.KV, self.MLP = H, KV, mlp
        self.sets = []
        for _ in range(max(1, min(weight_sets, n_layers))):
            if self.fuse_qkv:
                L = dict(qkv=_Lin(rng, H + 2 * KV, hidden, K, hadk, chunks=3), o=_Lin(rng, hidden, H, K, hadk),
                         gu=_Lin(rng, 2 * mlp, hidden, K, hadk, chunks=2), down=_Lin(rng, hidden, mlp, K, hadk))
            else:
                L = {name: _Lin(rng, m, n, K, hadk) for name, (m, n) in dict(q=(H, hidden), k=(KV, hidden), v=(KV, hidden),
                                                                              o=(hidden, H), gate=(mlp, hidden),
                                                                              up=(mlp, hidden), down=(hidden, mlp)).items()}
            L["ln1"] = _f16(1 + 0.02 * rng.standard_normal(hidden))
            L["ln2"] = _f16(1 + 0.02 * rng.standard_normal(hidden))
            self.sets.append(L)
        self.embed = _f16(0.02 * rng.standard_normal((vocab, hidden)))
        self.lm_head = _f16(0.02 * rng.standard_normal((vocab, hidden)))
        self.ln_f = _f16(1 + 0.02 * rng.standard_normal(hidden))
        self.cache_k = np.zeros((n_layers, max_positions, n_kv_heads, head_dim), dtype=np.float32)
        self.cache_v = np.zeros_like(self.cache_k)
        self.pos = 0
        self.rng = rng

    def fill_cache(self, n_positions):
        """Stand-in for a processed prompt: fp16 N(0,1) keys / values at positions 0..n_positions-1."""
        self.cache_k[:, :n_positions] = _f16(self.rng.standard_normal(self.cache_k[:, :n_positions].shape))
        self.cache_v[:, :n_positions] = _f16(self.rng.standard_normal(self.cache_v[:, :n_positions].shape))
        self.pos = n_positions

    def _norm(self, v, w):
        return _f16(w * _f16(v * (1.0 / np.sqrt(np.mean(v * v) + self.eps))))

    def step(self, token, temperature=0.6, top_k=5):
        hd, half, rep = self.hd, self.hd // 2, self.n_heads // self.n_kv
        inv = self.theta ** (-np.arange(half, dtype=np.float64) * 2 / hd)
        cs, sn = np.cos(self.pos * inv), np.sin(self.pos * inv)

        def rope(t):
            t = t.reshape(-1, hd).astype(np.float64)
            a, b = t[:, :half], t[:, half:]
            return _f16(np.concatenate([a * cs - b * sn, b * cs + a * sn], axis=1))

        x = self.embed[token].copy()
        ctx = self.pos + 1
        for li in range(self.n_layers):
            L = self.sets[li % len(self.sets)]
            h = self._norm(x, L["ln1"])
            if self.fuse_qkv:
                y = L["qkv"](h)
                q, k, v = rope(y[:self.H]), rope(y[self.H:self.H + self.KV]), y[self.H + self.KV:].reshape(-1, hd)
            else:
                q, k, v = rope(L["q"](h)), rope(L["k"](h)), L["v"](h).reshape(-1, hd)
            self.cache_k[li, self.pos], self.cache_v[li, self.pos] = k, v
            Kc = np.repeat(self.cache_k[li, :ctx], rep, axis=1)          # (ctx, heads, hd)
            Vc = np.repeat(self.cache_v[li, :ctx], rep, axis=1)
            sc = np.einsum("hd,chd->hc", q, Kc) / math.sqrt(hd)
            p = np.exp(sc - sc.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            att = _f16(np.einsum("hc,chd->hd", p, Vc).reshape(-1))
            x = _f16(x + L["o"](att))
            h = self._norm(x, L["ln2"])
            if self.fuse_qkv:
                y = L["gu"](h)
                g, u = y[:self.MLP], y[self.MLP:]
            else:
                g, u = L["gate"](h), L["up"](h)
            x = _f16(x + L["down"](_f16(_f16(g / (1.0 + np.exp(-g))) * u)))
        logits = self.lm_head @ self._norm(x, self.ln_f)
        top = np.argpartition(-logits, top_k)[:top_k]
        pr = np.exp((logits[top] - logits[top].max()) / max(temperature, 1e-5))
        self.pos += 1
        return int(self.rng.choice(top, p=pr / pr.sum()))
