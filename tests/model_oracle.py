"""CPU evaluation of a QtipLlama model with the oracle (shared by the GPU model test and the tensor-parallel worker)."""
import math

import numpy as np

import c_oracle as C
import qtip_oracle as O
from qtip_b200 import ops


def oracle_logits(model, tokens, tp=1):
    """The model (an UNSHARDED QtipLlama: tp_size = 1) evaluated with the CPU oracle: every linear is
    C.layer_forward (restating BitshiftLinear.forward upstream, lib/codebook/bitshift.py:415-472), everything
    between the linears is numpy in the precision of the fp16 torch modules (model/llama.py upstream:
    LlamaRMSNorm, rotary embedding, softmax attention, SwiGLU).  Nothing of the CUDA library is used.
    tp > 1 evaluates the tensor-parallel parametrisation of the same buffers: Hadamard transform per 1/tp chunk on
    the output side of q, k, v, gate, up (rcp = 2) and on the input side of o, down (rcp = 1), :437-441, :465-469."""
    s = model.shape
    f16 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)   # noqa: E731

    def hadk(n):
        return None if O.had_factor(n) == 1 else ops.get_hadK(n)[0].numpy()

    def lin(l, v, rcp=0):
        hl = hadk(l.n // tp if rcp == 1 else l.n)
        hr = hadk(l.m // tp if rcp == 2 else l.m)
        y = C.layer_forward(v.astype(np.float32), l.codes.cpu().numpy().view(np.uint16), l.m, l.n, l.K,
                            l.tlut.cpu().numpy(), l.SU.float().cpu().numpy(), l.SV.cpu().numpy(), hl, hr,
                            rcp=rcp if tp > 1 else 0, tp=tp)
        return f16(y.reshape(-1))

    def lin_chunks(l, v, chunks):
        """A fused matrix (q||k||v or gate||up): one input side, the output-side transform per chunk of out_features
        (upstream's rcp = 2 layout with `chunks` chunks)."""
        y = C.layer_forward(v.astype(np.float32), l.codes.cpu().numpy().view(np.uint16), l.m, l.n, l.K,
                            l.tlut.cpu().numpy(), l.SU.float().cpu().numpy(), l.SV.cpu().numpy(), hadk(l.n),
                            hadk(l.m // chunks), rcp=2, tp=chunks)
        return np.split(f16(y.reshape(-1)), chunks)

    COL, ROW = (2, 1) if tp > 1 else (0, 0)

    def norm(v, w):
        hn = f16(v * (1.0 / np.sqrt(np.mean(v.astype(np.float32) ** 2) + s.rms_eps)))
        return f16(w.float().cpu().numpy() * hn)

    embed = model.embed.float().cpu().numpy()
    half = s.head_dim // 2
    inv = s.rope_theta ** (-np.arange(half, dtype=np.float64) * 2 / s.head_dim)
    ks, vs = [[] for _ in range(s.n_layers)], [[] for _ in range(s.n_layers)]
    logits = None
    for pos, tok in enumerate(tokens):
        x = embed[tok].copy()
        cs, sn = np.cos(pos * inv), np.sin(pos * inv)

        def rope(t):
            t = t.reshape(-1, s.head_dim).astype(np.float64)
            a, b = t[:, :half], t[:, half:]
            return f16(np.concatenate([a * cs - b * sn, b * cs + a * sn], axis=1))

        for li, L in enumerate(model.layers):
            h = norm(x, L["ln1"])
            if "qkv" in L:
                q, k, v = lin_chunks(L["qkv"], h, 3)
            else:
                q, k, v = lin(L["q"], h, COL), lin(L["k"], h, COL), lin(L["v"], h, COL)
            q, k, v = rope(q), rope(k), v.reshape(-1, s.head_dim)
            ks[li].append(k); vs[li].append(v)
            Kc, Vc = np.stack(ks[li], 1).astype(np.float64), np.stack(vs[li], 1).astype(np.float64)   # (heads, ctx, hd)
            sc = np.einsum("hd,hcd->hc", q.astype(np.float64), Kc) / math.sqrt(s.head_dim)
            p = np.exp(sc - sc.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            att = f16(np.einsum("hc,hcd->hd", p, Vc).reshape(-1))
            x = f16(x + lin(L["o"], att, ROW))
            h = norm(x, L["ln2"])
            g, u = lin_chunks(L["gu"], h, 2) if "gu" in L else (lin(L["gate"], h, COL), lin(L["up"], h, COL))
            act = f16(f16(g / (1.0 + np.exp(-g))) * u)
            x = f16(x + lin(L["down"], act, ROW))
        h = norm(x, model.ln_f)
        logits = h @ model.lm_head.float().cpu().numpy().T
    return logits
