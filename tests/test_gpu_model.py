"""GPU: the decode harness (six launches per decoder layer of the Llama-2-7B shape, one CUDA graph per step) against
(a) a plain torch evaluation of the same random-init model from dense decoded weights - the self-consistency check
of the fused path on a tiny shape, where the fused kernels take their shared-memory fall-backs - and (b) the CPU
oracle at the benchmarked layer shape (hidden 4096, MLP 11008), where every fused path is live."""
import math

import numpy as np
import pytest
import torch

import qtip_oracle as O
from conftest import rel_l2
from model_oracle import oracle_logits
from qtip_b200 import ops
from qtip_b200.llama import LlamaShape, QtipLlama

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TINY = LlamaShape(n_layers=2, hidden=256, n_heads=2, n_kv_heads=2, head_dim=128, mlp=1376, vocab=512, K=2)


def had_matrix(n):
    """Dense orthonormal Hadamard matrix of the transform x -> hadamard(x) (float64, from the oracle)."""
    k = O.had_factor(n)
    hk = None if k == 1 else ops.get_hadK(n)[0].numpy()
    return torch.from_numpy(O.hadamard(np.eye(n), hk)).T.contiguous()  # row i of eye -> column i


def dense_linear(lin, x, Hn, Hm):
    """y = Had_m( (Had_n^T (x*SU) / 32).half @ W^T ) * SV*32 in float64 (BitshiftLinear.forward upstream)."""
    W = ops.decode_hyb(lin.codes, lin.tlut, lin.K, lin.m, lin.n).double()
    xs = (x.double() * lin.SU.double()) @ Hn.to(x.device) / 32       # Hn is H^T applied from the right: x @ H^T... see below
    y = xs.half().double() @ W.T
    return (y @ Hm.to(x.device)) * lin.SV32.double()


def reference_logits(model, tokens):
    s = model.shape
    H = s.n_heads * s.head_dim
    # hadamard(x) = Hmat @ x  =>  for row vectors x @ Hmat.T ; the input side uses the transposed transform
    Hh, Hm_ = had_matrix(s.hidden).to(DEV), had_matrix(s.mlp).to(DEV)
    # forward transform of a row vector: x @ Hmat.T ; transposed transform: x @ Hmat
    fwd = {s.hidden: Hh.T.contiguous(), s.mlp: Hm_.T.contiguous()}
    tr = {s.hidden: Hh, s.mlp: Hm_}
    ks, vs = [[] for _ in range(s.n_layers)], [[] for _ in range(s.n_layers)]
    logits = None
    for pos, tok in enumerate(tokens):
        x = model.embed[tok].double()

        def norm(v, w):
            v32 = v.float()
            hn = (v32 * torch.rsqrt(v32.pow(2).mean() + s.rms_eps)).half()
            return (w * hn).double()

        def lin(l, v):
            return dense_linear(l, v, tr[l.n], fwd[l.m]).half().double()

        for li, L in enumerate(model.layers):
            h = norm(x.half(), L["ln1"])
            q, k, v = lin(L["q"], h), lin(L["k"], h), lin(L["v"], h)
            half = s.head_dim // 2
            inv = s.rope_theta ** (-torch.arange(half, device=DEV, dtype=torch.float64) * 2 / s.head_dim)
            cs, sn = torch.cos(pos * inv), torch.sin(pos * inv)

            def rope(t):
                t = t.view(-1, s.head_dim)
                a, b = t[:, :half], t[:, half:]
                return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=1).half().double()

            q, k = rope(q), rope(k)
            ks[li].append(k); vs[li].append(v.view(-1, s.head_dim))
            Kc, Vc = torch.stack(ks[li], 1), torch.stack(vs[li], 1)            # (heads, ctx, hd)
            att = torch.softmax((q.unsqueeze(1) @ Kc.transpose(1, 2)) / math.sqrt(s.head_dim), dim=-1) @ Vc
            x = (x.half() + lin(L["o"], att.reshape(-1).half().double()).half()).double()
            h = norm(x.half(), L["ln2"])
            g, u = lin(L["gate"], h), lin(L["up"], h)
            act = (torch.nn.functional.silu(g.float()).half() * u.half()).double()
            x = (x.half() + lin(L["down"], act).half()).double()
        h = norm(x.half(), model.ln_f)
        logits = h.half().float() @ model.lm_head.float().T
    return logits


def test_decode_step_matches_dense_reference():
    torch.manual_seed(0)
    model = QtipLlama(TINY, max_positions=16, device=DEV, seed=11)
    tokens = [3, 77, 400, 9, 250]
    model.reset()
    for t in tokens:
        model.token.fill_(t)
        model.step()
    got = model.logits.clone()
    want = reference_logits(model, tokens)
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 2e-2
    assert int(model.pos.item()) == len(tokens)


def test_graph_replay_matches_eager():
    model = QtipLlama(TINY, max_positions=16, device=DEV, seed=12)
    tokens = torch.tensor([5, 6, 7, 8])
    model.reset()
    for t in tokens.tolist():
        model.token.fill_(t)
        model.step()
    eager = model.logits.clone()
    model.reset()
    model.capture()
    model.reset()
    model.feed(tokens)
    torch.cuda.synchronize()
    assert torch.equal(model.logits, eager)
    model.generate(3)
    torch.cuda.synchronize()
    assert int(model.pos.item()) == 7
    assert torch.all(model.out_tokens[1:8] >= 0) and torch.all(model.out_tokens[1:8] < TINY.vocab)


# ---------------------------------------------------------------------------------------------------------
# the benchmarked launch graph (register transforms, deferred output sides, fused attention, MLP middle) vs the oracle
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("fuse_qkv", [False, True])
def test_decode_step_at_the_benchmarked_shape_matches_the_oracle(fuse_qkv):
    """hidden 4096 / 32 heads / MLP 11008: the shape whose decode graph the benchmark times.  Here the input
    transforms run in registers inside the matvec launches, the output sides of o_proj / down_proj are deferred into
    the next launch, attention runs fused with the q/k/v output sides and the MLP middle is the cluster kernel.
    fuse_qkv: q||k||v and gate||up as one 12288 x 4096 and one 22016 x 4096 matrix (upstream's fused layers)."""
    shape = LlamaShape(n_layers=2, hidden=4096, n_heads=32, n_kv_heads=32, head_dim=128, mlp=11008, vocab=2048, K=2)
    model = QtipLlama(shape, max_positions=8, device=DEV, seed=21, fuse_qkv=fuse_qkv)
    assert model.defer_h and model.attn_fused and model.mid_fused and model.fuse_in_h and model.fuse_in_hl
    tokens = [7, 1999, 345]
    model.reset()
    for t in tokens:
        model.token.fill_(t)
        model.step()
    eager = model.logits.clone()
    want = oracle_logits(model, tokens)
    err = rel_l2(eager.cpu().numpy().reshape(-1), want.reshape(-1))
    assert err < 5e-3, err
    # and the captured graph replays to the same logits
    model.reset()
    model.capture()
    model.reset()
    model.feed(torch.tensor(tokens))
    torch.cuda.synchronize()
    assert torch.equal(model.logits, eager)
    model.check_status()


def test_batched_decode_matches_single_sequence_decode():
    """step_batch (B sequences in lockstep, unfused launches, batch rows inside the matvec) against step() run once per
    sequence on the same tokens."""
    shape = LlamaShape(n_layers=2, hidden=4096, n_heads=32, n_kv_heads=32, head_dim=128, mlp=11008, vocab=2048, K=2)
    seqs = [[5, 900, 33], [1200, 7, 7], [64, 65, 66]]
    model = QtipLlama(shape, max_positions=8, device=DEV, seed=31)
    want = []
    for toks in seqs:
        model.reset()
        for t in toks:
            model.token.fill_(t)
            model.step()
        want.append(model.logits.clone().reshape(-1))
    model.enable_batch(len(seqs))
    for i in range(3):
        model.b_token.copy_(torch.tensor([s_[i] for s_ in seqs], device=DEV))
        model.step_batch()
    torch.cuda.synchronize()
    assert model.b_pos.tolist() == [3, 3, 3]
    for b in range(len(seqs)):
        assert rel_l2(model.b_logits[b].cpu().numpy(), want[b].cpu().numpy()) < 5e-3
    model.check_status()


def test_state_dict_round_trip_into_decode_model():
    """A synthetic checkpoint with upstream's keys, shapes and dtypes (lib/linear/quantized_linear.py:41-67) loaded into
    a differently seeded model reproduces the source model's logits bit for bit; wrong shapes and tensor-parallel
    layouts are refused."""
    from qtip_b200.checkpoint import export_state_dict, load_state_dict_into
    qp = dict(L=16, K=2, V=2, tlut_bits=9, decode_mode="quantlut_sym", td_x=16, td_y=16, skip_list=None)
    src = QtipLlama(TINY, max_positions=8, device=DEV, seed=41)
    sd = export_state_dict(src)
    assert sd["model.layers.0.self_attn.q_proj.trellis"].dtype == torch.int16
    assert sd["model.layers.1.mlp.down_proj.SV"].dtype == torch.float32 and sd["model.layers.0.mlp.up_proj.tlut"].shape == (512, 2)
    dst = load_state_dict_into(QtipLlama(TINY, max_positions=8, device=DEV, seed=42), sd, qp)
    out = []
    for model in (src, dst):
        model.reset()
        for t in (3, 9, 27):
            model.token.fill_(t)
            model.step()
        out.append(model.logits.clone())
    assert torch.equal(out[0], out[1])
    bad = dict(sd)
    bad["model.layers.0.mlp.up_proj.trellis"] = bad["model.layers.0.mlp.up_proj.trellis"][:-1]
    with pytest.raises(ValueError, match="up_proj.trellis"):
        load_state_dict_into(QtipLlama(TINY, max_positions=8, device=DEV, seed=43), bad, qp)
    bad = dict(sd)
    bad["model.layers.1.self_attn.o_proj.rcp"] = torch.tensor(1)
    with pytest.raises(ValueError, match="rcp"):
        load_state_dict_into(QtipLlama(TINY, max_positions=8, device=DEV, seed=43), bad, qp)
