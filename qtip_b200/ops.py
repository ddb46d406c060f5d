"""Tensor-level wrappers over the C ABI (include/qtip_b200.h).

All functions run on the tensors' CUDA device and the current torch stream, never synchronise,
and raise RuntimeError on any non-zero status.  There is no CPU path.
"""
import math
import os

import numpy as np
import torch

from . import _lib
from ._lib import CODE_1MAD, CODE_3INST, CODE_HYB, F16, F32  # noqa: F401

CODE_IDS = {"quantlut_sym": CODE_HYB, "hyb": CODE_HYB, "3inst": CODE_3INST, "1mad": CODE_1MAD}
HAD_FACTORS = (172, 156, 140, 124, 116, 108, 60, 52, 36, 28, 20, 12)
MAX_MATVEC_BATCH = 8
MAX_GEMM_BATCH = 128
launch_count = 0   # kernel launches issued through this module (bench.py reports it)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("qtip_b200 runs on CUDA tensors only (no CPU fallback)")


def _check_device(*tensors):
    """The preallocated-tensor wrappers launch on the CURRENT device and stream (they must stay free of
    device switches so that a step can be captured into a CUDA graph): refuse tensors that live elsewhere
    instead of launching a kernel on one GPU with another GPU's pointers."""
    cur = torch.cuda.current_device()
    for t in tensors:
        if t is not None and t.device.index != cur:
            raise RuntimeError(f"tensor on cuda:{t.device.index} but the current device is cuda:{cur}: "
                               "call torch.cuda.set_device() / use torch.cuda.device() around qtip_b200 launches")


def _dtype_id(t):
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise RuntimeError(f"unsupported dtype {t.dtype} (fp16 / fp32 only)")


# ---------------------------------------------------------------------------------------------
# Hadamard factor matrices
# ---------------------------------------------------------------------------------------------
_HADK_NPZ = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "hadk.npz")
_hadk_cpu = {}
_hadk_bits_dev = {}


def had_factor(n):
    """Factor order K of n = K * 2^p, first match in the order of get_hadK upstream
    (lib/utils/matmul_had.py:9-63); 1 for a power of two."""
    for k in HAD_FACTORS:
        if n % k == 0:
            q = n // k
            if q & (q - 1) != 0:
                raise ValueError(f"{n} / {k} is not a power of two")
            return k
    if n <= 0 or n & (n - 1):
        raise ValueError(f"{n} has no supported Hadamard factorisation")
    return 1


def get_hadK(n, transpose=False):
    """(hadK fp32 (K, K) or None, K) for a width n - the contract of get_hadK upstream."""
    k = had_factor(n)
    if k == 1:
        return None, 1
    if k not in _hadk_cpu:
        with np.load(_HADK_NPZ) as z:
            bits = np.unpackbits(z[f"had{k}"])[:k * k].reshape(k, k)
        _hadk_cpu[k] = torch.from_numpy(bits.astype(np.float32) * 2 - 1)
    h = _hadk_cpu[k]
    return (h.T.contiguous() if transpose else h.clone()), k


def pack_hadk(hadK):
    """+-1 matrix (K, K) -> int32 tensor (K, ceil(K/32)) of sign bits for qtip_rht, on hadK's device."""
    k = hadK.shape[0]
    wpr = (k + 31) // 32
    bits = (hadK > 0).to(torch.int64)
    pad = torch.zeros(k, wpr * 32, dtype=torch.int64, device=hadK.device)
    pad[:, :k] = bits
    w = (pad.view(k, wpr, 32) << torch.arange(32, device=hadK.device, dtype=torch.int64)).sum(-1)
    w = torch.where(w >= 2**31, w - 2**32, w)
    return w.to(torch.int32).contiguous()


def hadk_bits_for(hadK, device):
    """Device-resident packed signs of a factor matrix, cached by (order, device, content hash)."""
    if hadK is None:
        return None
    k = hadK.shape[0]
    key = (k, str(device), hadK.data_ptr(), hadK._version)
    hit = _hadk_bits_dev.get(key)
    if hit is None:
        hit = pack_hadk(hadK.detach().to(device=device, dtype=torch.float32))
        _hadk_bits_dev[key] = hit
    return hit


# ---------------------------------------------------------------------------------------------
# workspace for the fused matvec (ticket counters + partial sums), zeroed once at allocation
# ---------------------------------------------------------------------------------------------
_workspaces = {}


def matvec_workspace(m, n, bs, device):
    """A zero-initialised workspace tensor private to (device, current stream)."""
    need = _lib.load().qtip_matvec_workspace_bytes(m, n, bs)
    key = (torch.device(device).index, _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


# ---------------------------------------------------------------------------------------------
# ops
# ---------------------------------------------------------------------------------------------
def decode_hyb(codes, tlut, K, m, n, out=None):
    """Kernel-layout HYB codes -> (m, n) fp16 (decode_compressed upstream)."""
    _require_cuda(codes, tlut)
    codes = codes.contiguous()
    tlut = tlut.to(torch.float16).contiguous()
    if codes.numel() * codes.element_size() != m * n * K // 8:
        raise RuntimeError(f"codes hold {codes.numel() * codes.element_size()} bytes, expected {m * n * K // 8}")
    if out is None:
        out = torch.empty(m, n, dtype=torch.float16, device=codes.device)
    with torch.cuda.device(codes.device):
        st = _lib.load().qtip_decode_hyb(out.data_ptr(), codes.data_ptr(), tlut.data_ptr(), K, m, n, _stream())
    _lib.check(st, "qtip_decode_hyb")
    global launch_count
    launch_count += 1
    return out


def decode_plain(codes, code, K, m, n, tlut=None, out=None):
    """Plain-layout codes of any of the three codes -> (m, n) fp16 (unpack_trellis + get_hatW upstream)."""
    _require_cuda(codes, tlut)
    code = CODE_IDS.get(code, code)
    codes = codes.contiguous()
    if codes.numel() * codes.element_size() != m * n * K // 8:
        raise RuntimeError(f"codes hold {codes.numel() * codes.element_size()} bytes, expected {m * n * K // 8}")
    tl = None if tlut is None else tlut.to(torch.float16).contiguous()
    if out is None:
        out = torch.empty(m, n, dtype=torch.float16, device=codes.device)
    with torch.cuda.device(codes.device):
        st = _lib.load().qtip_decode_plain(out.data_ptr(), codes.data_ptr(), code, None if tl is None else tl.data_ptr(),
                                           K, m, n, _stream())
    _lib.check(st, "qtip_decode_plain")
    global launch_count
    launch_count += 1
    return out


def viterbi_quantize(X, mode, K, tlut=None, return_cost=False):
    """bitshift_codebook.quantize upstream (lib/codebook/bitshift.py:283-292): X (N, T) -> trellis states (N, T/V) int32 of
    the tail-biting minimum-squared-error walk (X is rounded to fp16 first, as upstream does).  mode: 'quantlut_sym'
    (tlut: 512 x 2, used in fp32), '3inst' or '1mad'."""
    _require_cuda(X)
    code = CODE_IDS[mode]
    V = 2 if code == CODE_HYB else 1
    X = X.to(torch.float16).contiguous()
    N, T = X.shape
    tl = None
    if code == CODE_HYB:
        if tlut is None:
            raise RuntimeError("the HYB code needs its 512 x 2 table")
        tl = tlut.to(device=X.device, dtype=torch.float32).contiguous()
        if tl.numel() != 1024:
            raise RuntimeError("tlut must hold 512 x 2 values")
    lib = _lib.load()
    need = lib.qtip_viterbi_workspace_bytes(code, K, T, N)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=X.device)
    states = torch.empty(N, T // V, dtype=torch.int32, device=X.device)
    cost = torch.empty(N, dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        st = lib.qtip_viterbi_quantize(states.data_ptr(), cost.data_ptr(), X.data_ptr(), N, T, code, K,
                                       None if tl is None else tl.data_ptr(), ws.data_ptr(), ws.numel(), _stream())
    _lib.check(st, "qtip_viterbi_quantize")
    global launch_count
    launch_count += 1
    return (states, cost) if return_cost else states


def pack_trellis(states, K, V, check=True):
    """Trellis states (tiles, 256/V) int32 -> packed plain-layout words (tiles, 16K) int16 (pack_trellis upstream).
    check=True counts the state pairs that violate the overlap condition upstream asserts and raises if any."""
    _require_cuda(states)
    states = states.to(torch.int32).contiguous()
    tiles = states.shape[0]
    if states.shape[1] * V != 256:
        raise RuntimeError(f"states must be (tiles, {256 // V}) for V = {V}")
    words = torch.empty(tiles, 16 * K, dtype=torch.int16, device=states.device)
    bad = torch.zeros(1, dtype=torch.int32, device=states.device) if check else None
    with torch.cuda.device(states.device):
        st = _lib.load().qtip_pack_trellis(words.data_ptr(), states.data_ptr(), tiles, K, V,
                                           None if bad is None else bad.data_ptr(), _stream())
    _lib.check(st, "qtip_pack_trellis")
    global launch_count
    launch_count += 1
    if check and int(bad.item()):
        raise RuntimeError(f"pack_trellis: {int(bad.item())} consecutive state pairs do not overlap (not a trellis walk)")
    return words


def plain_to_kernel_layout(words, K, m, n):
    """Plain-layout words (tiles, 16K) -> kernel layout (same shape / dtype); lib/algo/finetune.py:196-201 upstream."""
    _require_cuda(words)
    words = words.contiguous()
    out = torch.empty_like(words)
    with torch.cuda.device(words.device):
        st = _lib.load().qtip_plain_to_kernel_layout(out.data_ptr(), words.data_ptr(), K, m, n, _stream())
    _lib.check(st, "qtip_plain_to_kernel_layout")
    global launch_count
    launch_count += 1
    return out


def kernel_to_plain_layout(codes, K, m, n):
    """Inverse of plain_to_kernel_layout (lib/utils/kernel_decompress.py:19-24 upstream)."""
    _require_cuda(codes)
    codes = codes.contiguous()
    out = torch.empty_like(codes)
    with torch.cuda.device(codes.device):
        st = _lib.load().qtip_kernel_to_plain_layout(out.data_ptr(), codes.data_ptr(), K, m, n, _stream())
    _lib.check(st, "qtip_kernel_to_plain_layout")
    global launch_count
    launch_count += 1
    return out


def decompress_matvec(codes, x, tlut, K, m, n, out=None, workspace=None):
    """out (bs, m) fp32 = x (bs, n) fp16 @ decode(codes)^T, HYB kernel layout, bs <= 8."""
    _require_cuda(codes, x, tlut)
    if x.dtype != torch.float16:
        x = x.to(torch.float16)
    x = x.reshape(-1, n).contiguous()
    bs = x.shape[0]
    if out is None:
        out = torch.empty(bs, m, dtype=torch.float32, device=x.device)
    if workspace is None:
        workspace = matvec_workspace(m, n, bs, x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().qtip_decompress_matvec(out.data_ptr(), codes.data_ptr(), x.data_ptr(), tlut.data_ptr(), K, m,
                                                n, bs, workspace.data_ptr(), workspace.numel(), _stream())
    _lib.check(st, "qtip_decompress_matvec")
    global launch_count
    launch_count += 1
    return out


def decompress_matvec_plain(codes, x, code, K, m, n, out=None, workspace=None):
    """Same for the 3INST / 1MAD compute codes (plain layout, V = 1)."""
    _require_cuda(codes, x)
    code = CODE_IDS.get(code, code)
    if x.dtype != torch.float16:
        x = x.to(torch.float16)
    x = x.reshape(-1, n).contiguous()
    bs = x.shape[0]
    if out is None:
        out = torch.empty(bs, m, dtype=torch.float32, device=x.device)
    if workspace is None:
        workspace = matvec_workspace(m, n, bs, x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().qtip_decompress_matvec_plain(out.data_ptr(), codes.data_ptr(), x.data_ptr(), code, K, m, n, bs,
                                                      workspace.data_ptr(), workspace.numel(), _stream())
    _lib.check(st, "qtip_decompress_matvec_plain")
    global launch_count
    launch_count += 1
    return out


def rht(x, sign_in=None, sign_out=None, hadk_bits=None, kfac=1, transpose=False, scale=1.0, out_dtype=None, out=None):
    """out = sign_out * H(sign_in * x) * scale over the last dim of x (rows, n); see qtip_rht."""
    _require_cuda(x, sign_in, sign_out, hadk_bits)
    n = x.shape[-1]
    x2 = x.reshape(-1, n)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    if out_dtype is None:
        out_dtype = x.dtype
    if out is None:
        out = torch.empty(rows, n, dtype=out_dtype, device=x.device)
    n_signs = n
    if sign_in is not None:
        sign_in = sign_in.contiguous()
        n_signs = sign_in.numel()
    if sign_out is not None:
        sign_out = sign_out.to(torch.float32).contiguous()
        if sign_in is not None and sign_out.numel() != n_signs:
            raise RuntimeError("sign_in and sign_out must have the same length")
        n_signs = sign_out.numel()
    with torch.cuda.device(x.device):
        st = _lib.load().qtip_rht(out.data_ptr(), _dtype_id(out), x2.data_ptr(), _dtype_id(x2), rows, n,
                                  None if sign_in is None else sign_in.data_ptr(),
                                  F16 if sign_in is None else _dtype_id(sign_in),
                                  None if sign_out is None else sign_out.data_ptr(), n_signs,
                                  None if hadk_bits is None else hadk_bits.data_ptr(), kfac, int(bool(transpose)),
                                  float(scale), _stream())
    _lib.check(st, "qtip_rht")
    global launch_count
    launch_count += 1
    return out.reshape(*x.shape[:-1], n)


def hadamard(x, hadK=None, K=1, transpose=False):
    """Orthonormal Hadamard over the last dim: drop-in for matmul_hadU_cuda / matmul_hadUt_cuda
    (lib/utils/matmul_had.py:105-119 upstream)."""
    n = x.shape[-1]
    bits = hadk_bits_for(hadK, x.device) if K > 1 else None
    return rht(x, hadk_bits=bits, kfac=K, transpose=transpose, scale=1.0 / math.sqrt(n))


def rht_fused(x, rows, n, out, *, in_row_stride=None, residual=None, residual_out=None, norm_weight=None, eps=1e-5,
              gate=None, sign_in=None, sign_out=None, hadk_bits=None, kfac=1, transpose=False, scale=1.0):
    """qtip_rht_fused on preallocated tensors (no allocation, graph-capturable); see include/qtip_b200.h."""
    _check_device(x, out, residual, residual_out, norm_weight, gate, sign_in, sign_out, hadk_bits)
    n_signs = n
    if sign_in is not None:
        n_signs = sign_in.numel()
    if sign_out is not None:
        n_signs = sign_out.numel()
    p = lambda t: None if t is None else t.data_ptr()  # noqa: E731
    st = _lib.load().qtip_rht_fused(out.data_ptr(), _dtype_id(out), x.data_ptr(), _dtype_id(x), rows,
                                    n if in_row_stride is None else in_row_stride, n, p(residual), p(residual_out),
                                    p(norm_weight), float(eps), p(gate), p(sign_in),
                                    F16 if sign_in is None else _dtype_id(sign_in), p(sign_out), n_signs, p(hadk_bits),
                                    kfac, int(bool(transpose)), float(scale), _stream())
    _lib.check(st, "qtip_rht_fused")
    global launch_count
    launch_count += 1
    return out


def mlp_mid_supported(n):
    """True when qtip_mlp_mid handles width n (a non-trivial Hadamard factor and a row length of 32..128)."""
    k = had_factor(n)
    return bool(k and k > 1 and _lib.load().qtip_mlp_mid_supported(int(n), int(k)))


_mid_tables = {}


def mlp_mid_table(n, device, hadk_bits=None):
    """Device table of qtip_mlp_mid_prepare for width n (cached per factor order and device)."""
    k = had_factor(n)
    key = (k, str(device), None if hadk_bits is None else hadk_bits.data_ptr())
    t = _mid_tables.get(key)
    if t is None:
        if hadk_bits is None:
            hadk_bits = pack_hadk(get_hadK(n)[0].to(device))
        lib = _lib.load()
        t = torch.zeros(lib.qtip_mlp_mid_table_bytes(), dtype=torch.uint8, device=device)
        with torch.cuda.device(t.device):
            _lib.check(lib.qtip_mlp_mid_prepare(t.data_ptr(), hadk_bits.data_ptr(), int(n), int(k), _stream()), "qtip_mlp_mid_prepare")
        _mid_tables[key] = t
    return t


def mlp_mid(out, y_gate, y_up, sign_gate, sign_up, sign_down, n, scale_out, scale_in, table=None):
    """qtip_mlp_mid: output side of gate/up + SwiGLU + input side of down_proj, one launch.  out: (n) fp16.
    table: mlp_mid_table(n, device); looked up (and built on first use, which allocates) when omitted."""
    _check_device(out, y_gate, y_up, sign_gate, sign_up, sign_down, table)
    if table is None:
        table = mlp_mid_table(n, out.device)
    st = _lib.load().qtip_mlp_mid(out.data_ptr(), y_gate.data_ptr(), y_up.data_ptr(), sign_gate.data_ptr(), sign_up.data_ptr(),
                                  sign_down.data_ptr(), table.data_ptr(), int(n), int(had_factor(n)),
                                  float(scale_out), float(scale_in), _stream())
    _lib.check(st, "qtip_mlp_mid")
    global launch_count
    launch_count += 1
    return out


def _status_ptr(status):
    return None if status is None else status.data_ptr()


def embed_token(res, delta, embed, token, status=None):
    """qtip_embed_token: res = embed[token], delta = 0.  A token outside the table leaves res / delta alone and
    sets bit 2 of `status` (a one-element int32 / uint32 device tensor)."""
    _check_device(res, delta, embed, token, status)
    _lib.check(_lib.load().qtip_embed_token(res.data_ptr(), delta.data_ptr(), embed.data_ptr(), token.data_ptr(),
                                            embed.shape[1], embed.shape[0], _status_ptr(status), _stream()),
               "qtip_embed_token")
    global launch_count
    launch_count += 1


def lm_head(logits, res, delta, norm_weight, weight, eps):
    """qtip_lm_head: logits = weight @ RMSNorm(res + delta) (fp16 norm semantics of LlamaRMSNorm, fp32 logits)."""
    vocab, hidden = weight.shape
    _check_device(logits, res, delta, norm_weight, weight)
    _lib.check(_lib.load().qtip_lm_head(logits.data_ptr(), res.data_ptr(), delta.data_ptr(), norm_weight.data_ptr(),
                                        weight.data_ptr(), hidden, vocab, float(eps), _stream()), "qtip_lm_head")
    global launch_count
    launch_count += 1
    return logits


def sample_top_k(token, out_tokens, pos, logits, temperature=0.6, top_k=5, seed=0, status=None):
    """qtip_sample_top_k: next token -> token, out_tokens[pos + 1]; pos += 1 (all on the device).  When the token
    log is full the token is not logged and bit 4 of `status` is set."""
    _check_device(token, out_tokens, pos, logits, status)
    _lib.check(_lib.load().qtip_sample_top_k(token.data_ptr(), out_tokens.data_ptr(), pos.data_ptr(), logits.data_ptr(),
                                             logits.numel(), float(temperature), int(top_k), int(seed),
                                             out_tokens.numel(), _status_ptr(status), _stream()),
               "qtip_sample_top_k")
    global launch_count
    launch_count += 1


def rope_kv_append(q, k, v, cache_k, cache_v, pos, n_heads, n_kv_heads, head_dim, theta=10000.0, status=None):
    """The caches are (max_positions, n_kv_heads*head_dim); a position outside them makes the kernel skip its work
    and set bit 1 of `status` (same for the three functions below)."""
    _check_device(q, k, v, cache_k, cache_v, pos, status)
    st = _lib.load().qtip_rope_kv_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                                         pos.data_ptr(), n_heads, n_kv_heads, head_dim, float(theta), cache_k.shape[0],
                                         _status_ptr(status), _stream())
    _lib.check(st, "qtip_rope_kv_append")
    global launch_count
    launch_count += 1


def rope_kv_append_fused(q_out, y_q, y_k, y_v, sign_q, sign_k, sign_v, scale_q, scale_kv, cache_k, cache_v, pos, n_heads,
                         n_kv_heads, head_dim, theta=10000.0, status=None):
    """qtip_rope_kv_append_fused: output side of the q/k/v linears + rotary embedding + cache append, one launch."""
    _check_device(q_out, y_q, y_k, y_v, sign_q, sign_k, sign_v, cache_k, cache_v, pos)
    ptr = lambda t: 0 if t is None else t.data_ptr()   # noqa: E731
    st = _lib.load().qtip_rope_kv_append_fused(q_out.data_ptr(), y_q.data_ptr(), y_k.data_ptr(), y_v.data_ptr(), ptr(sign_q),
                                               ptr(sign_k), ptr(sign_v), float(scale_q), float(scale_kv), cache_k.data_ptr(),
                                               cache_v.data_ptr(), pos.data_ptr(), n_heads, n_kv_heads, head_dim, float(theta),
                                               cache_k.shape[0], _status_ptr(status), _stream())
    _lib.check(st, "qtip_rope_kv_append_fused")
    global launch_count
    launch_count += 1


def attn_decode_fused(out, y_q, y_k, y_v, sign_q, sign_k, sign_v, scale_q, scale_kv, cache_k, cache_v, pos, n_heads,
                      n_kv_heads, head_dim, theta=10000.0, status=None):
    """qtip_attn_decode_fused: output side of q/k/v + rotary + cache append + single-query attention, one launch."""
    _check_device(out, y_q, y_k, y_v, sign_q, sign_k, sign_v, cache_k, cache_v, pos)
    ptr = lambda t: 0 if t is None else t.data_ptr()   # noqa: E731
    st = _lib.load().qtip_attn_decode_fused(out.data_ptr(), y_q.data_ptr(), y_k.data_ptr(), y_v.data_ptr(), ptr(sign_q),
                                            ptr(sign_k), ptr(sign_v), float(scale_q), float(scale_kv), cache_k.data_ptr(),
                                            cache_v.data_ptr(), pos.data_ptr(), n_heads, n_kv_heads, head_dim, float(theta),
                                            cache_k.shape[0], _status_ptr(status), _stream())
    _lib.check(st, "qtip_attn_decode_fused")
    global launch_count
    launch_count += 1
    return out


def attn_decode(out, q, cache_k, cache_v, pos, n_heads, n_kv_heads, head_dim, status=None):
    _check_device(out, q, cache_k, cache_v, pos, status)
    st = _lib.load().qtip_attn_decode(out.data_ptr(), q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), pos.data_ptr(),
                                      n_heads, n_kv_heads, head_dim, cache_k.shape[0], _status_ptr(status), _stream())
    _lib.check(st, "qtip_attn_decode")
    global launch_count
    launch_count += 1
    return out


def linear_fused(descs, K, m, n, bs=1):
    """qtip_linear_fused: one launch for up to four same-shape linears, transforms optionally fused.
    `descs` is a list of dicts with tensor values for the fields of qtip_linear_desc (missing = NULL):
    y, codes, tlut, x, workspace, in_raw, residual, residual_out, norm_weight, gate, sign_in, out, sign_out, in_y,
    in_y_sign plus floats in_scale, eps, out_scale, in_y_scale; for tensor parallelism without an all-reduce launch
    also peer_y / signal_y (lists of device addresses), peer_seq, peer_status, signal_seq (addresses)
    and peer_max_polls."""
    arr = (_lib.LinearDesc * len(descs))()
    for d, c in zip(descs, arr):
        _check_device(*(d.get(name) for name in ("y", "codes", "tlut", "x", "workspace", "in_raw", "out", "in_y")))
        for name in ("y", "codes", "tlut", "x", "workspace", "in_raw", "residual", "residual_out", "norm_weight", "gate",
                     "sign_in", "out", "sign_out", "in_y", "in_y_sign"):
            t = d.get(name)
            setattr(c, name, None if t is None else t.data_ptr())
        c.workspace_bytes = d["workspace"].numel()
        c.in_scale, c.eps, c.out_scale = float(d.get("in_scale", 1.0)), float(d.get("eps", 0.0)), float(d.get("out_scale", 1.0))
        c.in_y_scale = float(d.get("in_y_scale", 1.0))
        # raw device addresses (ints): peer-mapped memory has no tensor on this side
        peers = d.get("peer_y") or []
        c.peer_count = len(peers)
        for q, ptr in enumerate(peers):
            c.peer_y[q] = int(ptr)
        for name in ("peer_seq", "peer_status", "signal_seq"):
            setattr(c, name, int(d[name]) if d.get(name) else None)
        c.peer_max_polls = int(d.get("peer_max_polls", 0))
        sig = d.get("signal_y") or []
        c.signal_count = len(sig)
        for q, ptr in enumerate(sig):
            c.signal_y[q] = int(ptr)
        c.out_dtype = F16 if d.get("out") is None else _dtype_id(d["out"])
    st = _lib.load().qtip_linear_fused(arr, len(descs), K, m, n, bs, _stream())
    _lib.check(st, "qtip_linear_fused")
    global launch_count
    launch_count += 1


_gemm_status = {}


def gemm_status(device):
    """The status word of decompress_gemm on `device` (0 = every launch so far completed its waits)."""
    t = _gemm_status.get(torch.device(device).index)
    return 0 if t is None else int(t.item())


def decompress_gemm(codes, x, tlut, K, m, n, out=None):
    """out (bs, m) fp32 = x (bs, n) fp16 @ decode(codes)^T on the tcgen05 tensor cores, 1 <= bs <= 128."""
    _require_cuda(codes, x, tlut)
    if x.dtype != torch.float16:
        x = x.to(torch.float16)
    x = x.reshape(-1, n).contiguous()
    bs = x.shape[0]
    if out is None:
        out = torch.empty(bs, m, dtype=torch.float32, device=x.device)
    key = x.device.index
    if key not in _gemm_status:
        _gemm_status[key] = torch.zeros(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().qtip_decompress_gemm(out.data_ptr(), codes.data_ptr(), x.data_ptr(), tlut.data_ptr(), K, m, n, bs,
                                              _gemm_status[key].data_ptr(), _stream())
    _lib.check(st, "qtip_decompress_gemm")
    global launch_count
    launch_count += 1
    return out


def decompress_gemm_plain(codes, x, code, K, m, n, out=None):
    """decompress_gemm for the 3INST / 1MAD compute codes (plain layout, V = 1), 1 <= bs <= 128."""
    _require_cuda(codes, x)
    code = CODE_IDS.get(code, code)
    if x.dtype != torch.float16:
        x = x.to(torch.float16)
    x = x.reshape(-1, n).contiguous()
    bs = x.shape[0]
    if out is None:
        out = torch.empty(bs, m, dtype=torch.float32, device=x.device)
    key = x.device.index
    if key not in _gemm_status:
        _gemm_status[key] = torch.zeros(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().qtip_decompress_gemm_plain(out.data_ptr(), codes.data_ptr(), x.data_ptr(), code, K, m, n, bs,
                                                    _gemm_status[key].data_ptr(), _stream())
    _lib.check(st, "qtip_decompress_gemm_plain")
    global launch_count
    launch_count += 1
    return out


def gemm_plain_supported(m, n, bs):
    return 1 <= bs <= MAX_GEMM_BATCH and m % 128 == 0 and n % 64 == 0


def gemm_supported(m, n, bs):
    return MAX_MATVEC_BATCH < bs <= MAX_GEMM_BATCH and m % 128 == 0 and n % 64 == 0
