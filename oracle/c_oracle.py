"""ctypes binding of oracle/libqtip_oracle.so (the C restatement).  TEST INFRASTRUCTURE ONLY:
imported by tests/, the smoke check and the benchmark's CPU-baseline legs, never by the product."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libqtip_oracle.so")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "qtip_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libqtip_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.qo_init()
        _lib.qo_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def num_threads():
    return lib().qo_num_threads()


def use_all_cores():
    lib().qo_set_num_threads(os.cpu_count() or 1)
    return num_threads()


def float_to_half(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().qo_float_to_half(_p(x), _p(y), ctypes.c_long(x.size))
    return y.view(np.float16)


def hyb_expand_lut(tlut):
    t = np.ascontiguousarray(tlut, dtype=np.float16).reshape(-1)
    out = np.empty((65536, 2), dtype=np.float16)
    lib().qo_hyb_expand_lut(_p(t), _p(out))
    return out


def code_table(code):
    out = np.empty(65536, dtype=np.float16)
    lib().qo_code_table(ctypes.c_int(code), _p(out))
    return out


def decode_kernel(codes, m, n, K, tlut):
    c = np.ascontiguousarray(codes).reshape(-1)
    t = np.ascontiguousarray(tlut, dtype=np.float16).reshape(-1)
    W = np.empty((m, n), dtype=np.float16)
    lib().qo_decode_kernel(_p(c), m, n, K, _p(t), _p(W))
    return W


def decode_plain(codes, m, n, K, V, table):
    c = np.ascontiguousarray(codes).reshape(-1)
    t = np.ascontiguousarray(table, dtype=np.float16).reshape(-1)
    W = np.empty((m, n), dtype=np.float16)
    lib().qo_decode_plain(_p(c), m, n, K, V, _p(t), _p(W))
    return W


def matvec_dense(W, x):
    W = np.ascontiguousarray(W, dtype=np.float16)
    x = np.ascontiguousarray(x, dtype=np.float16)
    m, n = W.shape
    bs = x.size // n
    y = np.empty((bs, m), dtype=np.float32)
    lib().qo_matvec_dense(_p(W), _p(x), m, n, bs, _p(y))
    return y


def matvec_kernel(codes, m, n, K, tlut, x):
    c = np.ascontiguousarray(codes).reshape(-1)
    t = np.ascontiguousarray(tlut, dtype=np.float16).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float16)
    bs = x.size // n
    y = np.empty((bs, m), dtype=np.float32)
    lib().qo_matvec_kernel(_p(c), m, n, K, _p(t), _p(x), bs, _p(y))
    return y


def hadamard(x, hadK=None, transpose=False):
    x = np.array(x, dtype=np.float32, order="C", copy=True)
    n = x.shape[-1]
    k = 1 if hadK is None else hadK.shape[0]
    hk = None if hadK is None else np.ascontiguousarray(hadK, dtype=np.float32)
    lib().qo_hadamard(_p(x), ctypes.c_long(x.size // n), n, _p(hk), k, int(transpose))
    return x


def layer_forward(x, codes, m, n, K, tlut, SU, SV, had_left=None, had_right=None, rcp=0, tp=1):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, n)
    bs = x.shape[0]
    c = np.ascontiguousarray(codes).reshape(-1)
    t = np.ascontiguousarray(tlut, dtype=np.float16).reshape(-1)
    su = np.ascontiguousarray(SU, dtype=np.float32)
    sv = np.ascontiguousarray(SV, dtype=np.float32)
    hl = None if had_left is None else np.ascontiguousarray(had_left, dtype=np.float32)
    hr = None if had_right is None else np.ascontiguousarray(had_right, dtype=np.float32)
    y = np.empty((bs, m), dtype=np.float32)
    lib().qo_layer_forward(_p(x), bs, _p(c), m, n, K, _p(t), _p(su), _p(sv), _p(hl),
                           1 if hl is None else hl.shape[0], _p(hr), 1 if hr is None else hr.shape[0],
                           rcp, tp, _p(y))
    return y


def viterbi_quantize(X, K, V, recons):
    """bitshift_codebook.quantize (lib/codebook/bitshift.py:283-292): X (N, T) fp16 sequences, recons (V, 65536) fp32
    (upstream's recons_state) -> (states (N, T/V) int32, final path cost (N,) fp32)."""
    X = np.ascontiguousarray(X, dtype=np.float16)
    N, T = X.shape
    recons = np.ascontiguousarray(recons, dtype=np.float32).reshape(V, 65536)
    states = np.empty((N, T // V), dtype=np.int32)
    cost = np.empty(N, dtype=np.float32)
    lib().qo_viterbi_quantize(_p(X.view(np.uint16)), ctypes.c_long(N), ctypes.c_int(T), ctypes.c_int(K), ctypes.c_int(V),
                              _p(recons), _p(states), _p(cost))
    return states, cost
