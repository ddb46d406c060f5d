"""ctypes binding of libqtip_b200.so (the C ABI declared in include/qtip_b200.h).

There is no fallback: if the shared library is missing or a call returns a non-zero status a
RuntimeError is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libqtip_b200.so")

OK, ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_WORKSPACE, ERR_CUDA, ERR_ALIGNMENT, ERR_TOO_LARGE = range(7)
CODE_HYB, CODE_3INST, CODE_1MAD = 0, 1, 2
F16, F32 = 0, 1

_vp, _i, _l, _sz, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_size_t, ctypes.c_float

class LinearDesc(ctypes.Structure):
    """qtip_linear_desc of include/qtip_b200.h."""
    _fields_ = [("y", _vp), ("codes", _vp), ("tlut", _vp), ("x", _vp), ("workspace", _vp), ("workspace_bytes", _sz),
                ("in_raw", _vp), ("residual", _vp), ("residual_out", _vp), ("norm_weight", _vp), ("gate", _vp),
                ("sign_in", _vp), ("in_scale", _f), ("eps", _f), ("out", _vp), ("out_dtype", _i), ("sign_out", _vp),
                ("out_scale", _f), ("in_y", _vp), ("in_y_sign", _vp), ("in_y_scale", _f),
                ("peer_count", _i), ("peer_y", _vp * 8), ("peer_seq", _vp), ("peer_status", _vp),
                ("peer_max_polls", ctypes.c_uint), ("signal_count", _i), ("signal_y", _vp * 8), ("signal_seq", _vp)]


# name -> (restype, argtypes); mirrors include/qtip_b200.h
SIGNATURES = {
    "qtip_status_string": (ctypes.c_char_p, [_i]),
    "qtip_last_cuda_error": (_i, []),
    "qtip_version": (_i, []),
    "qtip_decode_hyb": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "qtip_decode_plain": (_i, [_vp, _vp, _i, _vp, _i, _i, _i, _vp]),
    "qtip_pipe_rate_count": (_i, []),
    "qtip_pipe_rate_name": (ctypes.c_char_p, [_i]),
    "qtip_measure_pipe_rates": (_i, [ctypes.POINTER(ctypes.c_double), _i, _i]),
    "qtip_viterbi_workspace_bytes": (_sz, [_i, _i, _i, _l]),
    "qtip_viterbi_quantize": (_i, [_vp, _vp, _vp, _l, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "qtip_pack_trellis": (_i, [_vp, _vp, _l, _i, _i, _vp, _vp]),
    "qtip_plain_to_kernel_layout": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "qtip_kernel_to_plain_layout": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "qtip_matvec_workspace_bytes": (_sz, [_i, _i, _i]),
    "qtip_decompress_matvec": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "qtip_decompress_matvec_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "qtip_decompress_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "qtip_decompress_gemm_plain": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "qtip_linear_fused": (_i, [ctypes.POINTER(LinearDesc), _i, _i, _i, _i, _i, _vp]),
    "qtip_linear_desc_layout": (_i, [ctypes.POINTER(ctypes.c_size_t), _i]),
    "qtip_decompress_matvec_plain": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "qtip_rht": (_i, [_vp, _i, _vp, _i, _l, _i, _vp, _i, _vp, _l, _vp, _i, _i, _f, _vp]),
    "qtip_rht_fused": (_i, [_vp, _i, _vp, _i, _l, _l, _i, _vp, _vp, _vp, _f, _vp, _vp, _i, _vp, _l, _vp, _i, _i, _f,
                            _vp]),
    "qtip_mlp_mid_supported": (_i, [_i, _i]),
    "qtip_mlp_mid_table_bytes": (_sz, []),
    "qtip_mlp_mid_prepare": (_i, [_vp, _vp, _i, _i, _vp]),
    "qtip_mlp_mid": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp]),
    "qtip_embed_token": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "qtip_lm_head": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "qtip_sample_top_k": (_i, [_vp, _vp, _vp, _vp, _i, _f, _i, ctypes.c_ulonglong, _i, _vp, _vp]),
    "qtip_rope_kv_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp, _vp]),
    "qtip_rope_kv_append_fused": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp,
                                       _vp]),
    "qtip_attn_decode_fused": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp, _vp]),
    "qtip_attn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
}

_lib = None


def load():
    """Load the library (once).  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(f"{SO_PATH} is missing: build it with `python -m qtip_b200.build` "
                               "(qtip_b200 has no fallback path)")
        lib = ctypes.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        check_desc_layout(lib)
        _lib = lib
    return _lib


def check_desc_layout(lib):
    """The ctypes mirror of qtip_linear_desc against the compiled struct (size and every field offset): a mirror that is
    out of step would hand the kernels pointer bits as counts and limits."""
    n = lib.qtip_linear_desc_layout(None, 0)
    got = (ctypes.c_size_t * n)()
    lib.qtip_linear_desc_layout(got, n)
    want = [ctypes.sizeof(LinearDesc)] + [getattr(LinearDesc, name).offset for name, _ in LinearDesc._fields_]
    if list(got) != want:
        raise RuntimeError(f"qtip_linear_desc layout mismatch between {SO_PATH} and qtip_b200/_lib.py: library {list(got)}, "
                           f"binding {want}")


def check(status, what):
    if status != OK:
        lib = load()
        msg = lib.qtip_status_string(status).decode()
        extra = f" (cudaError {lib.qtip_last_cuda_error()})" if status == ERR_CUDA else ""
        raise RuntimeError(f"{what}: {msg}{extra}")
