"""CPU: the C-ABI library loads, exports every symbol the header declares, and validates arguments
before touching the device (no compute call is made here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from qtip_b200 import _lib


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qtip_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qtip_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert names, "no declarations found"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_binding_argument_counts_match_header():
    text = open(os.path.join(ROOT, "include", "qtip_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, params in re.findall(r"\b(qtip_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        params = params.strip()
        count = 0 if params in ("", "void") else params.count(",") + 1
        assert count == len(_lib.SIGNATURES[name][1]), f"{name}: header has {count} parameters"


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(_lib.SO_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/qtip_b200.h but not exported"


def test_linear_desc_mirror_matches_the_compiled_struct():
    lib = ctypes.CDLL(_lib.SO_PATH)
    lib.qtip_linear_desc_layout.restype = ctypes.c_int
    lib.qtip_linear_desc_layout.argtypes = [ctypes.POINTER(ctypes.c_size_t), ctypes.c_int]
    n = lib.qtip_linear_desc_layout(None, 0)
    assert n == 1 + len(_lib.LinearDesc._fields_)
    got = (ctypes.c_size_t * n)()
    assert lib.qtip_linear_desc_layout(got, n) == n
    assert got[0] == ctypes.sizeof(_lib.LinearDesc)
    for k, (name, _) in enumerate(_lib.LinearDesc._fields_):
        assert got[1 + k] == getattr(_lib.LinearDesc, name).offset, name
    # the header declares the fields in the same order as the binding
    text = open(os.path.join(ROOT, "include", "qtip_b200.h")).read()
    body = re.search(r"typedef struct qtip_linear_desc \{(.*?)\} qtip_linear_desc;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = [re.search(r"(\w+)(\[\d+\])?\s*$", d.strip()).group(1) for d in body.split(";") if d.strip()]
    assert names == [name for name, _ in _lib.LinearDesc._fields_]
    # a mirror that is out of step is refused at load time
    class Short(ctypes.Structure):
        _fields_ = _lib.LinearDesc._fields_[:-1]
    orig = _lib.LinearDesc
    try:
        _lib.LinearDesc = Short
        with pytest.raises(RuntimeError, match="layout mismatch"):
            _lib.check_desc_layout(lib)
    finally:
        _lib.LinearDesc = orig


def test_status_strings():
    lib = _lib.load()
    assert lib.qtip_status_string(0) == b"ok"
    for s in range(1, 6):
        assert lib.qtip_status_string(s) not in (b"ok", b"unknown status")
    assert lib.qtip_status_string(99) == b"unknown status"
    assert lib.qtip_version() >= 1


def test_argument_validation_without_device():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    assert lib.qtip_decode_hyb(None, p, p, 2, 32, 32, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_decode_hyb(p, p, p, 5, 32, 32, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_decode_hyb(p, p, p, 2, 48, 32, None) == _lib.ERR_BAD_SHAPE
    assert lib.qtip_decode_hyb(p, p + 4, p, 2, 32, 32, None) == _lib.ERR_ALIGNMENT
    assert lib.qtip_decode_plain(p, p, 7, p, 2, 32, 32, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_decode_plain(p, p, _lib.CODE_HYB, None, 2, 32, 32, None) == _lib.ERR_BAD_ARG
    need = lib.qtip_matvec_workspace_bytes(64, 64, 1)
    assert need >= 256
    assert lib.qtip_decompress_matvec(p, p, p, p, 2, 64, 64, 9, p, need, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_decompress_matvec(p, p, p, p, 2, 64, 64, 1, None, 0, None) == _lib.ERR_WORKSPACE
    assert lib.qtip_decompress_matvec(p, p, p, p, 2, 64, 64, 1, p, need - 1, None) == _lib.ERR_WORKSPACE
    assert lib.qtip_decompress_matvec(p, p, p, p, 2, 64, 40, 1, p, need, None) == _lib.ERR_BAD_SHAPE
    assert lib.qtip_decompress_matvec_plain(p, p, p, _lib.CODE_HYB, 2, 64, 64, 1, p, need, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_rht(p, 0, p, 0, 1, 24, None, 0, None, 24, None, 1, 0, 1.0, None) == _lib.ERR_BAD_SHAPE
    assert lib.qtip_rht(p, 0, p, 0, 1, 344, None, 0, None, 344, None, 172, 0, 1.0, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_rht(p, 3, p, 0, 1, 64, None, 0, None, 64, None, 1, 0, 1.0, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_rht(p, 0, p, 0, 0, 64, None, 0, None, 64, None, 1, 0, 1.0, None) == _lib.OK  # zero rows: nothing to do
    # producers of the packed formats
    assert lib.qtip_pack_trellis(p, p, 0, 2, 2, None, None) == _lib.ERR_BAD_ARG          # no tiles
    assert lib.qtip_pack_trellis(p, p, 4, 2, 3, None, None) == _lib.ERR_BAD_ARG          # V is 1 or 2
    assert lib.qtip_pack_trellis(p, p + 2, 4, 2, 2, None, None) == _lib.ERR_ALIGNMENT
    assert lib.qtip_plain_to_kernel_layout(p, p, 2, 32, 32, None) == _lib.ERR_BAD_ARG     # in place
    assert lib.qtip_plain_to_kernel_layout(p, p + 2048, 2, 48, 32, None) == _lib.ERR_BAD_SHAPE
    assert lib.qtip_kernel_to_plain_layout(p, p + 2048, 5, 32, 32, None) == _lib.ERR_BAD_ARG
    need = lib.qtip_viterbi_workspace_bytes(_lib.CODE_HYB, 2, 256, 4)
    assert need == 4 * 128 * 4096
    assert lib.qtip_viterbi_workspace_bytes(_lib.CODE_3INST, 2, 256, 1000) == 148 * 256 * 16384 or \
        lib.qtip_viterbi_workspace_bytes(_lib.CODE_3INST, 2, 256, 1000) % (256 * 16384) == 0
    assert lib.qtip_viterbi_workspace_bytes(7, 2, 256, 4) == 0
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 256, _lib.CODE_HYB, 2, None, p, need, None) == _lib.ERR_BAD_ARG      # no table
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 256, _lib.CODE_HYB, 5, p, p, need, None) == _lib.ERR_BAD_ARG
    assert lib.qtip_viterbi_quantize(p, None, p, 0, 256, _lib.CODE_3INST, 2, None, p, need, None) == _lib.ERR_BAD_ARG     # no sequences
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 6, _lib.CODE_HYB, 2, p, p, need, None) == _lib.ERR_BAD_SHAPE          # T % 2V
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 2048, _lib.CODE_HYB, 2, p, p, need, None) == _lib.ERR_BAD_SHAPE
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 4, _lib.CODE_3INST, 2, None, p, need, None) == _lib.ERR_BAD_SHAPE     # 8 stream bits
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 256, _lib.CODE_HYB, 2, p, p, need - 1, None) == _lib.ERR_WORKSPACE
    assert lib.qtip_viterbi_quantize(p, None, p, 4, 256, _lib.CODE_HYB, 2, p + 4, p, need, None) == _lib.ERR_ALIGNMENT
    assert lib.qtip_measure_pipe_rates(None, 10, 1024) == _lib.ERR_BAD_ARG
    assert lib.qtip_pipe_rate_count() == 10 and lib.qtip_pipe_rate_name(0).startswith(b"IMAD") and lib.qtip_pipe_rate_name(99) == b""


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "SO_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from qtip_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.decode_hyb(torch.zeros(32 * 32 * 2 // 16, dtype=torch.int16), torch.zeros(512, 2, dtype=torch.float16), 2, 32, 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.rht(torch.zeros(1, 64))
