"""GPU: the allocation-free matvec entry point (scratch inside the library image) against the ordinary one.

Collected last on purpose: a run that stops at the first failure has then already run everything else.
The calls go straight through the C ABI.  Two calls in a row share the built-in scratch array, so the
second one starts from whatever the first left behind.
"""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from qtip_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a):
    return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(DEV)


def _static_call(lay, K, m, n, bs):
    codes, x, tlut = _dev(lay["codes"]), _dev(lay["x"]), _dev(lay["tlut"])
    out = torch.full((bs, m), float("nan"), device=DEV)
    with torch.cuda.device(DEV):
        st = _lib.load().qtip_decompress_matvec_static(out.data_ptr(), codes.data_ptr(), x.data_ptr(), tlut.data_ptr(), K,
                                                       m, n, bs, torch.cuda.current_stream().cuda_stream)
    assert st == _lib.OK, _lib.load().qtip_status_string(st)
    want = ops.decompress_matvec(codes, x, tlut, K, m, n)
    torch.cuda.synchronize()
    return out, want


def test_static_scratch_matches_workspace_version_twice_in_a_row():
    # (1024, 8192) is split across CTAs by columns, so tickets and partial sums in the scratch are really used;
    # the second call has another shape and bit width and reuses the same array.
    cases = [(2, 1024, 8192, 1, 91), (3, 4096, 4096, 4, 92)]
    for (K, m, n, bs, seed) in cases:
        lay = synth.make_layer(m, n, K, seed=seed, bs=bs)
        got, want = _static_call(lay, K, m, n, bs)
        assert not torch.isnan(got).any()
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 2e-6
    # and once more on the first problem: leftovers of the second call must not matter
    K, m, n, bs, seed = cases[0]
    got, want = _static_call(synth.make_layer(m, n, K, seed=seed, bs=bs), K, m, n, bs)
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 2e-6


def test_static_scratch_rejects_oversized_problem():
    lib = _lib.load()
    m, n = 262144, 32   # 8192 row blocks need 16 MiB of partial-sum slots
    assert lib.qtip_matvec_workspace_bytes(m, n, 1) > 4 * 1024 * 1024 + 65792
    buf = torch.zeros(1024, dtype=torch.uint8, device=DEV)
    with torch.cuda.device(DEV):
        st = lib.qtip_decompress_matvec_static(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 2, m, n, 1,
                                               torch.cuda.current_stream().cuda_stream)
    assert st == _lib.ERR_TOO_LARGE
    assert b"scratch" in lib.qtip_status_string(st)
