"""CPU checks of the identities the fused kernels are built on, against the oracle's Hadamard transform.

They run no kernel: they pin the index arithmetic (which thread owns which element after the register
transform, how a transform over n_heads x 128 splits per head, in which order the factor product and the
Walsh-Hadamard passes may run) that the CUDA code relies on.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle"))
import qtip_oracle as O  # noqa: E402


@pytest.mark.parametrize("E", [4, 8, 16])
def test_register_transform_ownership(E):
    """fwht_regs (qtip_b200/csrc/fwht.cuh): butterflies over the in-thread index bits and the five lane bits, a
    transpose that swaps warp and lane, butterflies over the lane bits again.  In: thread (w, l) holds elements
    (w*32 + l)*E + r.  Out: thread (w, l) holds elements (l*32 + w)*E + r of the transform - and applying the
    same procedure to data held in the second ownership returns it in the first."""
    n = 1024 * E
    rng = np.random.default_rng(E)
    x = rng.standard_normal(n)
    want = O.fwht(x)

    def procedure(held):                       # held[w, l, r]
        v = held.copy()
        v = O.fwht(v)                          # r bits (last axis)
        v = np.moveaxis(O.fwht(np.moveaxis(v, 1, 2)), 2, 1)   # lane bits
        v = np.transpose(v, (1, 0, 2))         # thread (w, l) now holds what thread (l, w) held
        v = np.moveaxis(O.fwht(np.moveaxis(v, 1, 2)), 2, 1)   # lane bits again (the former warp bits)
        return v

    a_in = x.reshape(32, 32, E)                # ownership A: [w][l][r] = element (w*32 + l)*E + r
    out = procedure(a_in)
    got = np.empty(n)
    w, l, r = np.meshgrid(np.arange(32), np.arange(32), np.arange(E), indexing="ij")
    got[((l * 32 + w) * E + r).ravel()] = out.ravel()          # ownership B
    assert np.allclose(got, want, rtol=0, atol=1e-9 * n)

    b_in = np.empty((32, 32, E))
    b_in[w, l, r] = x[(l * 32 + w) * E + r]    # the same vector held in ownership B
    out2 = procedure(b_in)                     # comes back in ownership A
    assert np.allclose(out2.reshape(n), want, rtol=0, atol=1e-9 * n)


@pytest.mark.parametrize("heads", [4, 8, 32, 128])
def test_transform_factors_over_heads(heads):
    """attn_decode_fused_kernel (qtip_b200/csrc/decode_aux.cu): the Walsh-Hadamard transform over heads x 128 values
    restricted to head h is the 128-point transform of z[d] = sum_h2 (-1)^popcount(h & h2) * y[h2*128 + d]."""
    rng = np.random.default_rng(heads)
    y = rng.standard_normal(heads * 128)
    want = O.fwht(y).reshape(heads, 128)
    yh = y.reshape(heads, 128)
    for h in (0, 1, heads // 2 + 1, heads - 1):
        signs = np.array([-1.0 if bin(h & h2).count("1") & 1 else 1.0 for h2 in range(heads)])
        z = (signs[:, None] * yh).sum(0)
        assert np.allclose(O.fwht(z), want[h], rtol=0, atol=1e-9 * heads * 128)


def test_factor_product_commutes_with_walsh_passes():
    """rht_kernel and mlp_mid_kernel multiply by the +-1 factor FIRST and transform only their own rows afterwards;
    mlp_mid_kernel's second product also runs before the second Walsh-Hadamard pass.  Both orders equal the oracle's
    (Walsh-Hadamard over the rows, then the factor)."""
    n, k = 11008, 172
    rng = np.random.default_rng(7)
    hadK = np.sign(rng.standard_normal((k, k)))          # any +-1 matrix: the identity is about ordering
    x = rng.standard_normal(n)
    for transpose in (False, True):
        want = O.hadamard(x, hadK, transpose=transpose)
        hk = hadK.T if transpose else hadK
        first = hk @ x.reshape(k, n // k)                 # factor on the untransformed values
        got = O.fwht(first).reshape(n) / np.sqrt(n)       # then the Walsh-Hadamard pass over each row
        assert np.allclose(got, want, rtol=0, atol=1e-9 * n)
        rows = slice(44, 66)                              # a CTA's rows only need their own Walsh-Hadamard pass
        assert np.allclose(O.fwht(first[rows]) / np.sqrt(n), want.reshape(k, -1)[rows], rtol=0, atol=1e-9 * n)


def test_head_remainder_split_keeps_fp32_inputs():
    """mlp_mid_kernel feeds fp32 data to fp16 tensor-core operands as head + remainder: the pair reproduces an fp32
    value to about 2^-22 relative (not below 2^-25 absolute, half the spacing of fp16 subnormals), and an fp16 value
    exactly (remainder zero)."""
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(100000) * 7).astype(np.float32)
    hi = x.astype(np.float16)
    lo = (x - hi.astype(np.float32)).astype(np.float16)
    rebuilt = hi.astype(np.float32) + lo.astype(np.float32)
    assert np.all(np.abs(rebuilt - x) <= np.maximum(np.abs(x) * 2.0 ** -21, 2.0 ** -25))
    exact = hi.astype(np.float32)                     # values that are fp16 numbers already
    assert np.all((exact - exact.astype(np.float16).astype(np.float32)).astype(np.float16) == 0)
