"""CPU restatement (numpy) of the QTIP quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared with.  It is imported by the
tests, by the smoke check and by the benchmark's CPU-baseline leg; the product
package never imports it and has no CPU fallback.

Every function cites the upstream file (path inside the QTIP project) and lines
whose arithmetic it restates.  Parity of this restatement is pinned two ways:
  * oracle/check_against_reference.py runs it against the upstream torch code
    (decode_compressed, unpack_trellis + get_hatW, matmul_hadU, BitshiftLinear.forward)
    on a machine that has the upstream tree, and
  * tests/golden/*.npz hold outputs of that upstream code for seeded inputs
    (generator: tests/golden/make_golden.py); tests/test_oracle.py replays them.

Conventions: K = bits per weight, V = weights per trellis state, L = 16 state bits,
m = out_features, n = in_features, decoded matrix W is (m, n) and y = x @ W.T.
fp16 values travel as numpy float16 (bit patterns via .view(np.uint16)).
"""
import numpy as np

L_BITS = 16
CODE_HYB, CODE_3INST, CODE_1MAD = 0, 1, 2
CODE_NAMES = {"quantlut_sym": CODE_HYB, "hyb": CODE_HYB, "3inst": CODE_3INST, "1mad": CODE_1MAD}


# ----------------------------------------------------------------------------------------------
# state -> weight(s)
# ----------------------------------------------------------------------------------------------
def hyb_hash(s):
    """h = s*(s+1) mod 2^16   (lib/codebook/bitshift.py:72-80, qtip-kernels/src/inference.cu:349)."""
    s = np.asarray(s).astype(np.uint32)
    return (s * (s + np.uint32(1))) & np.uint32(0xFFFF)


def hyb_expand_lut(tlut):
    """512x2 fp16 tunable LUT -> 65536x2 fp16 table indexed by the raw state.

    quantlut_sym (lib/codebook/bitshift.py:72-80): entry (h>>6)&511, first element negated
    when bit 15 of h is set.  The negation is a multiply by -1, i.e. a sign-bit flip
    (it turns +0 into -0), which is what the CUDA kernel's XOR does (inference.cu:358-359).
    """
    tl = np.ascontiguousarray(tlut, dtype=np.float16).reshape(512, 2).view(np.uint16)
    h = hyb_hash(np.arange(1 << L_BITS))
    out = tl[(h >> 6) & 511].copy()
    out[:, 0] ^= ((h >> 15) & 1).astype(np.uint16) << 15
    return out.view(np.float16)


def decode_3inst_table():
    """All 65536 3INST weights as fp16 (lib/codebook/bitshift.py:43-60)."""
    s = np.arange(1 << L_BITS, dtype=np.uint64)
    x = (s * np.uint64(89226354) + np.uint64(64248484)) & np.uint64(0xFFFFFFFF)
    mask = np.uint64(0x8FFF8FFF)
    r = ((x & mask) ^ np.uint64(996162400)).astype(np.uint32)
    top = (r >> 16).astype(np.uint16).view(np.float16)
    bot = (r & 0xFFFF).astype(np.uint16).view(np.float16)
    return (top + bot).astype(np.float16)  # the add is performed in fp16


def decode_1mad_table():
    """All 65536 1MAD weights as fp32 (lib/codebook/bitshift.py:17-26)."""
    s = np.arange(1 << L_BITS, dtype=np.uint64)
    x = (s * np.uint64(34038481) + np.uint64(76625530)) & np.uint64(0xFFFFFFFF)
    y = (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + ((x >> 24) & 255)
    y = y.astype(np.int64) - 510
    return (y.astype(np.float32) / np.float32(147.800537109375)).astype(np.float32)


def state_table(code, tlut=None):
    """(65536, V) fp16 table for a code; 1MAD is rounded fp32->fp16 once (round-to-nearest-even)."""
    if code == CODE_HYB:
        return hyb_expand_lut(tlut)
    if code == CODE_3INST:
        return decode_3inst_table().reshape(-1, 1)
    if code == CODE_1MAD:
        return decode_1mad_table().astype(np.float16).reshape(-1, 1)
    raise ValueError(code)


# ----------------------------------------------------------------------------------------------
# packed trellis -> states
# ----------------------------------------------------------------------------------------------
def states_kernel_layout(codes, m, n, K):
    """Kernel-layout packed codes -> states [m/32][n/32][lane 32][ks 2][ms 2][q 4].

    Layout written by lib/algo/finetune.py:196-201 and undone by
    lib/utils/kernel_decompress.py:19-24; consumed by inference.cu:212-222 / load_reg_cs :94-166.
    Bytes are [m/32][n/32][lane][k-subtile][m-subtile][K bytes]; the K bytes are the lane's slice
    of the tile's big-endian bit stream, byte-reversed, so a little-endian integer read yields the
    slice with its first bit as MSB.  The 16 wrap-around bits come from lane+1 (lane 31 -> lane 0).
    """
    assert m % 32 == 0 and n % 32 == 0 and K in (2, 3, 4)
    b = np.ascontiguousarray(codes).reshape(-1).view(np.uint8)
    assert b.size == m * n * K // 8
    b = b.reshape(m // 32, n // 32, 32, 2, 2, K)
    sl = np.zeros(b.shape[:-1], dtype=np.uint64)
    for i in range(K):
        sl |= b[..., i].astype(np.uint64) << np.uint64(8 * i)
    nxt = np.roll(sl, -1, axis=2)
    win = (sl << np.uint64(8 * K)) | nxt
    st = [(win >> np.uint64(16 * K - 16 - 2 * K * q)) & np.uint64(0xFFFF) for q in range(4)]
    return np.stack(st, axis=-1).astype(np.uint16)


def decode_kernel_layout(codes, m, n, K, tlut):
    """HYB (L=16, V=2, Q=9) kernel-layout decode -> (m, n) fp16.

    Same result as decode_compressed (lib/utils/kernel_decompress.py:4-55): lane l=4a+b, state
    q=2c+d gives the two weights at row 32M+16ms+8d+a, columns 32N+16ks+8c+2b+{0,1}
    (the mma.m16n8k16 A-fragment order, lib/algo/ldlq.py:10-13).
    """
    st = states_kernel_layout(codes, m, n, K)  # [M][N][l][ks][ms][q]
    w = hyb_expand_lut(tlut).view(np.uint16)[st]  # [...][e]
    M, N = m // 32, n // 32
    w = w.reshape(M, N, 8, 4, 2, 2, 2, 2, 2)  # M N a b ks ms c d e
    w = w.transpose(0, 5, 7, 2, 1, 4, 6, 3, 8)  # M ms d a N ks c b e
    return np.ascontiguousarray(w).reshape(m, n).view(np.float16)


def states_plain_layout(codes, m, n, K, V):
    """Plain-layout packed codes -> states [tiles][256/V]   (tiles row-major over (m/16, n/16)).

    unpack_trellis (lib/codebook/bitshift.py:329-353): each tile's 16*K words form a 256*K-bit
    stream, MSB first; state i is the 16-bit window starting at bit i*K*V, wrapping circularly
    (pack_trellis :294-317 drops the last L-KV bits because they repeat the first ones).
    """
    assert m % 16 == 0 and n % 16 == 0
    tiles = (m // 16) * (n // 16)
    wds = np.ascontiguousarray(codes).reshape(-1).view(np.uint16).reshape(tiles, 16 * K)
    bits = ((wds[:, :, None] >> np.arange(15, -1, -1, dtype=np.uint16)) & 1).astype(np.uint8)
    bits = bits.reshape(tiles, 256 * K)
    ext = np.concatenate([bits, bits[:, :L_BITS]], axis=1)
    T = 256 // V
    st = np.zeros((tiles, T), dtype=np.uint32)
    pos = np.arange(T) * (K * V)
    for j in range(L_BITS):
        st = (st << 1) | ext[:, pos + j]
    return st.astype(np.uint16)


def recons_table(code, tlut32=None):
    """Upstream's recons_state as the quantizer holds it: (V, 65536) fp32.  HYB: quantlut_sym on the fp32 table
    (lib/codebook/bitshift.py:72-80); 3INST: the fp16-exact values as fp32 (:43-60); 1MAD: the fp32 values (:17-26)."""
    if code == CODE_HYB:
        s = np.arange(1 << L_BITS, dtype=np.uint64)
        h = (s * (s + 1)) & 0xFFFF
        t = np.asarray(tlut32, dtype=np.float32).reshape(512, 2)[(h >> 6) & 511].copy()
        t[:, 0] *= (1 - 2 * ((h >> 15) & 1).astype(np.float32))
        return np.ascontiguousarray(t.T)
    if code == CODE_3INST:
        return decode_3inst_table().astype(np.float32).reshape(1, -1)
    return decode_1mad_table().astype(np.float32).reshape(1, -1)


def pack_trellis(states, K, V):
    """Trellis states [tiles][256/V] -> plain-layout words [tiles][16*K] uint16.

    pack_trellis (lib/codebook/bitshift.py:294-327): the bitstream of a tile is state 0's 16 bits (MSB first)
    followed by the low K*V bits of every later state; the last 16 - K*V bits are dropped (a tail-biting walk
    repeats the first bits there) and the stream is cut into 16-bit words, MSB first.  Raises ValueError where
    upstream asserts (:306-309): consecutive states must overlap by 16 - K*V bits."""
    st = np.asarray(states).astype(np.int64)
    tiles, T = st.shape
    kv = K * V
    assert T * V == 256 and (T * kv) % 16 == 0
    if not np.array_equal(st[:, :-1] & ((1 << (L_BITS - kv)) - 1), st[:, 1:] >> kv):
        raise ValueError("consecutive states do not overlap")
    bits = np.zeros((tiles, T * kv + L_BITS - kv), dtype=np.uint8)
    bits[:, :L_BITS] = (st[:, :1] >> np.arange(L_BITS - 1, -1, -1)) & 1
    low = (st[:, 1:, None] >> np.arange(kv - 1, -1, -1)) & 1              # tiles, T-1, kv
    bits[:, L_BITS:] = low.reshape(tiles, -1)
    bits = bits[:, :T * kv].reshape(tiles, -1, 16).astype(np.uint32)
    return (bits << np.arange(15, -1, -1, dtype=np.uint32)).sum(axis=2).astype(np.uint16)


def decode_plain_layout(codes, m, n, K, V, code, tlut=None):
    """Plain-layout decode -> (m, n) fp16.

    get_hatW (lib/codebook/bitshift.py:378-381): decoded sequence element t = i*V + v of a tile is
    tile element (t // 16, t % 16).
    """
    st = states_plain_layout(codes, m, n, K, V)
    tab = state_table(code, tlut)
    assert tab.shape[1] == V
    w = tab.view(np.uint16)[st]  # tiles, T, V
    w = w.reshape(m // 16, n // 16, 16, 16).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(w).reshape(m, n).view(np.float16)


# tile element <-> sequence position of the kernel layout (lib/algo/ldlq.py:10-13):
# sequence position j = a*32 + b*8 + c*4 + d*2 + e  holds tile element (8d + a, 8c + 2b + e).
def kernel_sequence_permutation():
    j = np.arange(256)
    a, b, c, d, e = j >> 5, (j >> 3) & 3, (j >> 2) & 1, (j >> 1) & 1, j & 1
    return (8 * d + a) * 16 + (8 * c + 2 * b + e)  # element index (row*16+col) at sequence pos j


def plain_words_to_kernel_layout(words, m, n, K):
    """Re-order plain-layout words (tiles, 16K) into the kernel byte layout (same shape).

    This is only the byte shuffle of lib/algo/finetune.py:196-201.  It does not change which
    sequence position a state has: a plain-layout tile whose sequence element j is meant to be
    tile element kernel_sequence_permutation()[j] becomes a valid kernel-layout buffer.
    """
    w = np.ascontiguousarray(words).view(np.uint16).reshape(m // 32, 2, n // 32, 2, 16 * K)
    # big-endian bytes of the stream: [M][ms][N][ks][32 lanes][K bytes]
    be = np.stack([(w >> 8).astype(np.uint8), (w & 0xFF).astype(np.uint8)], axis=-1)
    be = be.reshape(m // 32, 2, n // 32, 2, 32, K)
    out = be.transpose(0, 2, 4, 3, 1, 5)[..., ::-1]  # M N lane ks ms, bytes reversed
    return np.ascontiguousarray(out).reshape(-1).view(np.uint16).reshape(-1, 16 * K)


def kernel_layout_to_plain_words(codes, m, n, K):
    """Inverse of plain_words_to_kernel_layout (lib/utils/kernel_decompress.py:19-24)."""
    b = np.ascontiguousarray(codes).reshape(-1).view(np.uint8).reshape(m // 32, n // 32, 32, 2, 2, K)
    be = b[..., ::-1].transpose(0, 4, 1, 3, 2, 5)  # M ms N ks lane byte(big-endian order)
    be = np.ascontiguousarray(be).reshape(-1, 2)
    w = (be[:, 0].astype(np.uint16) << 8) | be[:, 1].astype(np.uint16)
    return w.reshape(-1, 16 * K)


# ----------------------------------------------------------------------------------------------
# Hadamard
# ----------------------------------------------------------------------------------------------
HAD_FACTORS = (172, 156, 140, 124, 116, 108, 60, 52, 36, 28, 20, 12)


def had_factor(n):
    """First-match factor table of get_hadK (lib/utils/matmul_had.py:9-63): n = K * 2^p."""
    for k in HAD_FACTORS:
        if n % k == 0:
            q = n // k
            assert q & (q - 1) == 0, f"{n} / {k} is not a power of two"
            return k
    assert n & (n - 1) == 0 and n > 0, f"{n} has no supported Hadamard factorisation"
    return 1


def fwht(x):
    """Unnormalised Sylvester-ordered Walsh-Hadamard transform over the last dim (power of two)."""
    n = x.shape[-1]
    y = np.array(x, dtype=np.float64).reshape(-1, n)
    h = 1
    while h < n:
        y = y.reshape(-1, n // (2 * h), 2, h)
        y = np.stack((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), axis=2).reshape(-1, n)
        h *= 2
    return y.reshape(x.shape)


def hadamard(x, hadK=None, transpose=False):
    """Orthonormal Hadamard over the last dim, the transform of matmul_hadU_cuda
    (lib/utils/matmul_had.py:105-119): n = K*2^p is viewed (K, n/K), a Walsh-Hadamard transform
    runs over the last dim, hadK (K x K, +-1; transposed for the input side) multiplies from the
    left, everything is scaled by n^-1/2.  float64 arithmetic.
    """
    n = x.shape[-1]
    k = had_factor(n)
    if k == 1:
        return fwht(x) / np.sqrt(n)
    assert hadK is not None and hadK.shape == (k, k)
    hk = np.asarray(hadK, dtype=np.float64)
    if transpose:
        hk = hk.T
    y = fwht(np.asarray(x, dtype=np.float64).reshape(-1, k, n // k))
    y = hk @ y
    return y.reshape(x.shape) / np.sqrt(n)


# ----------------------------------------------------------------------------------------------
# layer forward
# ----------------------------------------------------------------------------------------------
def matvec_fp16(W, x):
    """y = x @ W.T with fp16 operands and wide accumulation (the op of lib/codebook/__init__.py:85-92:
    x is rounded to fp16, products accumulate in fp32 in the kernel; float64 here)."""
    xh = np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float64)
    return xh @ np.asarray(W).astype(np.float64).T


def layer_forward(x, W, SU, SV, had_left=None, had_right=None, rcp=0, tp=1, scale=32.0):
    """BitshiftLinear.forward (lib/codebook/bitshift.py:415-472) for a decoded fp16 matrix W (m, n).

    x (bs, n) -> y (bs, m), float64 internally except the fp16 rounding of the activation at the
    matvec boundary.  rcp=1: input-side transform on each of `tp` chunks of n; rcp=2: output-side
    transform on each of `tp` chunks of m (:437-441, :465-469).
    """
    m, n = W.shape
    x = np.asarray(x, dtype=np.float64).reshape(-1, n) * np.asarray(SU, dtype=np.float64)
    bs = x.shape[0]
    if rcp == 1:
        x = hadamard(x.reshape(-1, n // tp), had_left, transpose=True).reshape(bs, n) / scale
    else:
        x = hadamard(x, had_left, transpose=True) / scale
    y = matvec_fp16(W, x)
    if rcp == 2:
        y = hadamard(y.reshape(-1, m // tp), had_right).reshape(bs, m)
    else:
        y = hadamard(y, had_right)
    return y * (np.asarray(SV, dtype=np.float64) * scale)
