"""Tensor-parallel layout of QTIP layers (one process per GPU).

Upstream ships only the *layout* for tensor parallelism (lib/algo/finetune.py:130-171 quantizes with the
Hadamard transform taken per 1/tp chunk of the split side; BitshiftLinear.forward applies it per chunk,
lib/codebook/bitshift.py:437-441, 465-469) and no runtime.  The runtime here:

  column-parallel (q, k, v, gate, up; rcp = 2): rank r owns output rows [r*m/tp, (r+1)*m/tp).  In the kernel
      layout that is one contiguous slab of `trellis`.  Input transform on the full, replicated activation;
      output transform on the local chunk with the local slice of SV.  No communication.
  row-parallel (o, down; rcp = 1): rank r owns input columns [r*n/tp, (r+1)*n/tp); the blocks are re-packed
      into a contiguous (m, n/tp) matrix once at load.  Input transform on the local chunk with the local
      slice of SU; the matvec yields a full-length partial result; ONE all-reduce (sum) of bs*m fp32 values;
      the output transform and SV then run redundantly on every rank.
"""
import numpy as np
import torch


def shard_column_parallel(trellis, SU, SV, m, n, K, rank, tp):
    """Rank's shard of a kernel-layout layer split along out_features.  Returns (trellis_r, SU, SV_r, m_r)."""
    assert m % (32 * tp) == 0, "m/tp must be a multiple of 32"
    m_r = m // tp
    words_per_row_block = (n // 32) * 64 * K            # int16 words of one 32-row block
    flat = trellis.reshape(-1)
    lo = rank * (m_r // 32) * words_per_row_block
    t = flat[lo:lo + (m_r // 32) * words_per_row_block].reshape(-1, 16 * K)
    return t, SU, SV[rank * m_r:(rank + 1) * m_r], m_r


def shard_row_parallel(trellis, SU, SV, m, n, K, rank, tp):
    """Rank's shard of a kernel-layout layer split along in_features (re-packed contiguous).
    Returns (trellis_r, SU_r, SV, n_r)."""
    assert n % (32 * tp) == 0, "n/tp must be a multiple of 32"
    n_r = n // tp
    blocks = trellis.reshape(m // 32, n // 32, 64 * K)   # [row block][column block][words of a 2x2 tile block]
    nb_r = n_r // 32
    t = blocks[:, rank * nb_r:(rank + 1) * nb_r, :]
    t = (t.contiguous() if torch.is_tensor(t) else np.ascontiguousarray(t)).reshape(-1, 16 * K)
    return t, SU[rank * n_r:(rank + 1) * n_r], SV, n_r
