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

The all-reduce does not have to be a launch of its own: with PeerBuffers the producing matvec stores its partial
result, every value stamped with a sequence number, into memory of every GPU of the node (torch symmetric memory,
NVLink peer stores), and the consuming launch on each GPU polls its own copy until all stamps are current, adds the
partial vectors and goes on with the output transform (qtip_linear_fused: signal_* / peer_* fields).
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


def peer_addresses(base, width, rank):
    """Device addresses of the stamped vectors, from the per-GPU base addresses of the symmetric allocation
    (layout [slot 2][source GPU][width] x 8 bytes).  Returns (signal_y, peer_y), both indexed [slot][gpu]:
    signal_y[slot][p] is where `rank` writes its vector on GPU p, peer_y[slot][p] is GPU p's vector in `rank`'s memory."""
    world = len(base)
    off = lambda slot, src: (slot * world + src) * width * 8   # noqa: E731
    signal_y = [[base[p] + off(slot, rank) for p in range(world)] for slot in (0, 1)]
    peer_y = [[base[rank] + off(slot, p) for p in range(world)] for slot in (0, 1)]
    return signal_y, peer_y


class PeerBuffers:
    """Peer-mapped vectors for the two row-parallel linears of a decoder layer.

    One symmetric allocation per GPU: for each of two slots (0: o_proj, 1: down_proj) one vector of `width` stamped
    values ({fp32 value, uint32 sequence number}, 8 bytes) PER SOURCE GPU.  GPU p's producer launch stores its partial
    result into vector [slot][p] on every GPU, so consumers poll and read local memory only.  Slots alternate, and a
    GPU cannot run more than one producer/consumer round ahead of the slowest GPU (each round needs every GPU's
    values), so a vector is never overwritten while another GPU still reads it.  The sequence counters and the
    time-out status word are ordinary local tensors.
    """
    MAX_PEERS = 8

    def __init__(self, width, rank, world, group, device):
        import os
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads / stores only
        import torch.distributed._symmetric_memory as symm_mem
        assert world <= self.MAX_PEERS
        self.width, self.rank, self.world = width, rank, world
        self.buf = symm_mem.empty(2 * world * width * 2, dtype=torch.int32, device=device)    # stamp 0 everywhere
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name if group is not None else dist.group.WORLD.group_name)
        base = [int(p) for p in self.handle.buffer_ptrs]
        self._signal_y, self._peer_y = peer_addresses(base, width, rank)
        self.max_polls = int(os.environ.get("QTIP_PEER_MAX_POLLS", 1 << 23))   # default ~10 s: ranks may start seconds apart
        self.seq = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                  # nobody stores before every buffer is zeroed

    def signal(self, slot):
        """Descriptor fields of the producer launch (qtip_linear_fused) of slot's partial vector."""
        return dict(signal_y=self._signal_y[slot], signal_seq=self.seq.data_ptr() + 4 * slot)

    def consume(self, slot):
        """Descriptor fields of the consumer launch that sums slot's partial vectors of all GPUs."""
        return dict(peer_y=self._peer_y[slot], peer_seq=self.seq.data_ptr() + 4 * slot, peer_status=self.status.data_ptr(),
                    peer_max_polls=self.max_polls)
