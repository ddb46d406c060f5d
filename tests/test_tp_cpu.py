"""CPU, world_size 2 over gloo: the tensor-parallel split of a QTIP layer reproduces the unsharded layer.

Each rank shards the layer with qtip_b200.tp, evaluates its shard with the C oracle, and the ranks combine
through torch.distributed (all_reduce for the row-parallel layer, all_gather for the column-parallel one)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "oracle")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import c_oracle as C
    import qtip_oracle as O
    from qtip_b200 import ops, synth, tp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, K = 256, 1664, 2          # 1664 = 52 * 32: chunk 832 = 52 * 16 keeps the factor 52
        lay = synth.make_layer(m, n, K, seed=5)
        x = lay["x"].astype(np.float32)
        SU, SV = lay["SU"].astype(np.float32), lay["SV"] * (0.5 + np.arange(m) / m).astype(np.float32)
        had = lambda d: (None if ops.get_hadK(d)[0] is None else ops.get_hadK(d)[0].numpy())  # noqa: E731
        # ---- row-parallel (rcp = 1): split n, all-reduce the partial outputs
        full = C.layer_forward(x, lay["codes"], m, n, K, lay["tlut"], SU, SV, had(n // world), had(m), rcp=1, tp=world)
        t_r, su_r, sv_r, n_r = tp.shard_row_parallel(lay["codes"], SU, SV, m, n, K, rank, world)
        xs = (x[:, rank * n_r:(rank + 1) * n_r] * su_r)
        xh = C.float_to_half(O.hadamard(xs, had(n_r), transpose=True).astype(np.float32) / 32)
        part = torch.from_numpy(C.matvec_kernel(t_r, m, n_r, K, lay["tlut"], xh))
        dist.all_reduce(part)
        y = O.hadamard(part.numpy(), had(m)) * sv_r * 32
        err_row = float(np.linalg.norm(y - full) / np.linalg.norm(full))
        # ---- column-parallel (rcp = 2): split m, gather the chunks
        m2, n2 = 1664, 256
        lay2 = synth.make_layer(m2, n2, K, seed=6)
        x2, SU2, SV2 = lay2["x"].astype(np.float32), lay2["SU"].astype(np.float32), lay2["SV"]
        full2 = C.layer_forward(x2, lay2["codes"], m2, n2, K, lay2["tlut"], SU2, SV2, had(n2), had(m2 // world), rcp=2, tp=world)
        t_c, su_c, sv_c, m_r = tp.shard_column_parallel(lay2["codes"], SU2, SV2, m2, n2, K, rank, world)
        xh2 = C.float_to_half(O.hadamard(x2 * su_c, had(n2), transpose=True).astype(np.float32) / 32)
        yc = O.hadamard(C.matvec_kernel(np.ascontiguousarray(t_c), m_r, n2, K, lay2["tlut"], xh2), had(m_r)) * sv_c * 32
        parts = [torch.zeros(1, m_r, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(yc))
        y2 = torch.cat(parts, dim=1).numpy()
        err_col = float(np.linalg.norm(y2 - full2) / np.linalg.norm(full2))
        ret[rank] = (err_row, err_col)
    finally:
        dist.destroy_process_group()


def test_tp_shards_reproduce_unsharded_layer_over_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err_row, err_col = ret[rank]
        assert err_row < 1e-5, f"row-parallel rank {rank}: {err_row}"
        assert err_col < 1e-5, f"column-parallel rank {rank}: {err_col}"


def test_shard_shapes():
    sys.path.insert(0, ROOT)
    from qtip_b200 import tp
    m, n, K = 256, 512, 3
    tr = torch.arange(m * n * K // 16, dtype=torch.int32).to(torch.int16).reshape(-1, 16 * K)
    SU, SV = torch.ones(n), torch.ones(m)
    for world in (2, 4, 8):
        rows = [tp.shard_column_parallel(tr, SU, SV, m, n, K, r, world) for r in range(world)]
        assert torch.equal(torch.cat([t for t, *_ in rows]), tr)            # contiguous slabs, in order
        assert all(sv.numel() == m // world and su.numel() == n for _, su, sv, _ in rows)
        cols = [tp.shard_row_parallel(tr, SU, SV, m, n, K, r, world) for r in range(world)]
        assert all(t.shape == (m * (n // world) // 256, 16 * K) and su.numel() == n // world for t, su, _, _ in cols)
        back = torch.cat([t.reshape(m // 32, -1, 64 * K) for t, *_ in cols], dim=1).reshape(-1, 16 * K)
        assert torch.equal(back, tr)
    with pytest.raises(AssertionError):
        tp.shard_column_parallel(tr, SU, SV, m, n, K, 0, 16)


def test_peer_address_layout():
    """Every (slot, source, destination) triple names one vector, producers and consumers agree on it, and the
    vectors of one GPU tile its buffer without overlap."""
    from qtip_b200 import tp
    world, width = 4, 4096
    base = [0x7000_0000_0000 + g * 0x1000_0000 for g in range(world)]
    tables = [tp.peer_addresses(base, width, r) for r in range(world)]
    for slot in (0, 1):
        for src in range(world):
            for dst in range(world):
                # where src writes on dst == where dst reads src's vector
                assert tables[src][0][slot][dst] == tables[dst][1][slot][src]
    for g in range(world):
        offs = sorted(a - base[g] for slot in (0, 1) for a in tables[g][1][slot])
        assert offs == [i * width * 8 for i in range(2 * world)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_stamped_vector_protocol_never_loses_a_round(world):
    """Model of the tensor-parallel protocol of qtip_linear_fused (signal_* / peer_* fields) with ranks that advance
    in arbitrary interleavings: per layer a rank runs producer(slot 0), consumer(slot 0), producer(slot 1) and, in
    the next layer, consumer(slot 1); the last layer's slot-1 result goes through an ordinary all-reduce (a point
    where all ranks meet).  A producer stamps its vector on every rank with its sequence counter + 1 and then
    advances the counter; a consumer needs every rank's vector to carry exactly its own counter value.  The check:
    whenever a consumer can run, no vector it needs has already been overwritten by a later round (the stamps are
    equal, never ahead), for every schedule tried."""
    import random
    layers, tokens = 3, 3
    program = []                                   # one rank's launches of one token
    for li in range(layers):
        if li > 0:
            program.append(("consume", 1))
        program.append(("produce", 0))
        program.append(("consume", 0))
        program.append(("produce", 1) if li != layers - 1 else ("allreduce", None))
    rng = random.Random(world)
    for trial in range(200):
        seq = [[0, 0] for _ in range(world)]                                   # per rank, per slot
        stamp = [[[0] * world for _ in range(2)] for _ in range(world)]        # stamp[holder][slot][source]
        pc = [0] * world
        total = len(program) * tokens
        at_allreduce = set()
        while any(p < total for p in pc):
            runnable = []
            for r in range(world):
                if pc[r] >= total:
                    continue
                op, slot = program[pc[r] % len(program)]
                if op == "consume":
                    have = stamp[r][slot]
                    assert all(s <= seq[r][slot] for s in have), "a vector was overwritten before it was read"
                    if all(s == seq[r][slot] for s in have):
                        runnable.append(r)
                elif op == "allreduce":
                    at_allreduce.add(r)
                    if len(at_allreduce) == world:
                        runnable.append(r)
                else:
                    runnable.append(r)
            assert runnable, "deadlock"
            r = rng.choice(runnable)
            op, slot = program[pc[r] % len(program)]
            if op == "produce":
                s = seq[r][slot] + 1
                for holder in range(world):
                    stamp[holder][slot][r] = s
                seq[r][slot] = s
            elif op == "allreduce":
                for q in range(world):                # every rank leaves the collective together
                    assert program[pc[q] % len(program)][0] == "allreduce"
                    pc[q] += 1
                at_allreduce.clear()
                continue
            pc[r] += 1
