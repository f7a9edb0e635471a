"""Host-side logic of the multi-GPU path, on CPU ranks (gloo, world_size 2 and 3).

Each rank takes its row block by the reference's partition rule, computes it (with the CPU oracle
standing in for the device operator), and the blocks are gathered: the result must equal the
single-rank result bit for bit, and B must arrive by broadcast from rank 0.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spoc_b200.sharding import gather_counts, partition, row_block


def test_partition_rule():
    assert partition(10, 3) == [(0, 4), (4, 3), (7, 3)]      # base + (i < rem)
    assert partition(8, 4) == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert partition(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    assert partition(0, 2) == [(0, 0), (0, 0)]
    assert row_block(65536, 8, 7) == (57344, 8192)
    assert gather_counts(10, 5, 3) == [20, 15, 15]
    with pytest.raises(ValueError):
        partition(4, 0)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, n, k, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tests import oracle_lib as O
        a_full, c_full = O.fill(m * k, 7, 1), O.fill(m * n, 7, 3)
        bias = O.fill(n, 7, 4, kind=1)
        b = torch.from_numpy(O.fill(k * n, 7, 2)) if rank == 0 else torch.zeros(k * n)
        dist.broadcast(b, src=0)                              # B replicated from rank 0
        r0, rows = row_block(m, world, rank)
        a = np.ascontiguousarray(a_full[r0 * k:(r0 + rows) * k])
        c = np.ascontiguousarray(c_full[r0 * n:(r0 + rows) * n])
        d = O.gemm(a, b.numpy(), rows, n, k, 1.5, 0.5, c, bias, 1) if rows else np.zeros((0, n), np.float32)
        counts = gather_counts(m, n, world)
        pad = max(counts)
        mine = torch.zeros(pad)
        mine[:rows * n] = torch.from_numpy(d.ravel())
        parts = [torch.zeros(pad) for _ in range(world)]
        dist.all_gather(parts, mine)                          # row blocks are contiguous in row-major D
        full = torch.cat([p[:cnt] for p, cnt in zip(parts, counts)]).numpy().reshape(m, n)
        if rank == 0:
            want = O.gemm(a_full, b.numpy(), m, n, k, 1.5, 0.5, c_full, bias, 1)
            out_q.put(bool(np.array_equal(full, want)))
        # max-over-ranks timing reduction used by bench.py
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,m", [(2, 64), (3, 50)])
def test_row_sharded_gemm_gathers_to_the_single_rank_result(world, m):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, 40, 24, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True
