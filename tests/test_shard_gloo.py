"""The N-shard plan with two CPU ranks over gloo: every rank computes its own column block with
the oracle (standing in for the device step), the blocks are all-gathered, and the row-major
re-assembly equals the unsharded result bit for bit."""
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
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, k, n, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load_package
    from oracle import fp8_oracle as fo
    sh = load_package().shard.column_shard(n, rank, world, align=16)
    A = fo.fill_normal(m * k, 0, 1.0, 5).reshape(m, k)                                   # replicated: same seed
    B = fo.fill_normal(sh.n * k, 0, 1.0, 6, index_offset=sh.n_begin * k).reshape(sh.n, k)  # own slab only
    C = torch.from_numpy(fo.gemm_ref_float(A, 0, B, 0))
    sizes = [load_package().shard.column_shard(n, r, world, align=16).n for r in range(world)]
    blocks = [torch.empty((m, s), dtype=torch.float32) for s in sizes]
    dist.all_gather(blocks, C)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)           # the bench's max-over-ranks reduction
    if rank == 0:
        full = load_package().shard.gather_layout_to_row_major(blocks, m).numpy()
        Bfull = fo.fill_normal(n * k, 0, 1.0, 6).reshape(n, k)
        ret["equal"] = bool(np.array_equal(full, fo.gemm_ref_float(A, 0, Bfull, 0)))
        ret["max"] = float(t.item())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_equals_unsharded(world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, 24, 64, 96, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret["equal"] is True and ret["max"] == float(world)
