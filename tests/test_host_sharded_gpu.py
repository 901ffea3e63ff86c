"""End to end from host buffers on two or more GPUs (skipped where fewer are visible): `shard.HostShardedGemm`.

Every rank uploads its rows of A and its rows of B, the rows of A go round over NVLink, the operator runs in row blocks
and C comes down block by block.  Each rank's downloaded column block must equal, bit for bit, the same columns of the
unsharded operator's result computed on that rank alone, with and without the per-phase time stamps."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, shape, ret):
    import datetime
    import traceback
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    result = {"error": None}
    try:
        from __graft_entry__ import load_package
        pkg = load_package()
        g, sh_mod = pkg.gemm, pkg.shard
        m, k, n = shape
        f8 = torch.float8_e4m3fn
        a = torch.empty((m, k), dtype=f8, device=dev)
        b = torch.empty((n, k), dtype=f8, device=dev)
        g.fill_normal(a, 1.0, 91)                       # replicated operands: the same seeds on every rank
        g.fill_normal(b, 1.0, 92)
        want = torch.empty((m, n), dtype=torch.float32, device=dev)
        g.gemm_ex(a, b, want)
        torch.cuda.synchronize()
        sh = sh_mod.column_shard(n, rank, world)
        rows = m // world
        ha = a[rank * rows:(rank + 1) * rows].cpu().pin_memory()
        hb = b[sh.n_begin:sh.n_end].cpu().pin_memory()
        hc = torch.full((m, sh.n), float("nan"), dtype=torch.float32).pin_memory()
        runner = sh_mod.HostShardedGemm(m, k, sh, f8, f8, dev)
        runner(ha, hb, hc)
        result["equal"] = bool(torch.equal(hc, want[:, sh.n_begin:sh.n_end].cpu()))
        hc.fill_(float("nan"))
        phases = runner(ha, hb, hc, breakdown=True)
        result["equal_again"] = bool(torch.equal(hc, want[:, sh.n_begin:sh.n_end].cpu()))
        result["phases_ordered"] = bool(phases["upload_a_rows"] <= phases["upload_b_shard"] <= phases["last_c_block_in_host_memory"]
                                        and phases["first_row_block_computed"] <= phases["last_row_block_computed"])
        result["status"] = int(g.device_status())
    except Exception:
        result["error"] = traceback.format_exc()
    finally:
        ret[rank] = result
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:
            pass
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("shape", [(2048, 1024, 4096), (4096, 512, 2048)])
def test_host_sharded_gemm_matches_unsharded_operator(shape):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, shape, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(600)
        results = {r: dict(ret[r]) if r in ret else None for r in range(world)}
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        for r in range(world):
            res = results[r]
            assert res is not None and res["error"] is None, f"rank {r}:\n{res and res['error']}"
            assert res["equal"] and res["equal_again"], f"rank {r}: downloaded block differs from the unsharded operator"
            assert res["phases_ordered"] and res["status"] == 0
