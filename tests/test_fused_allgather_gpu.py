"""Fused GEMM + all-gather on two or more GPUs of one box (skipped where fewer are visible).

Every rank computes its column block of C and its kernel's epilogue stores the block into every rank's
full C.  Afterwards each rank's C must equal, bit for bit, the C the same rank computes alone with the
unsharded operator (same kernels, same K order), and both must satisfy the path's tolerance against the
FP64 oracle on sampled points.
"""
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


def _worker(rank, world, port, shape, kernel, multicast, ret):
    """One rank.  Nothing in here asserts: whatever happens -- a wrong result, a non-zero status word, an exception --
    is recorded in `ret[rank]` and the rank still takes part in the collective `SharedC.close()` and in the process
    group's shutdown, so that no rank leaves while a peer still maps its C (or while its memory is bound to the
    NVSwitch multicast object) and no peer is left waiting in a barrier.  The parent judges `ret` after the joins."""
    import datetime
    import traceback
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    timeout = datetime.timedelta(seconds=120)
    if multicast:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=timeout)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timeout)
    shared = None
    result = {"error": None}
    try:
        from __graft_entry__ import load_package
        from oracle import fp8_oracle as fo
        pkg = load_package()
        g, sh_mod = pkg.gemm, pkg.shard
        m, k, n = shape
        dev = torch.device("cuda", rank)
        a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=dev)
        b = torch.empty((n, k), dtype=torch.float8_e4m3fn, device=dev)
        g.fill_normal(a, 1.0, 31)                      # replicated operands: same seeds on every rank
        g.fill_normal(b, 1.0, 32)
        try:
            shared = sh_mod.SharedC(m, n, dev, multicast=multicast)
        except RuntimeError as e:
            if multicast and "multicast" in str(e):
                result["skip"] = "no-multicast"
            else:
                raise
        if shared is not None:
            shared.own.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            sh = sh_mod.column_shard(n, rank, world)
            for _ in range(2):                             # twice: the second run overwrites a complete matrix
                sh_mod.gemm_allgather(a, b[sh.n_begin:sh.n_end], shared, sh, n, kernel=kernel)
                torch.cuda.synchronize()
                dist.barrier()
            result["status"] = int(g.device_status())
            alone = torch.empty((m, n), dtype=torch.float32, device=dev)
            g.gemm_ex(a, b, alone, kernel=kernel)
            torch.cuda.synchronize()
            result["equal"] = bool(torch.equal(shared.own, alone))
            rng = np.random.default_rng(rank)
            ms, ns = rng.integers(0, m, 512), rng.integers(0, n, 512)
            C64, S = fo.gemm_f64_points(a.view(torch.uint8).cpu().numpy(), 0, b.view(torch.uint8).cpu().numpy(), 0, ms, ns)
            got = shared.own[torch.from_numpy(ms).to(dev), torch.from_numpy(ns).to(dev)].cpu().numpy()
            bad, worst, _ = fo.check_tolerance(got, C64, S)
            result["bad"], result["worst"] = int(bad), float(worst)
    except Exception:                                  # recorded, not raised: the rank must reach the collective close
        result["error"] = traceback.format_exc()
    finally:
        ret[rank] = result
        try:
            torch.cuda.synchronize()
            if shared is not None:
                shared.close()                         # collective: every rank comes here, failed or not
        except Exception:
            result["error"] = (result["error"] or "") + traceback.format_exc()
            ret[rank] = result
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("multicast", [False, True], ids=["peer-stores", "multimem"])
@pytest.mark.parametrize("shape,kernel", [((1024, 512, 2048), 3), ((2048, 1024, 4096), 5), ((300, 272, 1024), 0)])
def test_fused_allgather_matches_unsharded(shape, kernel, multicast):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, shape, kernel, multicast, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(600)                                # the ranks end by themselves (process-group timeout 120 s)
        results = {r: dict(ret[r]) if r in ret else None for r in range(world)}
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert all(results[r] is not None for r in range(world))
        if any(results[r].get("skip") == "no-multicast" for r in range(world)):
            pytest.skip("no NVLink multicast support on this system")
        for r in range(world):
            res = results[r]
            assert res["error"] is None, f"rank {r}:\n{res['error']}"
            assert res["status"] == 0, f"rank {r}: device status word {res['status']}"
            assert res["equal"], f"rank {r}: gathered C differs from the unsharded result"
            assert res["bad"] == 0 and res["worst"] <= 1.0
