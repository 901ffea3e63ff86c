"""The C ABI's multi-GPU plan (b200fp8_multi_*): one process, one host thread per shard inside the library.

The plan is exercised with every visible GPU and -- because a device may carry several shards -- also with four
shards on GPU 0 alone, so the sharding, the in-place column blocks and the fused all-gather through (here: same-device)
pointers are covered on a one-GPU box too.  The assembled C must equal the unsharded operator's result bit for bit
(same kernels, same K order per element) and hold the path's tolerance against the FP64 oracle."""
import numpy as np
import pytest
import torch

from __graft_entry__ import load_package

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available()
    p = load_package()
    p._cabi.lib()
    torch.cuda.set_device(0)
    return p


def _device_lists():
    n = torch.cuda.device_count()
    lists = [[0], [0, 0, 0, 0], [0, 0, 0]]
    if n >= 2:
        lists.append(list(range(min(n, 8))))
    return lists


@pytest.mark.parametrize("gather", [False, True], ids=["blocks", "fused-gather"])
@pytest.mark.parametrize("devices", _device_lists(), ids=lambda d: "dev" + "".join(map(str, d)))
@pytest.mark.parametrize("shape,kernel", [((512, 512, 2048), 0), ((300, 272, 1284), 3), ((1024, 1024, 4096), 5)])
def test_plan_matches_unsharded_operator(pkg, oracle, devices, gather, shape, kernel):
    g, sh = pkg.gemm, pkg.shard
    m, k, n = shape
    f8 = torch.float8_e4m3fn
    a = torch.empty((m, k), dtype=f8, device="cuda")
    b = torch.empty((n, k), dtype=f8, device="cuda")
    g.fill_normal(a, 1.0, 71)
    g.fill_normal(b, 1.0, 72)
    want = torch.empty((m, n), dtype=torch.float32, device="cuda")
    g.gemm_ex(a, b, want, kernel=kernel)
    torch.cuda.synchronize()
    plan = sh.MultiGpuPlan(devices, m, k, n, gather=gather)
    try:
        plan.upload(a.cpu(), b.cpu())
        ms = plan.run(2, kernel=kernel)
        assert ms > 0
        for from_shard in ({0, len(devices) - 1} if gather else {0}):
            got = torch.full((m, n), float("nan"), dtype=torch.float32)
            plan.download(got, from_shard)
            assert torch.equal(got, want.cpu()), f"shard {from_shard}"
        # shard geometry: contiguous cover of the N columns in units of 256
        edges = [plan.shard(i)[1:3] for i in range(len(devices))]
        assert edges[0][0] == 0 and edges[-1][1] == n and all(edges[i][1] == edges[i + 1][0] for i in range(len(edges) - 1))
    finally:
        plan.close()
    for dev in set(devices):
        with torch.cuda.device(dev):
            assert g.device_status() == 0
    C64, S = oracle.gemm_f64(a.view(torch.uint8).cpu().numpy()[:64], 0, b.view(torch.uint8).cpu().numpy(), 0)
    bad, worst, _ = oracle.check_tolerance(got[:64].numpy(), C64, S)
    assert bad == 0 and worst <= 1.0


def test_plan_generates_the_same_operands_as_the_single_device_generator(pkg):
    g, sh = pkg.gemm, pkg.shard
    m, k, n = 256, 256, 1024
    devices = list(range(min(torch.cuda.device_count(), 4))) if torch.cuda.device_count() >= 2 else [0, 0]
    plan = sh.MultiGpuPlan(devices, m, k, n)
    try:
        plan.fill_normal(1.0, 5, 1.0, 6)
        plan.run(1)
        got = plan.download(torch.empty((m, n), dtype=torch.float32))
    finally:
        plan.close()
    a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device="cuda")
    b = torch.empty((n, k), dtype=torch.float8_e4m3fn, device="cuda")
    g.fill_normal(a, 1.0, 5)
    g.fill_normal(b, 1.0, 6)
    want = g.gemm_ex(a, b)
    torch.cuda.synchronize()
    assert torch.equal(got, want.cpu())


def test_plan_rejects_bad_arguments(pkg):
    import ctypes
    lib = pkg._cabi.lib()
    plan = ctypes.c_void_p()
    one = (ctypes.c_int * 1)(0)
    assert lib.b200fp8_multi_create(0, one, 128, 128, 128, 0, 0, 0, ctypes.byref(plan)) == 1
    assert lib.b200fp8_multi_create(1, one, 128, 72, 128, 0, 0, 0, ctypes.byref(plan)) == 1          # K % 16
    assert lib.b200fp8_multi_create(1, one, 128, 128, 130, 0, 0, 1, ctypes.byref(plan)) == 1         # gather needs N % 4 == 0
    bad = (ctypes.c_int * 1)(99)
    assert lib.b200fp8_multi_create(1, bad, 128, 128, 128, 0, 0, 0, ctypes.byref(plan)) != 0
    assert lib.b200fp8_multi_run(None, 1, None, None) == 1
