"""Host threads and streams: the reference operator keeps no global state (GEMM/src/gemm.cu:263-277 launches and
returns), so it is trivially thread-safe; the library keeps a per-device context (status word, pacing counters)
behind a mutex and must stay safe when several host threads enqueue on their own streams of one GPU."""
import threading

import pytest
import torch

from __graft_entry__ import load_package

pytestmark = pytest.mark.gpu

SHAPES = [(512, 1024, 768, 3), (300, 512, 520, 1), (64, 2048, 1024, 4), (1024, 384, 1024, 2),
          (2560, 256, 5120, 3), (16, 4096, 512, 4)]


@pytest.fixture(scope="module")
def g():
    assert torch.cuda.is_available()
    pkg = load_package()
    pkg._cabi.lib()
    torch.cuda.set_device(0)
    return pkg.gemm


def test_concurrent_host_threads_on_own_streams_match_sequential_results(g):
    f8 = torch.float8_e4m3fn
    ops = []
    for i, (m, k, n, kernel) in enumerate(SHAPES):
        a = torch.empty((m, k), dtype=f8, device="cuda")
        b = torch.empty((n, k), dtype=f8, device="cuda")
        g.fill_normal(a, 1.0, 50 + 2 * i)
        g.fill_normal(b, 1.0, 51 + 2 * i)
        want = torch.empty((m, n), dtype=torch.float32, device="cuda")
        g.gemm_ex(a, b, want, kernel=kernel)
        ops.append((a, b, want, kernel))
    torch.cuda.synchronize()
    errors = []

    def worker(idx):
        try:
            torch.cuda.set_device(0)
            a, b, want, kernel = ops[idx]
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(25):
                    out = torch.full_like(want, float("nan"))
                    g.gemm_ex(a, b, out, kernel=kernel)
                    stream.synchronize()
                    if not torch.equal(out, want):
                        errors.append(f"thread {idx}: result differs")
                        return
        except Exception as e:          # surfaced below: a thread's exception must fail the test
            errors.append(f"thread {idx}: {e!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(ops))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads)
    assert not errors, errors
    torch.cuda.synchronize()
    assert g.device_status() == 0


def test_host_entry_point_from_two_threads_with_growing_sizes(g):
    """`b200fp8_gemm_rowcol_f32_host` owns per-device staging buffers that grow to the largest problem seen.  Two host
    threads calling it at once on one device, one of them with ever larger problems (so that the buffers are
    re-allocated while the other thread is active), must each get exactly the device entry point's result: calls
    on one device are serialised inside the library.  `b200fp8_host_release` between calls frees the buffers."""
    pkg = load_package()
    lib = pkg._cabi.lib()
    f8 = torch.float8_e4m3fn
    plans = [[(256, 512, 384), (512, 1024, 768), (1024, 1024, 2048), (2048, 2048, 2048)],
             [(300, 272, 520), (300, 272, 520), (64, 1024, 512), (1536, 512, 1024)]]
    work = []
    for t, shapes in enumerate(plans):
        items = []
        for i, (m, k, n) in enumerate(shapes):
            a = torch.empty((m, k), dtype=f8, device="cuda")
            b = torch.empty((n, k), dtype=f8, device="cuda")
            g.fill_normal(a, 1.0, 300 + 10 * t + i)
            g.fill_normal(b, 1.0, 400 + 10 * t + i)
            want = torch.empty((m, n), dtype=torch.float32, device="cuda")
            g.gemm_ex(a, b, want)
            torch.cuda.synchronize()
            items.append((a.cpu(), b.cpu(), want.cpu()))
        work.append(items)
    errors = []

    def worker(t):
        try:
            torch.cuda.set_device(0)
            for rnd in range(3):
                for (ha, hb, want) in work[t]:
                    out = torch.full(want.shape, float("nan"), dtype=torch.float32)
                    g.gemm_host(ha, hb, out)
                    if not torch.equal(out, want):
                        errors.append(f"thread {t}: result differs at {tuple(want.shape)}")
                        return
                if t == 1 and lib.b200fp8_host_release() != 0:
                    errors.append("host_release failed")
        except Exception as e:
            errors.append(f"thread {t}: {e!r}")

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=300)
    assert not any(th.is_alive() for th in threads)
    assert not errors, errors
    assert g.device_status() == 0
