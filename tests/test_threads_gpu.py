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
