"""Diagnostics: where the time of one split-K (decode-shaped) launch goes.

    B200FP8_DEBUG=1024 python tensor-core-fp8_b200/diagnostics.py [M ...]      (N = K = 8192)

With diagnostics bit 1024 set the split-K kernel records eight %globaltimer stamps per CTA: kernel entry, set-up
done, first operand block in shared memory, last MMA issued, accumulator complete, first cluster barrier passed,
reduce-scatter and stores done, end.  This prints, per stamp, the minimum / median / maximum over the CTAs of one
launch on cold operands, relative to the first CTA's entry.  The bit is read once per process, hence the variable.
"""
from __future__ import annotations

import ctypes
import importlib.util
import os
import sys

STAMPS = ["entry", "set-up done", "first block", "MMAs issued", "accumulator", "barrier 1", "reduced", "end"]


def _package():
    name = "tcfp8_b200"
    if name in sys.modules:
        return sys.modules[name]
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location(name, os.path.join(here, "__init__.py"), submodule_search_locations=[here])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules[name] = pkg
    spec.loader.exec_module(pkg)
    return pkg


def skinny_phase_timeline(ms=(1, 16, 32, 64, 128), n=8192, k=8192, out=sys.stdout):
    import numpy as np
    import torch
    pkg = _package()
    g, lib = pkg.gemm, pkg._cabi.lib()
    lib.b200fp8_debug_trace_copy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    f8 = torch.float8_e4m3fn
    bs = [torch.empty((n, k), dtype=f8, device="cuda") for _ in range(6)]       # rotated: every launch reads HBM
    for i, b in enumerate(bs):
        g.fill_normal(b, 1.0, 5 + i)
    host = np.zeros(3 * 4096, dtype=np.int64)
    for m in ms:
        a = torch.empty((m, k), dtype=f8, device="cuda")
        g.fill_normal(a, 1.0, 3)
        c = torch.empty((m, n), dtype=torch.float32, device="cuda")
        for i in range(12):
            g.gemm_ex(a, bs[i % 6], c)
        lib.b200fp8_debug_trace_copy(host.ctypes.data, host.size, 1)
        g.gemm_ex(a, bs[0], c)
        if lib.b200fp8_debug_trace_copy(host.ctypes.data, host.size, 1) == 0:
            raise SystemExit("no trace: run with B200FP8_DEBUG=1024 and M <= 128")
        t = host.reshape(-1, 8)
        t = t[t[:, 0] != 0]
        base = t[:, 0].min()
        print(f"M={m} N={n} K={k}: {len(t)} CTAs, microseconds after the first CTA's entry (min / median / max)", file=out)
        for j, name in enumerate(STAMPS):
            col = (t[:, j][t[:, j] != 0] - base) / 1e3
            if len(col):
                print(f"   {name:12s} {col.min():7.2f} {np.median(col):7.2f} {col.max():7.2f}", file=out)


if __name__ == "__main__":
    skinny_phase_timeline(tuple(int(x) for x in sys.argv[1:]) or (1, 16, 32, 64, 128))
