"""Audit of the library's automatic kernel choice: every shape with each tile kernel forced, the planner's choice
(b200fp8_choose_kernel) among them, so that a shape where the rules pick a slower kernel shows up as a ratio above 1.

    python tensor-core-fp8_b200/planner_audit.py [MxKxN ...] [--threshold 1.05] [--json FILE]

The reference has one kernel per operator and nothing to choose (GEMM/src/gemm.cu:263-277 computes a grid for the one
128 x 128 tile); this library picks among six tile kernels and the split-K kernel by shape, by rules that were
measured on one kind of GPU.  Run this after changing a rule or on a different part.  Protocol: each (shape, kernel)
as a CUDA graph of back-to-back launches over rotating B / C buffers larger than L2 (shapes of more than 2 TFLOP
launch by launch), the kernels of a shape timed in turn five times in shuffled order, every turn after a lead-in of
the same history (the AUTO kernel for one replay, or 50 ms for the long shapes whose clocks the power cap sets, then
one untimed replay of the kernel itself), the median turn counted.  M <= 128 shapes also time the split-K kernels
(ids 4 and 8).  Exit code 1 when a shape exceeds the threshold.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

# The shapes the rules were last checked on (M x K x N): cubes, decode-like and FFN-like shapes, short and long K,
# narrow N, one-round and few-round tile counts.
DEFAULT_SHAPES = """
256x256x256 512x512x512 1024x1024x1024 1536x1536x1536 2048x2048x2048 3072x3072x3072 4096x4096x4096 6144x6144x6144
8192x8192x8192 192x8192x8192 256x8192x8192 384x8192x8192 512x8192x8192 768x8192x8192 1024x8192x8192 2048x8192x8192
4096x4096x14336 4096x14336x4096 2048x4096x4096 1024x4096x4096 512x4096x4096 256x4096x4096 8192x2048x8192
8192x1024x8192 8192x512x8192 4096x512x4096 2304x1024x2304 2048x2048x8192 300x1024x3000 8192x8192x128 8192x8192x256
8192x8192x512 8192x8192x1024 16384x4096x128 4096x4096x384 640x5120x5120 1280x4096x12288 200x4096x11008
1152x8192x4096 1152x4096x8192 1536x6144x1536 4096x11008x4096 8192x8192x28672 8192x28672x8192 8192x16384x12288
16384x16384x8192 8192x32768x8192 32768x32768x4096 16x8192x8192 64x8192x8192 128x8192x8192 128x2048x2048
32x512x8192 32x2048x8192 64x2048x4096 64x512x8192 48x2048x2048 128x4096x1024 16x1024x4096 1x2048x2048 32x8192x57344
""".split()

TILE_KERNELS = (1, 2, 3, 5, 6, 7)
SPLIT_K_KERNELS = (4, 8)


def load_package():
    name = "tcfp8_b200"                  # the directory name is not an identifier: load the package under this one
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(HERE, "__init__.py"), submodule_search_locations=[HERE])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules[name] = pkg
    spec.loader.exec_module(pkg)
    return pkg


def time_shape(torch, g, m, k, n, kernels, rounds=5):
    """{kernel: microseconds per launch} (kernels that do not take the shape are left out).  All kernels share one set
    of buffers and are timed in turn, `rounds` times in shuffled order, each turn a lead-in and then a timed replay;
    a kernel's figure is the median of its turns, so that none owes its place to the order."""
    f8 = torch.float8_e4m3fn
    per_set = n * k + 4 * m * n
    nsets = 1 if m * k + per_set > (512 << 20) else max(2, min(8, (1 << 30) // per_set))
    a = torch.empty((m, k), dtype=f8, device="cuda")
    g.fill_normal(a, 1.0, 1)
    bs = [torch.empty((n, k), dtype=f8, device="cuda") for _ in range(nsets)]
    cs = [torch.empty((m, n), dtype=torch.float32, device="cuda") for _ in range(nsets)]
    for i, b in enumerate(bs):
        g.fill_normal(b, 1.0, 2 + i)
    flops = 2.0 * m * k * n
    est = max(flops / 2.5e15, (m * k + n * k + 4.0 * m * n) / 5e12, 4e-6)
    iters = 10 if flops >= 2e12 else int(max(4, min(48, 2.5e-3 / est)))
    runners = {}
    for kernel in kernels:
        def launches(kernel=kernel):
            for i in range(iters):
                g.gemm_ex(a, bs[i % nsets], cs[i % nsets], kernel=kernel)
        try:
            launches()
            torch.cuda.synchronize()
        except g.B200Fp8Error:
            continue
        if flops < 2e12:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                launches()
            runners[kernel] = graph.replay
        else:
            runners[kernel] = launches
    turns = {kernel: [] for kernel in runners}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    lead = torch.cuda.Event(enable_timing=True)
    long_steps = flops >= 2e12
    rng = random.Random(m * 1000003 + k * 1009 + n)
    order = list(runners)
    common = runners[kernels[0]] if kernels[0] in runners else next(iter(runners.values()))
    for _ in range(rounds):
        rng.shuffle(order)
        for kernel in order:
            # the same history before every timed replay, whatever ran before in the shuffled order: the first kernel
            # of the list (AUTO) for a while (one replay; 50 ms for long steps, whose clocks the power cap sets), then
            # one untimed replay of the kernel itself.  Without it a kernel timed after an inefficient one inherits
            # that one's power headroom and reads up to a tenth faster.
            lead.record()
            while True:
                common()
                e0.record()
                torch.cuda.synchronize()
                if not long_steps or lead.elapsed_time(e0) >= 50.0:
                    break
            runners[kernel]()
            e0.record()
            runners[kernel]()
            e1.record()
            torch.cuda.synchronize()
            turns[kernel].append(e0.elapsed_time(e1) / iters * 1e3)
    assert g.device_status() == 0
    return {kernel: sorted(v)[len(v) // 2] for kernel, v in turns.items()}


def audit(torch, g, lib, shapes, threshold):
    """`chosen / best`: the time of the kernel the planner selects (asked through b200fp8_choose_kernel and timed as a
    forced kernel like the others, so that both sides of the ratio come from the same protocol) over the best forced
    time.  The AUTO call itself is timed too, as a check that it runs what the planner reports."""
    rows, flagged = [], []
    for spec in shapes:
        m, k, n = (int(v) for v in spec.lower().split("x"))
        forced = TILE_KERNELS + (SPLIT_K_KERNELS if m <= 128 else ())
        chosen = lib.b200fp8_choose_kernel(m, k, n)
        times = time_shape(torch, g, m, k, n, (0,) + forced)
        valid = {kern: t for kern, t in times.items() if kern}
        best_kernel = min(valid, key=valid.get)
        ratio = valid[chosen] / valid[best_kernel]
        rows.append({"m": m, "k": k, "n": n, "chosen_kernel": chosen, "chosen_us": round(valid[chosen], 2),
                     "auto_us": round(times[0], 2), "best_kernel": best_kernel, "best_us": round(valid[best_kernel], 2),
                     "chosen_over_best": round(ratio, 3), "us_by_kernel": {str(kern): round(t, 2) for kern, t in valid.items()}})
        mark = "  <-- above threshold" if ratio > threshold else ""
        print(f"{spec:>20s}  chosen id {chosen} {valid[chosen]:9.2f} us (as AUTO {times[0]:9.2f})   best id {best_kernel} "
              f"{valid[best_kernel]:9.2f} us   chosen / best {ratio:5.3f}{mark}", flush=True)
        if ratio > threshold:
            flagged.append(spec)
    return rows, flagged


def main(argv=None, pkg=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("shapes", nargs="*", help="MxKxN (default: the built-in list)")
    ap.add_argument("--threshold", type=float, default=1.05,
                    help="flag a shape when the chosen kernel is slower than the best forced kernel by more than this factor "
                         "(the same kernel timed twice differs by a few per cent on a power-capped GPU)")
    ap.add_argument("--json", default=None, help="write the table to this file")
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("planner_audit needs a GPU", file=sys.stderr)
        return 2
    pkg = pkg or load_package()
    pkg._cabi.lib()                      # no fallback: the library must be built
    torch.cuda.set_device(0)
    rows, flagged = audit(torch, pkg.gemm, pkg._cabi.lib(), args.shapes or DEFAULT_SHAPES, args.threshold)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    print(f"{len(rows)} shapes, {len(flagged)} above {args.threshold}: {' '.join(flagged)}")
    return 1 if flagged else 0


if __name__ == "__main__":
    sys.exit(main())
