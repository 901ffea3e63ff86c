"""The reference benchmark driver's command line on top of this library, with working CSV output.

    python tensor-core-fp8_b200/sweep.py dimM dimK dimN kernel verify record testbench [--cublaslt] [--data-dir DIR]
                                         [--jsonl FILE [--resume]] [--plot FILE.svg]

Same seven positional arguments, kernel numbering, timing protocol and CSV lines as the
reference driver (GEMM/gemm_main.cpp:196-313 argument handling, :25-26 and :69-84 timing:
20 warm-up calls, then 100 calls each bracketed by its own event pair and synchronised;
GFLOPS = 2 M K N / 1e6 / total_ms * repeat; :87-110 one appended line "M,K,N,GFLOPS" per
shape in ./data/fp8_gemm_v<kernel>.csv):

    kernel 1 / 3 / 5 / 7   gemm::GEMM   e4m3 x e4m3 / e5m2 x e5m2 / e4m3 x e5m2 / e5m2 x e4m3
    kernel 2 / 4 / 6 / 8   gemm::GEMM4  the same four pairs (the reference has 4, 6, 8 commented out)
    kernel 9               the cuBLASLt comparator (GEMM/src/cublas.cu), like for like: alpha = 1, beta = 0
    testbench != 0         the 64-cube sweep M = K = N = 256 .. 16384 (GEMM/gemm_main.cpp:264-270)

Differences, on purpose: the data directory is created (the reference appends into a directory
that does not exist and silently records nothing); `verify` checks on the device in FP64
(a random-vector product check of the whole C plus full rows against an FP64 matmul) instead
of the O(MNK) single-thread CPU loop, so that it stays usable at 16384^3; `--cublaslt` records
the comparator beside every shape in fp8_gemm_cublaslt.csv; `--jsonl` appends one JSON object per measured
(shape, kernel) and `--resume` skips what that file already holds, so an interrupted sweep continues where it
stopped; `--plot` draws every CSV of the data directory (this library's kernels and cuBLASLt) as TFLOP/s over the
cube size into one SVG file (no plotting package needed).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

PAIRS = {1: (0, 0), 2: (0, 0), 3: (1, 1), 4: (1, 1), 5: (0, 1), 6: (0, 1), 7: (1, 0), 8: (1, 0), 9: (0, 0)}
NAMES = {0: "e4m3", 1: "e5m2"}
WARMUP, REPEAT = 20, 100          # GEMM/gemm_main.cpp:25-26


def parse(argv):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    for name in ("dimM", "dimK", "dimN", "kernel", "verify", "record", "testbench"):
        ap.add_argument(name, type=int)
    ap.add_argument("--cublaslt", action="store_true", help="also time cuBLASLt on the same buffers and record it")
    ap.add_argument("--data-dir", default="./data")
    ap.add_argument("--max-dim", type=int, default=16384, help="largest cube of the sweep (the reference's is 16384)")
    ap.add_argument("--jsonl", default=None, help="append one JSON object per measured (shape, kernel) to this file")
    ap.add_argument("--resume", action="store_true", help="skip the (shape, kernel) pairs the --jsonl file already holds")
    ap.add_argument("--plot", default=None, help="after the run, draw the CSV files of the data directory into this SVG file")
    args = ap.parse_args(argv)
    if args.kernel not in PAIRS:
        ap.error("kernel must be 1..9")
    return args


def shapes(args):
    """The shapes one invocation covers: the given one, or the reference's 64 cubes."""
    if args.testbench == 0:
        return [(args.dimM, args.dimK, args.dimN)]
    return [(256 * (i + 1),) * 3 for i in range(64) if 256 * (i + 1) <= args.max_dim]


def gflops(m, k, n, total_ms, repeat=REPEAT):
    """The driver's figure (GEMM/gemm_main.cpp:84): despite the 1e6 it is GFLOP/s, because the time is in ms."""
    return float(m) * k * n * 2 / 1000 / 1000 / total_ms * repeat


def csv_name(kernel):
    return "fp8_gemm_cublaslt.csv" if kernel == 9 else f"fp8_gemm_v{kernel}.csv"


def record_line(data_dir, kernel, m, k, n, perf):
    os.makedirs(data_dir, exist_ok=True)
    path = os.path.join(data_dir, csv_name(kernel))
    with open(path, "a") as f:
        f.write(f"{m},{k},{n},{perf}\n")
    return path


def jsonl_done(path):
    """The (m, k, n, kernel) tuples a JSONL log already holds (lines that do not parse are ignored: a run that was
    killed in the middle of a line must not block the resume)."""
    done = set()
    if path and os.path.exists(path):
        with open(path) as f:
            for line in f:
                try:
                    r = json.loads(line)
                    done.add((int(r["m"]), int(r["k"]), int(r["n"]), int(r["kernel"])))
                except (ValueError, KeyError, TypeError):
                    continue
    return done


def jsonl_append(path, record):
    d = os.path.dirname(os.path.abspath(path))
    os.makedirs(d, exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(record) + "\n")
        f.flush()
        os.fsync(f.fileno())


def read_csvs(data_dir):
    """{label: [(m, gflops), ...]} of every CSV the sweep writes into `data_dir` (cube shapes only, sorted by size)."""
    series = {}
    if not os.path.isdir(data_dir):
        return series
    for name in sorted(os.listdir(data_dir)):
        if not (name.startswith("fp8_gemm_") and name.endswith(".csv")):
            continue
        label = name[len("fp8_gemm_"):-len(".csv")]
        pts = {}
        with open(os.path.join(data_dir, name)) as f:
            for line in f:
                try:
                    m, k, n, perf = line.strip().split(",")
                    if int(m) == int(k) == int(n):
                        pts[int(m)] = float(perf)          # a later line for the same shape replaces the earlier one
                except ValueError:
                    continue
        if pts:
            series[label] = sorted(pts.items())
    return series


def plot_svg(data_dir, out_path, width=960, height=540):
    """TFLOP/s over the cube size, one polyline per CSV file, as a self-contained SVG (the reference plots nothing;
    its CSV lines are what a plotting script would read: GEMM/gemm_main.cpp:87-110, GEMM/src/cublas.cu:126-134)."""
    series = read_csvs(data_dir)
    if not series:
        return None
    xs = [m for pts in series.values() for m, _ in pts]
    ys = [p / 1000.0 for pts in series.values() for _, p in pts]
    x0, x1, y1 = min(xs), max(xs), max(ys) * 1.05
    left, right, top, bottom = 70, 190, 30, 50
    pw, ph = width - left - right, height - top - bottom
    sx = lambda m: left + (pw * (m - x0) / (x1 - x0) if x1 > x0 else pw / 2)
    sy = lambda t: top + ph * (1 - t / y1)
    colours = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e", "#8c564b", "#e377c2", "#17becf", "#7f7f7f"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<text x="{left}" y="18" font-size="14">FP8 GEMM, M = K = N: TFLOP/s (reference protocol: mean of 100 synchronised calls)</text>']
    for i in range(6):
        t = y1 * i / 5
        out.append(f'<line x1="{left}" y1="{sy(t):.1f}" x2="{left + pw}" y2="{sy(t):.1f}" stroke="#dddddd"/>')
        out.append(f'<text x="{left - 8}" y="{sy(t) + 4:.1f}" text-anchor="end">{t:.0f}</text>')
    for m in sorted(set(xs))[::max(1, len(set(xs)) // 8)]:
        out.append(f'<text x="{sx(m):.1f}" y="{top + ph + 18}" text-anchor="middle">{m}</text>')
    out.append(f'<rect x="{left}" y="{top}" width="{pw}" height="{ph}" fill="none" stroke="black"/>')
    for i, (label, pts) in enumerate(series.items()):
        c = colours[i % len(colours)]
        path = " ".join(f"{sx(m):.1f},{sy(p / 1000.0):.1f}" for m, p in pts)
        out.append(f'<polyline points="{path}" fill="none" stroke="{c}" stroke-width="2"/>')
        for m, p in pts:
            out.append(f'<circle cx="{sx(m):.1f}" cy="{sy(p / 1000.0):.1f}" r="2.5" fill="{c}"/>')
        out.append(f'<rect x="{left + pw + 14}" y="{top + 18 * i}" width="12" height="12" fill="{c}"/>')
        out.append(f'<text x="{left + pw + 32}" y="{top + 18 * i + 11}">{label}</text>')
    out.append("</svg>")
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    with open(out_path, "w") as f:
        f.write("\n".join(out) + "\n")
    return out_path


def time_calls(call, torch):
    """The driver's protocol: every call between its own event pair, synchronised; warm-up calls not counted."""
    total = 0.0
    for i in range(WARMUP + REPEAT):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        call()
        end.record()
        end.synchronize()
        if i >= WARMUP:
            total += start.elapsed_time(end)
    return total


def verify_on_device(torch, a, b, c, rows=16):
    """Worst |C - C64| / (1e-3 * sum|a b| + 1e-6) over `rows` full rows (FP64 matmul on the device), and a
    random-vector check C r = A (B^T r) of the whole matrix with the summed bound."""
    m, n = c.shape
    gen = torch.Generator(device=c.device).manual_seed(1)
    pick = torch.randint(0, m, (min(rows, m),), device=c.device, generator=gen)
    worst = 0.0
    a64 = a[pick].double()
    for n0 in range(0, n, 4096):
        b64 = b[n0:n0 + 4096].double()
        want = a64 @ b64.T
        bound = 1e-3 * (a64.abs() @ b64.abs().T) + 1e-6
        worst = max(worst, float(((c[pick, n0:n0 + 4096].double() - want).abs() / bound).max()))
    r = torch.randint(0, 2, (n,), device=c.device, generator=gen).double() * 2 - 1
    btr = torch.zeros(b.shape[1], dtype=torch.float64, device=c.device)
    babs = torch.zeros_like(btr)
    for n0 in range(0, n, 4096):
        blk = b[n0:n0 + 4096].double()
        btr += blk.T @ r[n0:n0 + 4096]
        babs += blk.abs().sum(dim=0)
    for m0 in range(0, m, 4096):
        ablk = a[m0:m0 + 4096].double()
        bound = 1e-3 * (ablk.abs() @ babs) + 1e-6 * n
        worst = max(worst, float((((c[m0:m0 + 4096].double() @ r) - ablk @ btr).abs() / bound).max()))
    return worst


def run_shape(pkg, torch, args, m, k, n):
    g = pkg.gemm
    fa, fb = PAIRS[args.kernel]
    f8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}
    a = torch.empty((m, k), dtype=f8[fa], device="cuda")
    b = torch.empty((n, k), dtype=f8[fb], device="cuda")
    g.fill_normal(a, 2.0 if fa else 1.0, 0xB200F800)
    g.fill_normal(b, 2.0 if fb else 1.0, 0xB200F801)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    results = []
    if args.kernel == 9 or args.cublaslt:
        cmp = ctypes.CDLL(os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "libb200fp8_cmp.so"))
        vp, ci = ctypes.c_void_p, ctypes.c_int
        cmp.b200fp8_cmp_cublaslt.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, ci, ci, ctypes.POINTER(ctypes.c_float),
                                             ctypes.POINTER(ci), vp]
        cmp.b200fp8_cmp_cublaslt_enqueue.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, vp]
        ms, found = ctypes.c_float(), ci()
        rc = cmp.b200fp8_cmp_cublaslt(m, k, n, a.data_ptr(), fa, b.data_ptr(), fb, c.data_ptr(), 5, 8, 0,
                                      ctypes.byref(ms), ctypes.byref(found), None)
        if rc == 0:
            total = time_calls(lambda: cmp.b200fp8_cmp_cublaslt_enqueue(m, k, n, a.data_ptr(), fa, b.data_ptr(), fb,
                                                                        c.data_ptr(), None), torch)
            results.append((9, gflops(m, k, n, total)))
        else:
            print(f"cuBLASLt: no kernel for {NAMES[fa]} x {NAMES[fb]} (status {rc})")
    if args.kernel != 9:
        op = g.GEMM if args.kernel % 2 else g.GEMM4
        total = time_calls(lambda: op(m, k, n, a, b, c), torch)
        results.append((args.kernel, gflops(m, k, n, total)))
        print(f"GEMM-stage{2 if args.kernel % 2 else 4}:  M = {m}, K = {k}, N = {n}")
    for kern, perf in results:
        label = "cuBLASLt" if kern == 9 else "FP8-TC"
        print(f"{label} Avager Performance = {perf:f} GFlops")
        if args.record:
            record_line(args.data_dir, kern, m, k, n, perf)
        if args.jsonl:
            jsonl_append(args.jsonl, {"m": m, "k": k, "n": n, "kernel": kern, "a": NAMES[fa], "b": NAMES[fb], "gflops": perf,
                                      "protocol": f"{WARMUP} warm-up + {REPEAT} synchronised calls"})
    if args.verify and args.kernel != 9:
        worst = verify_on_device(torch, a, b, c)
        status = g.device_status()
        print(f"verify: worst error / tolerance = {worst:.3g}, device status {status}: {'pass' if worst <= 1 and status == 0 else 'FAIL'}")
        if worst > 1 or status != 0:
            return 1
    return 0


def main(argv=None, pkg=None):
    args = parse(sys.argv[1:] if argv is None else argv)
    import torch
    if pkg is None:
        import importlib.util
        here = os.path.dirname(os.path.abspath(__file__))
        name = "tcfp8_b200"
        if name in sys.modules:
            pkg = sys.modules[name]
        else:
            spec = importlib.util.spec_from_file_location(name, os.path.join(here, "__init__.py"), submodule_search_locations=[here])
            pkg = importlib.util.module_from_spec(spec)
            sys.modules[name] = pkg
            spec.loader.exec_module(pkg)
    pkg._cabi.lib()               # fail here, loudly, if the CUDA library is missing
    fa, fb = PAIRS[args.kernel]
    print(f"{NAMES[fa]} * {NAMES[fb]} = fp32" if args.kernel != 9 else "cuBLASLt: e4m3 * e4m3 = fp32")
    rc = 0
    done = jsonl_done(args.jsonl) if args.resume else set()
    for (m, k, n) in shapes(args):
        if (m, k, n, args.kernel) in done:
            print(f"M = {m}, K = {k}, N = {n}: already in {args.jsonl}, skipped")
            continue
        rc |= run_shape(pkg, torch, args, m, k, n)
    if args.plot:
        out = plot_svg(args.data_dir, args.plot)
        print(f"plot: {out if out else 'nothing recorded in ' + args.data_dir}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
