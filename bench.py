"""Benchmark of the FP8 GEMM path (one JSON line on stdout, printed by rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic operands, N(0,1) cast to e4m3 with RNE + saturate-to-finite, seeded):
    shard32768  M = N = K = 32768, B and C column-split evenly over the N GPUs, A replicated
                (default; total work fixed => "strong" scaling; no collective in the timed step)
    gemm8192    M = N = K = 8192 on every GPU (replicas)
    gemm4096    M = N = K = 4096
    ffn_up      M = 8192, K = 8192, N = 28672
    ffn_down    M = 8192, K = 28672, N = 8192
    skinny16    M = 16, N = K = 8192 (HBM-bound; rotates over distinct B buffers so each step streams from HBM)

A step is one operator call on operands resident in HBM.  `value` is whole-job TFLOPS over all
GPUs from the max-over-ranks device time; `e2e` is the same quantity through the host-pointer
entry point (pinned host buffers, uploads and the download of C inside the timed region).

Beside the headline the default run reports, in the same line:
    parity      the C buffer that was timed, checked after the timed region (FP64 oracle on sampled rows, columns and
                points over the full K; a randomised product check of every element on the device)
    configs     (N = 1) every other benchmark configuration -- 1024^3, 4096^3 x 4 dtype pairs x ring depths, 8192^3,
                the FFN shapes, the decode shapes -- each timed as CUDA graphs over rotating buffers, alternating with
                cuBLASLt on the same buffers, with the parity of its own timed buffer
    side        (N = 1) the reference's own kernels where they build for sm_100 (time only)
    sustained, allgather, fused_allgather   (N > 1) a one-second steady-state leg per GPU, the NCCL all-gather of the C
                blocks, and the GEMM with the all-gather fused into its epilogue, each with its own parity
`--impl reference` times the reference's own CPU implementation of the path (its verification
loop, GEMM/gemm_main.cpp:45-52, as restated by the oracle) on all host threads over a bounded
sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, K, N, sharded)
    "shard32768": (32768, 32768, 32768, True),
    "gemm8192": (8192, 8192, 8192, False),
    "gemm4096": (4096, 4096, 4096, False),
    "ffn_up": (8192, 8192, 28672, False),
    "ffn_down": (8192, 28672, 8192, False),
    "gemm1024": (1024, 1024, 1024, False),
    "skinny1": (1, 8192, 8192, False),
    "skinny16": (16, 8192, 8192, False),
    "skinny64": (64, 8192, 8192, False),
    "skinny128": (128, 8192, 8192, False),
    "skinny_wide": (32, 8192, 57344, False),
    "m256": (256, 8192, 8192, False),
    "m512": (512, 8192, 8192, False),
}
# Sparse workloads (blocked-ELL A, 128 x 128 blocks; one GPU): name -> (op, M, K, N, stored blocks per block row)
SPARSE_WORKLOADS = {
    "spmm8192_d25": ("spmm", 8192, 8192, 8192, 16),      # a quarter of the 64 block columns
    "spmm8192_d100": ("spmm", 8192, 8192, 8192, 64),     # every block stored: the table lookup's overhead
    "spmv16384_d25": ("spmv", 16384, 16384, 1, 32),
    "gemv16384": ("gemv", 1, 16384, 16384, 0),
}
SEED_BASE = 0xB200F800
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
NVLINK_PEER_COPY_GBS = 770.0      # measured peer-copy rate per direction per GPU on this pool (nominal 900)
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's kernel, from one ncu capture at N = 1
NCU_TRAFFIC_BYTES = {"shard32768": 30.11e9, "gemm8192": 547.7e6, "skinny16": 67.84e6, "skinny128": 69.3e6}
DTYPE_NAMES = {0: "e4m3", 1: "e5m2"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def host_threads() -> int:
    """Host threads this process may run on.  Launchers for multi-rank runs export OMP_NUM_THREADS=1, which would make
    the CPU arm a single-thread run: the team is sized from the scheduler's affinity mask instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_rate(M, K, N, rows_per_thread: int, seed_a: int, seed_b: int):
    """The reference's CPU loop (oracle port) on a bounded sample: returns (TFLOPS, threads, description, seconds)."""
    import numpy as np
    from oracle import fp8_oracle as fo
    threads = host_threads()
    rows = min(M, rows_per_thread * threads)
    cols = min(N, 512)
    A = fo.fill_normal(rows * K, fo.E4M3, 1.0, seed_a).reshape(rows, K)
    B = fo.fill_normal(cols * K, fo.E4M3, 1.0, seed_b).reshape(cols, K)
    t0 = time.perf_counter()
    C = fo.gemm_ref_float(A, fo.E4M3, B, fo.E4M3, threads=threads)
    dt = time.perf_counter() - t0
    assert np.isfinite(C).all()
    flops = 2.0 * rows * cols * K
    return flops / dt / 1e12, threads, f"rows 0..{rows - 1} x cols 0..{cols - 1} of C at full K={K} ({flops / 1e9:.2f} GFLOP)", dt


def reference_binary_rate(size: int = 512):
    """The reference's OWN compiled CPU loop (its unmodified gemm_main.cpp built over host stand-ins, oracle/_ref):
    wall time of a run with verify = 1 minus a run with verify = 0 at size^3 -- the difference is exactly its
    single-threaded verification loop (GEMM/gemm_main.cpp:39-53).  None where the binary was not built."""
    import subprocess
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_gemm_cpu")
    if not os.path.exists(exe):
        return None

    def run(verify):
        t0 = time.perf_counter()
        subprocess.run([exe, str(size), str(size), str(size), "2", str(verify), "0", "0"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=120)
        return time.perf_counter() - t0
    try:
        base = min(run(0), run(0))
        full = min(run(1), run(1))
    except Exception:
        return None
    loop = full - base
    if loop <= 0:
        return None
    return {"value": 2.0 * size ** 3 / loop / 1e12, "unit": "TFLOPS", "cores": 1, "kind": "reference",
            "sample": f"{size}^3 e4m3 x e4m3, the reference driver's own verification loop, {loop:.2f} s "
                      "(run with verify = 1 minus run with verify = 0)"}


def workload_config(args, M, K, N, n_local, world, sharded, l2, timing):
    """The `config` object: the same keys and, for one workload and N, the same values in both arms."""
    return {"workload": args.workload, "M": M, "K": K, "N": N, "n_per_rank": n_local, "layout": "row-col",
            "a": args.a_dtype, "b": args.b_dtype, "out": "f32",
            "parallelism": f"n-shard x{world}" if sharded else f"replicas x{world}", "l2": l2,
            "kernel": args.kernel, "depth": args.depth, "timing": timing}


def describe_l2(nsets):
    return "inputs larger than L2" if nsets == 1 else f"rotating over {nsets} distinct B/C buffer sets larger than L2"


def operand_sets(M, K, n_local):
    bytes_per_set = n_local * K + 4 * M * n_local
    return 1 if (M * K + bytes_per_set) > (512 << 20) else max(2, min(8, (1 << 30) // max(1, bytes_per_set)))


def graph_timed(M, K, n_local):
    # Short steps are launch-bound when driven call by call from Python, so their K steps are captured
    # once in a CUDA graph and replayed; long steps are timed launch by launch.
    return 2.0 * M * K * n_local < 2e12


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    if args.workload in SPARSE_WORKLOADS:       # the CPU loop has no sparse form: the dense problem of the same shape
        M, K, N, sharded = SPARSE_WORKLOADS[args.workload][1:4] + (False,)
    else:
        M, K, N, sharded = WORKLOADS[args.workload]
    world = max(1, args.gpus)
    if sharded:
        from __graft_entry__ import load_package
        n_local = load_package().shard.column_shard(N, 0, world).n
    else:
        n_local = N
    # bounded sample per step: about a second of work per step on all host threads
    rates = []
    for i in range(args.warmup + args.steps):
        r, threads, sample, dt = cpu_reference_rate(M, K, N, 128, SEED_BASE + 64, SEED_BASE + 65)
        if i >= args.warmup:
            rates.append((r, dt))
    total_t = sum(d for _, d in rates)
    value = sum(r * d for r, d in rates) / total_t
    line = {
        "impl": "reference", "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_t / len(rates),
        "higher_is_better": True, "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "fp8",
        "data": "synthetic",
        # the GPU arm's description of the same problem (the CPU arm runs a bounded sample of it, see cpu_baseline)
        "config": workload_config(args, M, K, N, n_local, world, sharded, describe_l2(operand_sets(M, K, n_local)),
                                  "one CUDA graph of all steps, replayed" if graph_timed(M, K, n_local) else "launch by launch"),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port",
                         "sample": "each step: " + sample + "; the reference's float loop "
                                   "(GEMM/gemm_main.cpp:45-52) restated in oracle/fp8_oracle.c, OpenMP over rows"},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_loop = reference_binary_rate()
    if ref_loop is not None:
        line["cpu_baseline"]["reference_loop"] = ref_loop
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# parity of a timed buffer
# ---------------------------------------------------------------------------------------------------------------

def freivalds(torch, a, b, c, n_cols=None):
    """C r against A (B^T r) in FP64 on the device, bound = the summed per-element tolerance: covers every element."""
    n = b.shape[0]
    dev = a.device
    gen = torch.Generator(device=dev).manual_seed(7)
    r = (torch.randint(0, 2, (n,), device=dev, generator=gen).double() * 2 - 1)
    worst = 0.0
    btr = torch.zeros(b.shape[1], dtype=torch.float64, device=dev)
    babs = torch.zeros_like(btr)
    for n0 in range(0, n, 4096):
        blk = b[n0:n0 + 4096].double()
        btr += blk.T @ r[n0:n0 + 4096]
        babs += blk.abs().sum(dim=0)
        del blk
    for m0 in range(0, a.shape[0], 4096):
        ablk = a[m0:m0 + 4096].double()
        want = ablk @ btr
        bound = 1e-3 * (ablk.abs() @ babs) + 1e-6 * n
        got = c[m0:m0 + 4096].double() @ r
        worst = max(worst, float(((got - want).abs() / bound).max()))
        del ablk
    return worst


def parity_of(torch, g, a, b, c, rows=8, cols=8, points=4096):
    """Checks a C buffer the benchmark has just timed: `rows` full rows, `cols` full columns and `points` random
    elements against the FP64 oracle (|C - C_ref| <= 1e-3 * sum_k |a b| + 1e-6, every sampled element over the full
    K), and every element through the randomised product check on the device.  `worst` is the largest error as a
    fraction of the tolerance over both: <= 1 passes."""
    import numpy as np
    from oracle import fp8_oracle as fo
    t0 = time.perf_counter()
    m, k = a.shape
    n = b.shape[0]
    fa, fb = g.dtype_code(a), g.dtype_code(b)
    dev = a.device
    rng = np.random.default_rng(11)
    pick_m = np.unique(np.concatenate([[0, m - 1], rng.integers(0, m, rows)]))
    pick_n = np.unique(np.concatenate([[0, n - 1], rng.integers(0, n, cols)]))
    ms, ns = rng.integers(0, m, points), rng.integers(0, n, points)
    tm, tn = torch.from_numpy(pick_m).to(dev), torch.from_numpy(pick_n).to(dev)
    a8, b8 = a.view(torch.uint8), b.view(torch.uint8)
    worst, bad = 0.0, 0
    # full rows: A's sampled rows against all of B (B comes to the host once; A only in the sampled rows)
    B = b8.cpu().numpy()
    C64, S = fo.gemm_f64(np.ascontiguousarray(a8[tm].cpu().numpy()), fa, B, fb)
    nb, w, _ = fo.check_tolerance(c[tm].cpu().numpy(), C64, S)
    bad, worst = bad + int(nb), max(worst, float(w))
    A = a8.cpu().numpy()
    C64, S = fo.gemm_f64(A, fa, np.ascontiguousarray(B[pick_n]), fb)
    nb, w, _ = fo.check_tolerance(np.ascontiguousarray(c[:, tn].cpu().numpy()), C64, S)
    bad, worst = bad + int(nb), max(worst, float(w))
    C64, S = fo.gemm_f64_points(A, fa, B, fb, ms, ns)
    nb, w, _ = fo.check_tolerance(c[torch.from_numpy(ms).to(dev), torch.from_numpy(ns).to(dev)].cpu().numpy(), C64, S)
    bad, worst = bad + int(nb), max(worst, float(w))
    del A, B
    fr = freivalds(torch, a, b, c)
    return {"worst": max(worst, fr), "oracle_worst": worst, "elements_outside_tolerance": bad, "freivalds": fr,
            "sample": f"{len(pick_m)} rows + {len(pick_n)} columns + {points} points (FP64 oracle, full K); every element "
                      "by the randomised product check", "seconds": round(time.perf_counter() - t0, 2)}


# ---------------------------------------------------------------------------------------------------------------
# the other benchmark configurations, ours alternating with cuBLASLt on the same buffers
# ---------------------------------------------------------------------------------------------------------------

class Comparator:
    """cuBLASLt FP8 through the separate comparator library (never part of libb200fp8.so)."""

    def __init__(self, path):
        self.lib = ctypes.CDLL(path) if os.path.exists(path) else None
        if self.lib is not None:
            ci, vp, fp = ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)
            self.lib.b200fp8_cmp_cublaslt.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, ci, ci, fp, ctypes.POINTER(ci), vp]
            self.lib.b200fp8_cmp_cublaslt_enqueue.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, vp]

    def choose(self, m, k, n, a, fa, b, fb, c, stream):
        """Picks the fastest of cuBLASLt's candidates for the shape; False when it offers none (e5m2 x e5m2)."""
        if self.lib is None:
            return False
        ms, found = ctypes.c_float(-1), ctypes.c_int(0)
        return self.lib.b200fp8_cmp_cublaslt(m, k, n, a.data_ptr(), fa, b.data_ptr(), fb, c.data_ptr(), 3, 8, 0,
                                             ctypes.byref(ms), ctypes.byref(found), stream) == 0

    def enqueue(self, m, k, n, a, fa, b, fb, c, stream):
        return self.lib.b200fp8_cmp_cublaslt_enqueue(m, k, n, a.data_ptr(), fa, b.data_ptr(), fb, c.data_ptr(), stream)


def measure_config(torch, g, cmp, dev, name, M, K, N, fa, fb, depth, kernel, peaks, check=True, seed=0):
    """One configuration on one GPU.  Ours and cuBLASLt each as a CUDA graph of `iters` launches over rotating B/C
    buffers larger than L2 (long steps: launch by launch), four alternating rounds of lead-in + timed replay, the
    first round dropped.  Then the parity of C buffer 0, which every timed replay rewrote."""
    f8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}
    nsets = operand_sets(M, K, N)
    a = torch.empty((M, K), dtype=f8[fa], device=dev)
    g.fill_normal(a, 2.0 if fa else 1.0, SEED_BASE + 128 + seed)
    bs, cs = [], []
    for i in range(nsets):
        b = torch.empty((N, K), dtype=f8[fb], device=dev)
        g.fill_normal(b, 2.0 if fb else 1.0, SEED_BASE + 129 + seed + 1000 * i)
        bs.append(b)
        cs.append(torch.empty((M, N), dtype=torch.float32, device=dev))
    flops = 2.0 * M * K * N
    nbytes = float(M * K + N * K + 4 * M * N)
    est = max(flops / 2.5e15, nbytes / 5e12, 4e-6)
    iters = int(max(4, min(48, 2.5e-3 / est)))
    long_step = flops >= 2e12
    if long_step:
        iters = 10
    stream = torch.cuda.current_stream().cuda_stream
    have_cmp = cmp.choose(M, K, N, a, fa, bs[0], fb, cs[0], stream)

    def ours(i, _cap=None):
        g.gemm_ex(a, bs[i % nsets], cs[i % nsets], depth=depth, kernel=kernel)

    def theirs(i, cap=None):
        cmp.enqueue(M, K, N, a, fa, bs[i % nsets], fb, cs[i % nsets], cap or stream)

    def as_graph(fn):
        for i in range(2):
            fn(i)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            cap = torch.cuda.current_stream().cuda_stream
            for i in range(iters):
                fn(i, cap)
        return gr.replay

    def as_loop(fn):
        def run():
            for i in range(iters):
                fn(i)
        return run

    wrap = as_loop if long_step else as_graph
    run_ours = wrap(ours)
    run_theirs = wrap(theirs) if have_cmp else None
    t_ours, t_theirs = [], []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rnd in range(4):
        for run, acc in ((run_ours, t_ours), (run_theirs, t_theirs)):
            if run is None:
                continue
            run()                                   # lead-in: clocks and caches settle to THIS kernel's steady state
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            if rnd:
                acc.append(e0.elapsed_time(e1) / iters)
    if have_cmp:                                    # the last writer of the buffers must be OUR kernel: parity is of our C
        run_ours()
        torch.cuda.synchronize()
    status = g.device_status()
    ms = sum(t_ours) / len(t_ours)
    row = {"M": M, "K": K, "N": N, "a": DTYPE_NAMES[fa], "b": DTYPE_NAMES[fb], "depth": depth, "kernel": kernel,
           "ms": ms, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
           "timing": ("launch by launch" if long_step else f"CUDA graph of {iters} launches")
                     + f" over {nsets} rotating B/C sets, 3 alternating rounds", "launches_per_replay": iters,
           "device_status": status}
    if M <= 128:
        row.update({"bound": "hbm", "frac": row["gbs"] / peaks["hbm_gbs"], "peak": peaks["hbm_gbs"], "peak_unit": "GB/s",
                    "frac_of_nominal_8TBs": row["gbs"] / NOMINAL_HBM_GBS})
    else:
        peak = 2.0 * peaks["bf16_burst"]            # a few milliseconds of launches: the burst figure applies
        row.update({"bound": "tensor", "frac": row["tflops"] / peak, "peak": peak, "peak_unit": "TFLOP/s (2 x burst cuBLAS bf16)",
                    "frac_of_nominal_4500": row["tflops"] / NOMINAL_FP8_TFLOPS})
    if t_theirs:
        t = sum(t_theirs) / len(t_theirs)
        row.update({"cublaslt_ms": t, "vs_cublaslt": t / ms})
    else:
        row.update({"cublaslt_ms": None, "vs_cublaslt": None,
                    "cublaslt_note": "no cuBLASLt kernel for this dtype pair" if cmp.lib is not None else "comparator library not built"})
    if check:
        row["parity"] = parity_of(torch, g, a, bs[0], cs[0], rows=8, cols=8, points=2048)
    del a, bs, cs
    torch.cuda.empty_cache()
    return row


def run_configs(torch, g, cmp, dev, peaks, budget_s=150.0):
    """Every benchmark configuration other than the headline.  Short ones first: after the power-capped long runs the
    clocks need a while to recover."""
    combos = [(0, 0), (1, 1), (0, 1), (1, 0)]
    plan = []
    for m in (1, 16, 64, 128):
        plan.append((f"decode_m{m}_8192x8192", m, 8192, 8192, 0, 0, 0, 0))
    plan.append(("decode_m32_n57344_k8192", 32, 8192, 57344, 0, 0, 0, 0))
    for depth in (2, 4, 0):
        plan.append((f"gemm1024_depth{depth}", 1024, 1024, 1024, 0, 0, depth, 0))
    for (fa, fb) in combos:
        for depth in (2, 4, 0):
            plan.append((f"gemm4096_{DTYPE_NAMES[fa]}x{DTYPE_NAMES[fb]}_depth{depth}", 4096, 4096, 4096, fa, fb, depth, 0))
    plan.append(("m256_8192x8192", 256, 8192, 8192, 0, 0, 0, 0))
    plan.append(("m512_8192x8192", 512, 8192, 8192, 0, 0, 0, 0))
    plan.append(("gemm8192", 8192, 8192, 8192, 0, 0, 0, 0))
    plan.append(("ffn_up_8192x8192x28672", 8192, 8192, 28672, 0, 0, 0, 0))
    plan.append(("ffn_down_8192x28672x8192", 8192, 28672, 8192, 0, 0, 0, 0))
    out, t0 = {}, time.perf_counter()
    for idx, (name, M, K, N, fa, fb, depth, kernel) in enumerate(plan):
        if time.perf_counter() - t0 > budget_s:
            out[name] = {"skipped": "time budget of the configs leg spent"}
            continue
        out[name] = measure_config(torch, g, cmp, dev, name, M, K, N, fa, fb, depth, kernel, peaks, seed=2 * idx)
    worst = [r["parity"]["worst"] for r in out.values() if "parity" in r]
    summary = {"rows": len(out), "measured": len(worst), "parity_worst": max(worst) if worst else None,
               "all_within_tolerance": bool(worst) and max(worst) <= 1.0, "seconds": round(time.perf_counter() - t0, 1)}
    return out, summary


def reference_kernels_side(torch, g, dev):
    """The reference's own mma.sync kernels (built unmodified from a scratch copy without its unbuildable kernel 2,
    baseline/Makefile) with the reference driver's protocol (GEMM/gemm_main.cpp:25-26, :69-84: 20 warm-up calls, then
    100 calls each bracketed by events and synchronised, mean).  Time only: the kernels never zero their accumulators
    and write full 128 x 128 tiles only, so their C is not checked.  Ours runs with the same protocol beside them."""
    path = os.path.join(ROOT, "baseline", "_ref", "libref_kernels.so")
    if not os.path.exists(path):
        return {"unavailable": "baseline/_ref/libref_kernels.so is not built (needs the reference checkout at build time)"}
    lib = ctypes.CDLL(path)
    ci, vp = ctypes.c_int, ctypes.c_void_p
    entries = {"kernel1_e4m3xe4m3 (GEMM/src/gemm.cu:29-262)": ("_ZN4gemm4GEMMEiiiPK13__nv_fp8_e4m3S2_Pf", torch.float8_e4m3fn, 1.0),
               "kernel3_e5m2xe5m2 (GEMM/src/gemm.cu:696-921)": ("_ZN4gemm4GEMMEiiiPK13__nv_fp8_e5m2S2_Pf", torch.float8_e5m2, 2.0)}
    out = {"protocol": "20 warm-up calls, 100 calls individually timed with events and synchronised, mean "
                       "(GEMM/gemm_main.cpp:69-84); legacy default stream; results of the reference kernels not checked"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def protocol(call):
        for _ in range(20):
            call()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(100):
            e0.record()
            call()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        return total / 100

    for size in (4096, 8192):
        for label, (sym, dt, sigma) in entries.items():
            fn = getattr(lib, sym)
            fn.argtypes = [ci, ci, ci, vp, vp, vp]
            a = torch.empty((size, size), dtype=dt, device=dev)
            b = torch.empty((size, size), dtype=dt, device=dev)
            c = torch.zeros((size, size), dtype=torch.float32, device=dev)
            g.fill_normal(a, sigma, SEED_BASE + 300)
            g.fill_normal(b, sigma, SEED_BASE + 301)
            torch.cuda.synchronize()
            with torch.cuda.stream(torch.cuda.default_stream(dev)):      # the reference launches on the legacy default stream
                ref_ms = protocol(lambda: fn(size, size, size, a.data_ptr(), b.data_ptr(), c.data_ptr()))
                ours_ms = protocol(lambda: g.GEMM4(size, size, size, a, b, c))
                best_ms = protocol(lambda: g.gemm_ex(a, b, c))
            fl = 2.0 * size ** 3
            out[f"{size}^3 {label}"] = {"reference_ms": ref_ms, "reference_tflops": fl / ref_ms / 1e9,
                                        "ours_GEMM4_ms": ours_ms, "ours_GEMM4_tflops": fl / ours_ms / 1e9,
                                        "ours_auto_depth_ms": best_ms, "ours_auto_depth_tflops": fl / best_ms / 1e9,
                                        "speedup_GEMM4_over_reference": ref_ms / ours_ms}
            del a, b, c
    torch.cuda.empty_cache()
    return out


def fused_epilogue_side(torch, g, dev):
    """The extended epilogue on the 8192^3 shape: FP32 plain store against BF16 output with per-row scales of A and
    of B, bias and GELU (the epilogue of a row-wise quantised linear layer), each as a CUDA graph of 8 launches over two
    B / D sets, three alternating rounds.  Parity of the timed BF16 buffer: sampled full rows against FP64
    (tolerance of the operator scaled by the factors, widened by the activation's slope and BF16 rounding)."""
    import numpy as np
    from oracle import fp8_oracle as fo
    M = K = N = 8192
    iters, nsets = 8, 2
    a = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=dev)
    g.fill_normal(a, 1.0, SEED_BASE + 700)
    bs, c32, d16 = [], [], []
    for i in range(nsets):
        b = torch.empty((N, K), dtype=torch.float8_e4m3fn, device=dev)
        g.fill_normal(b, 1.0, SEED_BASE + 701 + i)
        bs.append(b)
        c32.append(torch.empty((M, N), dtype=torch.float32, device=dev))
        d16.append(torch.empty((M, N), dtype=torch.bfloat16, device=dev))
    gen = torch.Generator(device=dev).manual_seed(SEED_BASE + 710)
    ra = torch.rand(M, generator=gen, device=dev) * 0.02 + 0.001
    rb = torch.rand(N, generator=gen, device=dev) * 0.02 + 0.001
    bias = torch.randn(N, generator=gen, device=dev)

    def graph_of(fn):
        fn(0)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for i in range(iters):
                fn(i)
        return gr.replay

    variants = {
        "f32_plain": graph_of(lambda i: g.gemm_ex(a, bs[i % nsets], c32[i % nsets])),
        "bf16_rowscales_bias_gelu_tanh": graph_of(lambda i: g.gemm_epilogue(
            a, bs[i % nsets], d16[i % nsets], a_row_scale=ra, b_row_scale=rb, bias=bias, activation="gelu_tanh")),
        "bf16_rowscales_bias_gelu_erf": graph_of(lambda i: g.gemm_epilogue(
            a, bs[i % nsets], d16[i % nsets], a_row_scale=ra, b_row_scale=rb, bias=bias, activation="gelu")),
    }
    times = {k: [] for k in variants}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rnd in range(4):
        for name, run in variants.items():
            run()
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            if rnd:
                times[name].append(e0.elapsed_time(e1) / iters)
    out = {"shape": "8192^3 e4m3 x e4m3", "timing": f"CUDA graph of {iters} launches over {nsets} B / D sets, 3 alternating rounds",
           "ms": {k: sum(v) / len(v) for k, v in times.items()}}
    # parity of D buffer 0 as the last timed replay (erf form) left it
    rng = np.random.default_rng(12)
    pick = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 6)]))
    tm = torch.from_numpy(pick).to(dev)
    C64, S = fo.gemm_f64(np.ascontiguousarray(a.view(torch.uint8)[tm].cpu().numpy()), 0, bs[0].view(torch.uint8).cpu().numpy(), 0)
    f = ra[tm].cpu().numpy().astype(np.float64)[:, None] * rb.cpu().numpy().astype(np.float64)[None, :]
    pre = f * C64 + bias.cpu().numpy().astype(np.float64)[None, :]
    from math import sqrt
    from scipy.special import erf
    want = 0.5 * pre * (1.0 + erf(pre / sqrt(2.0)))
    tol = 1.13 * (f * (1e-3 * S + 1e-6) + 2.0 ** -21 * (np.abs(pre) + np.abs(f * C64))) + 2e-6 * np.abs(pre) + 2.0 ** -8 * np.abs(want)
    got = d16[0][tm].float().cpu().numpy().astype(np.float64)
    ratio = np.abs(got - want) / tol
    out["parity"] = {"worst": float(ratio.max()), "elements_outside_tolerance": int((ratio > 1).sum()),
                     "sample": f"{len(pick)} full rows of the timed BF16 buffer against FP64 (scales, bias, GELU by erf)"}
    out["device_status"] = g.device_status()
    return out


def run_sparse(args, g, torch, dev, json_fd):
    """GEMV / blocked-ELL SpMM / SpMV on one GPU: all steps in one CUDA graph over rotating operand sets larger than
    L2; FLOPs and bytes count the STORED blocks only (algorithmic work of the sparse problem)."""
    op, M, K, N, blocks = SPARSE_WORKLOADS[args.workload]
    f8 = torch.float8_e4m3fn
    width = blocks * 128
    gen = torch.Generator(device=dev).manual_seed(SEED_BASE & 0x7FFFFFFF)
    if op == "gemv":
        set_bytes = N * K
    else:
        set_bytes = M * width + (N * K + 4 * M * N if op == "spmm" else 0)
    nsets = max(2, min(8, (1 << 30) // set_bytes))
    sets = []
    for i in range(nsets):
        if op == "gemv":
            b = torch.empty((N, K), dtype=f8, device=dev)
            g.fill_normal(b, 1.0, SEED_BASE + 80 + i)
            sets.append((b, torch.empty(N, dtype=torch.float32, device=dev)))
            continue
        vals = torch.empty((M, width), dtype=f8, device=dev)
        g.fill_normal(vals, 1.0, SEED_BASE + 80 + i)
        ind = torch.rand((M // 128, K // 128), generator=gen, device=dev).argsort(dim=1)[:, :blocks].sort(dim=1).values.int().contiguous()
        if op == "spmm":
            b = torch.empty((N, K), dtype=f8, device=dev)
            g.fill_normal(b, 1.0, SEED_BASE + 90 + i)
            sets.append((vals, ind, b, torch.empty((M, N), dtype=torch.float32, device=dev)))
        else:
            sets.append((vals, ind, torch.empty(M, dtype=torch.float32, device=dev)))
    x = torch.empty(K, dtype=f8, device=dev)
    g.fill_normal(x, 1.0, SEED_BASE + 99)

    def step(i):
        t = sets[i % nsets]
        if op == "spmm":
            g.spmm_bell(t[0], t[1], t[2], t[3], kernel=args.kernel, depth=args.depth)
        elif op == "spmv":
            g.spmv_bell(t[0], t[1], x, t[2])
        else:
            g.gemv(t[0], x, t[1])

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    launches0 = g.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(i)
    launches = g.launch_count() - launches0
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(dev.index)) as clk:
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
    if g.device_status() != 0:
        raise SystemExit("device status word is non-zero: a kernel's bounded wait ran out")
    ms = e0.elapsed_time(e1) / args.steps
    peaks = measured_peaks()
    if op == "spmm":
        flops = 2.0 * M * N * width
        nbytes = float(M * width + N * K + 4 * M * N + 4 * (M // 128) * blocks)
    elif op == "spmv":
        flops = 2.0 * M * width
        nbytes = float(M * width + K + 4 * M + 4 * (M // 128) * blocks)
    else:
        flops = 2.0 * N * K
        nbytes = float(N * K + K + 4 * N)
    tflops = flops / (ms * 1e-3) / 1e12
    if op == "spmm":
        peak = 2.0 * peaks["bf16_sustained"]
        roof = {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                "peak_source": peaks["source"] + ": 2 x sustained cuBLAS bf16", "traffic": None}
    else:
        gbs = nbytes / (ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                "peak_source": peaks["source"] + " (copy bandwidth)", "traffic": None}
    roof.update({"algorithmic_bytes": nbytes, "algorithmic_flops": flops, "kernel_ms": ms})
    line = {"metric": "fp8_gemm_tflops", "value": tflops, "unit": "TFLOPS", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8", "data": "synthetic",
            "config": {"workload": args.workload, "op": op, "M": M, "K": K, "N": N, "ell_block": 128,
                       "stored_blocks_per_block_row": blocks, "block_columns": K // 128, "a": "e4m3", "b": "e4m3",
                       "out": "f32", "l2": f"rotating over {nsets} distinct operand sets larger than L2",
                       "timing": "one CUDA graph of all steps, replayed", "flops": "stored blocks only"},
            "roofline": roof, "gpu_launches": int(launches), "clocks": clk.summary(), "e2e": None, "cpu_baseline": None}
    os.write(json_fd, (json.dumps(line) + "\n").encode())
    return 0


def run_phase_timeline(args, g, torch, dev, json_fd, pkg):
    """Where one launch spends its time, from the kernels' own %globaltimer stamps: the phases of the M <= 128 kernels
    (B200FP8_DEBUG=1024), or the epilogue chain of the tile kernels (M > 128 workloads, B200FP8_DEBUG=4096).  Needs the
    diagnostics build of the library (make -C tensor-core-fp8_b200/csrc diag; B200FP8_LIBRARY points at it): the product
    build has no such code."""
    import numpy as np
    lib = pkg._cabi.lib()
    if not hasattr(lib, "b200fp8_debug_trace_copy"):
        raise SystemExit("--phase-timeline needs the diagnostics build: B200FP8_LIBRARY=.../libb200fp8_diag.so B200FP8_DEBUG=1024")
    lib.b200fp8_debug_trace_copy.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.c_int, ctypes.c_int]
    M, K, N, _ = WORKLOADS[args.workload]
    if M > 128:
        # tile kernels (B200FP8_DEBUG=4096): the epilogue chain of CTA 0's first epilogue warp on its last work item --
        # accumulator complete, then per 32-column chunk: in registers / staging box free / staged / fenced / store issued,
        # finally: last store has read its box / all stores complete -- nanoseconds after the first stamp
        f8 = torch.float8_e4m3fn
        a = torch.empty((M, K), dtype=f8, device=dev)
        b = torch.empty((N, K), dtype=f8, device=dev)
        g.fill_normal(a, 1.0, 1)
        g.fill_normal(b, 1.0, 2)
        c = torch.empty((M, N), dtype=torch.float32, device=dev)
        for _ in range(3):
            g.gemm_ex(a, b, c, kernel=args.kernel, depth=args.depth)
        torch.cuda.synchronize()
        buf = (ctypes.c_longlong * 64)()
        lib.b200fp8_debug_trace_copy(buf, 64, 1)
        g.gemm_ex(a, b, c, kernel=args.kernel, depth=args.depth)
        torch.cuda.synchronize()
        lib.b200fp8_debug_trace_copy(buf, 64, 1)
        t = [int(x) for x in buf[:32] if x > 0]
        line = {"epilogue_chain_ns": [x - t[0] for x in t] if t else [],
                "config": {"workload": args.workload, "M": M, "K": K, "N": N, "kernel": args.kernel, "depth": args.depth},
                "stamps": "accumulator complete; per chunk: [in registers (even chunks),] box free, staged, fenced, issued; "
                          "last store has read its box; all stores complete"}
        os.write(json_fd, (json.dumps(line) + "\n").encode())
        return 0
    kernel = args.kernel or 4
    names = {4: ["entry", "set-up done", "first block in shared memory", "accumulator complete", "epilogue woke",
                 "first cluster barrier passed", "reduce-scatter + stores done", "end"],
             8: ["entry", "grid dependency wait passed", "first block in shared memory", "MMA warp done",
                 "finisher saw its peers' flags", "finisher's first bulk copy landed", "epilogue done", "end"]}.get(kernel)
    if names is None:
        raise SystemExit("--phase-timeline of an M <= 128 workload takes --kernel 4 or 8")
    f8 = torch.float8_e4m3fn
    a = torch.empty((M, K), dtype=f8, device=dev)
    g.fill_normal(a, 1.0, 1)
    bs = [torch.empty((N, K), dtype=f8, device=dev) for _ in range(6)]
    for i, b in enumerate(bs):
        g.fill_normal(b, 1.0, 2 + i)
    c = torch.empty((M, N), dtype=torch.float32, device=dev)
    for i in range(3):
        g.gemm_ex(a, bs[i], c, kernel=kernel)
    torch.cuda.synchronize()
    words = 3 * 4096
    buf = (ctypes.c_longlong * words)()
    lib.b200fp8_debug_trace_copy(buf, words, 1)
    g.gemm_ex(a, bs[3], c, kernel=kernel)      # two launches back to back: the stamps kept are the second launch's,
    g.gemm_ex(a, bs[4], c, kernel=kernel)      # which started under the first one's tail (dependent launch)
    torch.cuda.synchronize()
    nw = lib.b200fp8_debug_trace_copy(buf, words, 1)
    t = np.array(buf[:nw], dtype=np.int64).reshape(-1, 8)
    t = t[t[:, 0] > 0]
    t0 = t[:, 0].min()
    rows = {}
    for i, nm in enumerate(names):
        col = t[:, i][t[:, i] > 0]
        if nm and len(col):
            rows[nm] = {"median_us": float(np.median(col - t0)) / 1e3, "min_us": float(col.min() - t0) / 1e3,
                        "max_us": float(col.max() - t0) / 1e3, "ctas": int(len(col))}
    line = {"phase_timeline": rows, "config": {"workload": args.workload, "M": M, "K": K, "N": N, "kernel": kernel},
            "ctas": int(len(t)), "unit": "microseconds after the first CTA's entry"}
    os.write(json_fd, (json.dumps(line) + "\n").encode())
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="shard32768", choices=sorted(WORKLOADS) + sorted(SPARSE_WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the configs / reference-kernel / collective legs")
    ap.add_argument("--no-parity", action="store_true", help="skip the check of the timed C buffer")
    ap.add_argument("--multimem", action="store_true", help="fused all-gather through NVSwitch multicast only (multimem stores)")
    ap.add_argument("--phase-timeline", action="store_true", help="kernel time stamps of one launch (diagnostics build)")
    ap.add_argument("--kernel", type=int, default=0)
    ap.add_argument("--depth", type=int, default=0)
    ap.add_argument("--a-dtype", default="e4m3", choices=["e4m3", "e5m2"])
    ap.add_argument("--b-dtype", default="e4m3", choices=["e4m3", "e5m2"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)

    # Only the final JSON line may reach stdout: libraries (NCCL's version banner for one) write there too,
    # so everything else on file descriptor 1 goes to stderr until the line is printed.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # the launcher exports OMP_NUM_THREADS=1; the parity checks run the FP64 oracle on the host, so every rank
        # gets its share of the host threads instead (set before any OpenMP runtime is loaded)
        os.environ["OMP_NUM_THREADS"] = str(max(1, host_threads() // world))

    import datetime
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    g = pkg.gemm
    shard_mod = pkg.shard

    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.workload in SPARSE_WORKLOADS:
        if world > 1:
            raise SystemExit("the sparse workloads run on one GPU")
        return run_sparse(args, g, torch, dev, json_fd)
    if args.phase_timeline:
        return run_phase_timeline(args, g, torch, dev, json_fd, pkg)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at NCCL_DEBUG=VERSION
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    M, K, N, sharded = WORKLOADS[args.workload]
    sh = shard_mod.column_shard(N, rank, world) if sharded else shard_mod.Shard(rank, world, 0, N)
    n_local = sh.n
    seed_a, seed_b = SEED_BASE + 64, SEED_BASE + 65
    f8_of = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
    fa, fb = f8_of[args.a_dtype], f8_of[args.b_dtype]
    sig_a, sig_b = (1.0 if args.a_dtype == "e4m3" else 2.0), (1.0 if args.b_dtype == "e4m3" else 2.0)
    peaks = measured_peaks()

    # operands: several B (and C) buffers for small workloads so that every step reads from HBM, not L2
    nsets = operand_sets(M, K, n_local)
    a = torch.empty((M, K), dtype=fa, device=dev)
    g.fill_normal(a, sig_a, seed_a)
    bs, cs = [], []
    for i in range(nsets):
        b = torch.empty((n_local, K), dtype=fb, device=dev)
        g.fill_normal(b, sig_b, seed_b + 1000 * i, index_offset=sh.n_begin * K)
        bs.append(b)
        cs.append(torch.empty((M, n_local), dtype=torch.float32, device=dev))
    torch.cuda.synchronize()

    def step(i):
        g.gemm_ex(a, bs[i % nsets], cs[i % nsets], depth=args.depth, kernel=args.kernel)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(args.warmup):
        step(i)
    barrier()
    use_graph = graph_timed(M, K, n_local)
    launches0 = g.launch_count()
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.steps):
                step(i)
        launches = g.launch_count() - launches0          # kernel nodes in the graph = launches per replay
        graph.replay()
        barrier()
        e_beg, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(physical_gpu_index(local_rank)) as clk:
            e_beg.record()
            graph.replay()
            e_end.record()
            torch.cuda.synchronize()
        barrier()
        total_ms = e_beg.elapsed_time(e_end)
        per_launch_ms = [total_ms / args.steps] * args.steps
    else:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        with ClockSampler(physical_gpu_index(local_rank)) as clk:
            ev[0].record()
            for i in range(args.steps):
                step(i)
                ev[i + 1].record()
            torch.cuda.synchronize()
        launches = g.launch_count() - launches0
        barrier()
        total_ms = ev[0].elapsed_time(ev[-1])
        per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    if g.device_status() != 0:
        raise SystemExit("device status word is non-zero: a kernel's bounded wait ran out")
    max_ms = max_over_ranks(total_ms)
    ms_per_step = max_ms / args.steps

    replicas = 1 if sharded else world
    flops_job = 2.0 * M * K * N * replicas                      # per step, all ranks together
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # roofline of the dominant kernel on this rank
    flops_launch = 2.0 * M * K * n_local
    bytes_launch = float(M * K + n_local * K + 4 * M * n_local)
    avg_launch_ms = sum(per_launch_ms) / len(per_launch_ms)
    hbm_bound = M <= 128
    if hbm_bound:
        ach = bytes_launch / (avg_launch_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (copy bandwidth)",
                "frac_of_nominal_8TBs": ach / NOMINAL_HBM_GBS}
    else:
        ach = flops_launch / (avg_launch_ms * 1e-3) / 1e12
        # a timed region of at least a few hundred milliseconds runs at the power cap: the sustained figure applies
        sustained = total_ms >= 200.0
        peak = 2.0 * (peaks["bf16_sustained"] if sustained else peaks["bf16_burst"])
        roof = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "peak_source": peaks["source"] + (": 2 x sustained cuBLAS bf16" if sustained else ": 2 x burst cuBLAS bf16 (timed region shorter than 0.2 s)")
                               + " (fp8 issues at twice the bf16 rate)",
                "frac_of_sustained_peak": ach / (2.0 * peaks["bf16_sustained"]),
                "frac_of_burst_peak": ach / (2.0 * peaks["bf16_burst"]),
                "frac_of_nominal_4500": ach / NOMINAL_FP8_TFLOPS}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None   # captured at N = 1
    roof["algorithmic_bytes"] = bytes_launch
    roof["algorithmic_flops"] = flops_launch
    roof["kernel_ms"] = avg_launch_ms

    line = {
        "metric": "fp8_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": workload_config(args, M, K, N, n_local, world, sharded, describe_l2(nsets),
                                  "one CUDA graph of all steps, replayed" if use_graph else "launch by launch"),
        "roofline": roof, "gpu_launches": int(launches), "clocks": clk.summary(),
        "pct_of_nominal_fp8_peak": 100.0 * value / (NOMINAL_FP8_TFLOPS * world),
    }

    # ---- the buffer that was timed, checked (every rank checks its own block; the worst over ranks is reported) ----
    if not args.no_parity:
        p = parity_of(torch, g, a, bs[0], cs[0], rows=8 if world == 1 else 4, cols=8 if world == 1 else 4, points=4096 if world == 1 else 2048)
        p["worst"] = max_over_ranks(p["worst"])
        p["buffer"] = "C of the timed steps (every rank its own column block; worst over ranks)"
        line["parity"] = p
        if p["worst"] > 1.0:
            raise SystemExit(f"the timed C buffer is outside the tolerance: {p}")

    # ---- N > 1: a steady-state leg.  The counted steps above last a few milliseconds per rank at N = 8 and never reach
    #      the power-capped clocks the N = 1 run sits at, so 1 -> N would compare two power regimes: here every rank runs
    #      back to back for at least a second, and the per-GPU rate comes with the SM clock it was measured at ----
    if world > 1 and not args.no_extras:
        per = max(avg_launch_ms, 1e-3)
        reps = int(min(2000, max(args.steps, 1100.0 / per)))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with ClockSampler(physical_gpu_index(local_rank)) as sclk:
            e0.record()
            for i in range(reps):
                step(i)
            e1.record()
            torch.cuda.synchronize()
        barrier()
        sus_ms = max_over_ranks(e0.elapsed_time(e1)) / reps
        mhz = sclk.summary()["sm_mhz"]
        mhz_max = max_over_ranks(float(mhz or 0))
        mhz_min = -max_over_ranks(-float(mhz or 0))
        line["sustained"] = {"steps": reps, "ms_per_step": sus_ms, "tflops_per_gpu": flops_launch / sus_ms / 1e9,
                             "tflops_job": flops_job / sus_ms / 1e9, "median_sm_mhz_rank0": mhz,
                             "median_sm_mhz_over_ranks": [mhz_min, mhz_max], "reasons_rank0": sclk.summary()["reasons"],
                             "ms_times_mhz_rank0": (sus_ms * mhz) if mhz else None,
                             "frac_of_sustained_peak": flops_launch / sus_ms / 1e9 / (2.0 * peaks["bf16_sustained"]),
                             "note": "max over ranks; compare with the N = 1 line's ms_per_step x clocks.sm_mhz"}

    # ---- end to end from pinned HOST buffers: uploads, operator and the download of C inside the timed region.
    #      N = 1: the C ABI's host-pointer entry point.  N > 1 (sharded): every rank uploads M/N rows of A and its
    #      rows of B, the rows of A go round over NVLink, C blocks are downloaded while the next block computes. ----
    if not args.no_e2e:
        hb = torch.empty((n_local, K), dtype=torch.uint8).pin_memory().view(fb)
        hc = torch.empty((M, n_local), dtype=torch.float32).pin_memory()
        hb.view(torch.uint8).copy_(bs[0].view(torch.uint8))
        sharded_e2e = world > 1 and sharded and M % world == 0
        phases = None
        if sharded_e2e:
            rows = M // world
            ha = torch.empty((rows, K), dtype=torch.uint8).pin_memory().view(fa)
            ha.view(torch.uint8).copy_(a[rank * rows:(rank + 1) * rows].view(torch.uint8))
            runner = shard_mod.HostShardedGemm(M, K, sh, fa, fb, dev, col_blocks=int(os.environ.get("B200FP8_E2E_COL_BLOCKS", "4")))
            call = lambda **kw: runner(ha, hb, hc, depth=args.depth, kernel=args.kernel, **kw)
            api = ("shard.HostShardedGemm (upload M/N rows of A and the B shard; rows of A broadcast rank by rank over NVLink; "
                   "the own rows against the B shard piece by piece as it lands, the other row blocks as their rows arrive; download of C overlapped), wall clock, max over ranks")
            h2d = rows * K + n_local * K
        else:
            ha = torch.empty((M, K), dtype=torch.uint8).pin_memory().view(fa)
            ha.view(torch.uint8).copy_(a.view(torch.uint8))
            call = lambda **kw: g.gemm_host(ha, hb, hc, depth=args.depth)
            api = "b200fp8_gemm_rowcol_f32_host (upload A, B; operator; download C), wall clock, max over ranks"
            h2d = M * K + n_local * K
        call()                                                   # warm-up: allocates device buffers
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            call()
        e2e_ms = (time.perf_counter() - t0) * 1e3               # each call returns when C is in host memory
        e2e_ms = max_over_ranks(e2e_ms) / args.e2e_steps
        if sharded_e2e:
            barrier()
            phases = call(breakdown=True)                        # one more call, with device time stamps per phase
            phases = {k: max_over_ranks(v) for k, v in phases.items()}
            barrier()
        # the downloaded block must be the operator's result: bit for bit the device-resident C of the timed steps
        same = bool(torch.equal(hc[:2048].to(dev), cs[0][:2048]) and torch.equal(hc[-2048:].to(dev), cs[0][-2048:]))
        if not same:
            raise SystemExit("end-to-end result differs from the device-resident result")
        line["e2e"] = {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                       "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(4 * M * n_local),
                       "ms_per_step": e2e_ms, "steps": args.e2e_steps, "api": api,
                       "parity": "first and last 2048 rows of the downloaded C equal the device-resident C of the timed steps bit for bit"}
        if phases is not None:
            line["e2e"]["phase_end_ms"] = phases
            line["e2e"]["phase_note"] = "device time stamps of one more call, milliseconds after its start, max over ranks"
        del ha, hb, hc
        if sharded_e2e:
            del runner
        if world == 1:
            pkg._cabi.lib().b200fp8_host_release()
        torch.cuda.empty_cache()

    # ---- N > 1: the all-gather of the C blocks, separately (NCCL) and fused into the GEMM's epilogue ----
    if world > 1 and sharded and not args.no_extras:
        recv_bytes = 4.0 * M * n_local * (world - 1)
        full = torch.empty((world, M, n_local), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(full, cs[0])
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            dist.all_gather_into_tensor(full, cs[0])
        e1.record()
        torch.cuda.synchronize()
        ag_ms = max_over_ranks(e0.elapsed_time(e1) / reps)
        own_ok = bool(torch.equal(full[rank], cs[0]))
        line["allgather"] = {"ms": ag_ms, "bytes_received_per_rank": int(recv_bytes), "gbs_received_per_gpu": recv_bytes / ag_ms / 1e6,
                             "frac_of_measured_nvlink": recv_bytes / ag_ms / 1e6 / NVLINK_PEER_COPY_GBS,
                             "layout": "[rank][M][N/R] blocks (a re-layout pass would still be needed for row-major C)",
                             "gemm_plus_allgather_ms": ms_per_step + ag_ms, "parity": {"own_block_bitwise": own_ok}}
        barrier()
        variants = [("fused_allgather_multimem", True)] if args.multimem else [("fused_allgather", False), ("fused_allgather_multimem", True)]
        # reference for the parity of the gathered matrix: the unsharded operator on a row block, computed here
        rb = 1024
        b_full = torch.empty((N, K), dtype=fb, device=dev)
        g.fill_normal(b_full, sig_b, seed_b)
        want_rows = torch.empty((rb, N), dtype=torch.float32, device=dev)
        g.gemm_ex(a[:rb], b_full, want_rows, depth=args.depth, kernel=args.kernel)
        torch.cuda.synchronize()
        for key, mc in variants:
            shared = None
            entry = {}
            try:
                try:
                    shared = shard_mod.SharedC(M, N, dev, multicast=mc)
                except RuntimeError as e:
                    if mc and "multicast" in str(e):
                        entry = {"unavailable": "no NVLink multicast for symmetric memory on this system"}
                    else:
                        raise
                if shared is not None:
                    shared.own.fill_(float("nan"))
                    fsteps = max(3, min(args.steps, 10))
                    for _ in range(2):
                        shard_mod.gemm_allgather(a, bs[0], shared, sh, N, depth=args.depth, kernel=args.kernel)
                    barrier()
                    e0.record()
                    for _ in range(fsteps):
                        shard_mod.gemm_allgather(a, bs[0], shared, sh, N, depth=args.depth, kernel=args.kernel)
                    e1.record()
                    torch.cuda.synchronize()
                    barrier()
                    fms = max_over_ranks(e0.elapsed_time(e1) / fsteps)
                    status = g.device_status()
                    # parity of the gathered matrix on THIS rank: a row block against the unsharded operator (bitwise),
                    # and sampled points of the whole matrix against the FP64 oracle
                    rows_equal = bool(torch.equal(shared.own[:rb], want_rows))
                    import numpy as np
                    from oracle import fp8_oracle as fo
                    rng = np.random.default_rng(100 + rank)
                    pm, pn = rng.integers(0, M, 1024), rng.integers(0, N, 1024)
                    C64, S = fo.gemm_f64_points(a.view(torch.uint8).cpu().numpy(), g.dtype_code(a),
                                                b_full.view(torch.uint8).cpu().numpy(), g.dtype_code(b_full), pm, pn)
                    got = shared.own[torch.from_numpy(pm).to(dev), torch.from_numpy(pn).to(dev)].cpu().numpy()
                    nbad, w, _ = fo.check_tolerance(got, C64, S)
                    ok_all = max_over_ranks(0.0 if (rows_equal and nbad == 0 and status == 0) else 1.0) == 0.0
                    sent = 4.0 * M * n_local * (1 if mc else world - 1)
                    entry = {"ms_per_step": fms, "tflops": 2.0 * M * K * N / (fms * 1e-3) / 1e12, "steps": fsteps,
                             "stores": "multimem (NVSwitch multicast)" if mc else "unicast peer stores",
                             "nvlink_bytes_sent_per_rank": int(sent), "bytes_received_per_rank": int(recv_bytes),
                             "gbs_received_per_gpu": recv_bytes / fms / 1e6,
                             "frac_of_measured_nvlink": recv_bytes / fms / 1e6 / NVLINK_PEER_COPY_GBS,
                             "roofline_ms": max(flops_launch / (2.0 * peaks["bf16_sustained"]) / 1e9, recv_bytes / NVLINK_PEER_COPY_GBS / 1e6),
                             "vs_gemm_plus_nccl_allgather": (ms_per_step + ag_ms) / fms,
                             "result": "every rank holds the full row-major C; no separate collective, no re-layout",
                             "parity": {"rows_0_1023_bitwise_equal_unsharded_operator": rows_equal, "oracle_points": 1024,
                                        "oracle_worst": max_over_ranks(float(w)), "device_status": status, "all_ranks_ok": ok_all}}
            finally:
                if shared is not None:
                    shared.close()                               # collective; reached on every rank whatever happened above
            line[key] = entry
        del full, b_full, want_rows
        torch.cuda.empty_cache()

    # ---- N = 1, default workload: the other configurations and the comparator arms ----
    if rank == 0 and world == 1 and not args.no_extras:
        del a, bs, cs
        torch.cuda.empty_cache()
        cmp = Comparator(pkg._cabi.CMP_LIB_PATH)
        if args.workload == "shard32768":
            line["configs"], line["configs_summary"] = run_configs(torch, g, cmp, dev, peaks)
        else:
            code = {"e4m3": 0, "e5m2": 1}
            line["configs"] = {args.workload: measure_config(torch, g, cmp, dev, args.workload, M, K, N, code[args.a_dtype],
                                                             code[args.b_dtype], args.depth, args.kernel, peaks)}
        line["side"] = {"reference_kernels": reference_kernels_side(torch, g, dev)}
        if args.workload == "shard32768":
            line["side"]["fused_epilogue"] = fused_epilogue_side(torch, g, dev)

    # ---- the reference's CPU loop timed on this box's host cores (rank 0, N = 1 only) ----
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r, threads, sample, dt = cpu_reference_rate(M, K, N, 1024, seed_a, seed_b)
        line["cpu_baseline"] = {"value": r, "unit": "TFLOPS", "cores": threads, "kind": "port",
                                "sample": sample + f", {dt:.1f} s; the reference's float loop "
                                "(GEMM/gemm_main.cpp:45-52) restated in oracle/fp8_oracle.c, OpenMP over rows"}
        ref_loop = reference_binary_rate()
        if ref_loop is not None:                  # the reference's own binary, single thread as it ships
            line["cpu_baseline"]["reference_loop"] = ref_loop

    if rank == 0:
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
