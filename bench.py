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
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised under profiles/
NCU_TRAFFIC_BYTES = {
    "shard32768": 30.11e9,   # profiles/gemm_fp8_rowcol_kernel__shard32768__launch_list_and_dram.md
    "gemm8192": 537.6e6,     # profiles/gemm_fp8_rowcol_kernel__gemm8192__full_set.md
    "skinny16": 67.8e6,      # profiles/gemm_fp8_skinny_kernel__skinny16__full_set.md
}


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


def cpu_reference_rate(M, K, N, rows_per_thread: int, seed_a: int, seed_b: int):
    """The reference's CPU loop (oracle port) on a bounded sample: returns (TFLOPS, threads, description, seconds)."""
    import numpy as np
    from oracle import fp8_oracle as fo
    threads = fo.max_threads()
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    if args.workload in SPARSE_WORKLOADS:       # the CPU loop has no sparse form: the dense problem of the same shape
        M, K, N, sharded = SPARSE_WORKLOADS[args.workload][1:4] + (False,)
    else:
        M, K, N, sharded = WORKLOADS[args.workload]
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
        "config": {"workload": args.workload, "M": M, "K": K, "N": N, "layout": "row-col", "a": "e4m3", "b": "e4m3",
                   "out": "f32"},
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
    ap.add_argument("--no-extras", action="store_true", help="skip the cuBLASLt / 8192^3 side measurements")
    ap.add_argument("--allgather", action="store_true", help="also time an NCCL all-gather of the C shards (N > 1)")
    ap.add_argument("--fused-allgather", action="store_true",
                    help="also time the GEMM with the all-gather fused into its epilogue (N > 1): every rank ends with all of C")
    ap.add_argument("--multimem", action="store_true", help="fused all-gather through NVSwitch multicast (multimem stores)")
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

    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    g = pkg.gemm
    shard_mod = pkg.shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
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
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at NCCL_DEBUG=VERSION
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)

    M, K, N, sharded = WORKLOADS[args.workload]
    sh = shard_mod.column_shard(N, rank, world) if sharded else shard_mod.Shard(rank, world, 0, N)
    n_local = sh.n
    seed_a, seed_b = SEED_BASE + 64, SEED_BASE + 65
    f8_of = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
    fa, fb = f8_of[args.a_dtype], f8_of[args.b_dtype]
    sig_a, sig_b = (1.0 if args.a_dtype == "e4m3" else 2.0), (1.0 if args.b_dtype == "e4m3" else 2.0)
    f8 = torch.float8_e4m3fn

    # operands: several B (and C) buffers for small workloads so that every step reads from HBM, not L2
    bytes_per_set = n_local * K + 4 * M * n_local
    nsets = 1 if (M * K + bytes_per_set) > (512 << 20) else max(2, min(8, (1 << 30) // max(1, bytes_per_set)))
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

    for i in range(args.warmup):
        step(i)
    barrier()
    # Short steps are launch-bound when driven call by call from Python, so their K steps are captured
    # once in a CUDA graph and replayed; long steps are timed launch by launch.
    use_graph = 2.0 * M * K * n_local < 2e12
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
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_ms = float(t.item())
    ms_per_step = max_ms / args.steps

    replicas = 1 if sharded else world
    flops_job = 2.0 * M * K * N * replicas                      # per step, all ranks together
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # roofline of the dominant kernel on this rank
    peaks = measured_peaks()
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
        peak = 2.0 * peaks["bf16_sustained"]
        roof = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "peak_source": peaks["source"] + ": 2 x sustained cuBLAS bf16 (fp8 issues at twice the bf16 rate)",
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
        "config": {"workload": args.workload, "M": M, "K": K, "N": N, "n_per_rank": n_local, "layout": "row-col",
                   "a": args.a_dtype, "b": args.b_dtype, "out": "f32", "parallelism": f"n-shard x{world}" if sharded else f"replicas x{world}",
                   "l2": "inputs larger than L2" if nsets == 1 else f"rotating over {nsets} distinct B/C buffer sets larger than L2",
                   "kernel": args.kernel, "depth": args.depth,
                   "timing": "one CUDA graph of all steps, replayed" if use_graph else "launch by launch"},
        "roofline": roof, "gpu_launches": int(launches), "clocks": clk.summary(),
        "pct_of_nominal_fp8_peak": 100.0 * value / (NOMINAL_FP8_TFLOPS * world),
    }

    # ---- end to end from pinned HOST buffers: uploads, operator and the download of C inside the timed region.
    #      N = 1: the C ABI's host-pointer entry point.  N > 1 (sharded): every rank uploads M/N rows of A and its
    #      rows of B, A is all-gathered over NVLink, C blocks are downloaded while the next block computes. ----
    if not args.no_e2e:
        hb = torch.empty((n_local, K), dtype=torch.uint8).pin_memory().view(fb)
        hc = torch.empty((M, n_local), dtype=torch.float32).pin_memory()
        hb.view(torch.uint8).copy_(bs[0].view(torch.uint8))
        sharded_e2e = world > 1 and sharded and M % world == 0
        if sharded_e2e:
            rows = M // world
            ha = torch.empty((rows, K), dtype=torch.uint8).pin_memory().view(fa)
            ha.view(torch.uint8).copy_(a[rank * rows:(rank + 1) * rows].view(torch.uint8))
            runner = shard_mod.HostShardedGemm(M, K, sh, fa, fb, dev)
            call = lambda: runner(ha, hb, hc, depth=args.depth, kernel=args.kernel)
            api = ("shard.HostShardedGemm (upload M/N rows of A and the B shard; NCCL all-gather of A; operator in row "
                   "blocks; download of C overlapped), wall clock, max over ranks")
            h2d = rows * K + n_local * K
        else:
            ha = torch.empty((M, K), dtype=torch.uint8).pin_memory().view(fa)
            ha.view(torch.uint8).copy_(a.view(torch.uint8))
            call = lambda: g.gemm_host(ha, hb, hc, depth=args.depth)
            api = "b200fp8_gemm_rowcol_f32_host (upload A, B; operator; download C), wall clock, max over ranks"
            h2d = M * K + n_local * K
        call()                                                   # warm-up: allocates device buffers
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            call()
        e2e_ms = (time.perf_counter() - t0) * 1e3               # each call returns when C is in host memory
        tt = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item()) / args.e2e_steps
        if sharded_e2e:                                          # the downloaded block must be the operator's result
            if not torch.equal(hc[:4096].to(dev), cs[0][:4096]):
                raise SystemExit("end-to-end result differs from the device-resident result")
        line["e2e"] = {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                       "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(4 * M * n_local),
                       "ms_per_step": e2e_ms, "steps": args.e2e_steps, "api": api}
        del ha, hb, hc

    # ---- optional NCCL all-gather of the C shards, timed separately ----
    if args.allgather and world > 1 and sharded:
        full = torch.empty((world, M, n_local), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(full, cs[0])
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.all_gather_into_tensor(full, cs[0])
        e1.record()
        torch.cuda.synchronize()
        tg = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        line["allgather"] = {"ms": float(tg.item()), "bytes_received_per_rank": int(4 * M * n_local * (world - 1)),
                             "layout": "[rank][M][N/R] blocks"}
        del full

    # ---- the same step with the all-gather of C fused into the kernel's epilogue (peer stores over NVLink) ----
    if args.fused_allgather and world > 1 and sharded:
        shared = shard_mod.SharedC(M, N, dev, multicast=args.multimem)
        fsteps = max(3, min(args.steps, 10))
        for _ in range(2):
            shard_mod.gemm_allgather(a, bs[0], shared, sh, N, depth=args.depth, kernel=args.kernel)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(fsteps):
            shard_mod.gemm_allgather(a, bs[0], shared, sh, N, depth=args.depth, kernel=args.kernel)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        tf = torch.tensor([e0.elapsed_time(e1) / fsteps], dtype=torch.float64, device=dev)
        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
        fms = float(tf.item())
        line["fused_allgather"] = {"ms_per_step": fms, "tflops": 2.0 * M * K * N / (fms * 1e-3) / 1e12, "steps": fsteps,
                                   "stores": "multimem (NVSwitch multicast)" if args.multimem else "unicast peer stores",
                                   "nvlink_bytes_sent_per_rank": int(4 * M * n_local * (1 if args.multimem else world - 1)),
                                   "result": "every rank holds the full row-major C; no separate collective, no re-layout"}
        if g.device_status() != 0:
            raise SystemExit("device status word is non-zero after the fused run")
        shared.close()

    # ---- side measurements on rank 0 at N = 1: the 8192^3 target shape and the bench workload, ours against
    #      cuBLASLt on the same buffers, ALTERNATING so that both see the same clocks and temperature ----
    if rank == 0 and world == 1 and not args.no_extras:
        extras = {}
        cmp_path = pkg._cabi.CMP_LIB_PATH
        cmp = ctypes.CDLL(cmp_path) if os.path.exists(cmp_path) else None
        ci, vp, fp = ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)
        if cmp is not None:
            cmp.b200fp8_cmp_cublaslt.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, ci, ci, fp, ctypes.POINTER(ci), vp]
            cmp.b200fp8_cmp_cublaslt_run.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, fp, vp]
        stream = torch.cuda.current_stream().cuda_stream
        # a short workload goes first: after the power-capped 8192^3 runs the clocks need a while to recover
        order = (args.workload, "gemm8192") if 2.0 * M * K * n_local < 2e12 else ("gemm8192", args.workload)
        for name in order:
            if name in extras:
                continue
            m2, k2, n2, _ = WORKLOADS[name]
            if name == args.workload:
                a2, b2, c2 = a, bs[0], cs[0]
                n2 = n_local
            else:
                a2 = torch.empty((m2, k2), dtype=f8, device=dev)
                b2 = torch.empty((n2, k2), dtype=f8, device=dev)
                c2 = torch.empty((m2, n2), dtype=torch.float32, device=dev)
                g.fill_normal(a2, 1.0, seed_a + 7)
                g.fill_normal(b2, 1.0, seed_b + 7)
            fl = 2.0 * m2 * k2 * n2
            # every round: a lead-in that is not timed (the clocks settle to THIS kernel's steady state: a power-capped
            # GPU carries the other kernel's clocks over the switch), then the timed launches
            iters, lead = (20, 20) if fl < 5e12 else (6, 3)
            have_cmp = False
            if cmp is not None:
                ms = ctypes.c_float(-1)
                found = ci(0)
                have_cmp = cmp.b200fp8_cmp_cublaslt(m2, k2, n2, a2.data_ptr(), g.dtype_code(a2), b2.data_ptr(), g.dtype_code(b2), c2.data_ptr(), 3, 8, 0,
                                                    ctypes.byref(ms), ctypes.byref(found), stream) == 0
            ours, theirs = [], []
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # short kernels: both sides as CUDA graphs of `iters` launches (no launch gaps on either side) over the
            # workload's rotating operand sets (every launch streams from HBM); long ones launch by launch
            side_graph = their_graph = None
            rot_b, rot_c = (bs, cs) if name == args.workload else ([b2], [c2])
            if fl < 2e12:
                for i in range(2):
                    g.gemm_ex(a2, rot_b[i % len(rot_b)], rot_c[i % len(rot_c)], depth=args.depth, kernel=args.kernel)
                torch.cuda.synchronize()
                side_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(side_graph):
                    for i in range(iters):
                        g.gemm_ex(a2, rot_b[i % len(rot_b)], rot_c[i % len(rot_c)], depth=args.depth, kernel=args.kernel)
                if have_cmp:
                    cmp.b200fp8_cmp_cublaslt_enqueue.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, vp]
                    their_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(their_graph):
                        cap = torch.cuda.current_stream().cuda_stream
                        for i in range(iters):
                            cmp.b200fp8_cmp_cublaslt_enqueue(m2, k2, n2, a2.data_ptr(), g.dtype_code(a2), rot_b[i % len(rot_b)].data_ptr(),
                                                             g.dtype_code(b2), rot_c[i % len(rot_c)].data_ptr(), cap)

            def ours_launches(count):
                if side_graph is not None:
                    side_graph.replay()                   # the graph holds `iters` (= lead) launches
                else:
                    for _ in range(count):
                        g.gemm_ex(a2, b2, c2, depth=args.depth, kernel=args.kernel)

            for rnd in range(4):
                ours_launches(lead)
                e0.record()
                ours_launches(iters)
                e1.record()
                torch.cuda.synchronize()
                if rnd:                                   # the first pass warms both up
                    ours.append(e0.elapsed_time(e1) / iters)
                if their_graph is not None:
                    their_graph.replay()
                    e0.record()
                    their_graph.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    if rnd:
                        theirs.append(e0.elapsed_time(e1) / iters)
                elif have_cmp:
                    ms = ctypes.c_float(-1)
                    cmp.b200fp8_cmp_cublaslt_run(m2, k2, n2, a2.data_ptr(), g.dtype_code(a2), b2.data_ptr(), g.dtype_code(b2), c2.data_ptr(), lead,
                                                 ctypes.byref(ms), stream)
                    cmp.b200fp8_cmp_cublaslt_run(m2, k2, n2, a2.data_ptr(), g.dtype_code(a2), b2.data_ptr(), g.dtype_code(b2), c2.data_ptr(), iters,
                                                 ctypes.byref(ms), stream)
                    if rnd:
                        theirs.append(ms.value)
            o = sum(ours) / len(ours)
            entry = {"ms": o, "tflops": fl / o / 1e9,
                     "protocol": f"3 alternating rounds, each {lead} untimed lead-in launches then {iters} timed"
                                 + ("; both sides as CUDA graphs" + (f" over {len(rot_b)} rotating operand sets" if len(rot_b) > 1 else "")
                                    if side_graph is not None else "")}
            if theirs:
                t_ = sum(theirs) / len(theirs)
                entry.update({"cublaslt_ms": t_, "cublaslt_tflops": fl / t_ / 1e9, "vs_cublaslt": t_ / o})
            extras[name] = entry
        line["side"] = extras

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
