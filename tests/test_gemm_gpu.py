"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU oracle.

Acceptance rule (floating point, from the path's specification): per element
    |C - C_ref| <= 1e-3 * sum_k |a_ik * b_kj| + 1e-6
with C_ref the FP64 product of the decoded FP8 bytes actually given to the kernel.  Exact
known-answer cases (one-hot, powers of two) must match bit for bit.  The reference's own
tests are `make gemm_test` (GEMM/makefile:48-49: 128^3, kernel 2, absolute tolerance 0.25,
GEMM/gemm_main.cpp:159-184); its shapes and criterion are reproduced here on the golden
fixtures recorded from its code.
"""
import glob
import os
import subprocess

import numpy as np
import pytest
import torch

from __graft_entry__ import ROOT, load_package

pytestmark = pytest.mark.gpu

F8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}
COMBOS = [(0, 0), (1, 1), (0, 1), (1, 0)]
SKINNY = (4, 8)          # the clustered split-K kernel and the stream-K kernel: both take M <= 128 only


@pytest.fixture(scope="module")
def g():
    assert torch.cuda.is_available()
    pkg = load_package()
    pkg._cabi.lib()          # the library must be present: there is no fallback
    torch.cuda.set_device(0)
    return pkg.gemm


def dev_bytes(x_np, fmt):
    return torch.from_numpy(np.ascontiguousarray(x_np)).cuda().view(F8[fmt])


def random_operands(g, m, k, n, fa, fb, seed=1):
    a = torch.empty((m, k), dtype=F8[fa], device="cuda")
    b = torch.empty((n, k), dtype=F8[fb], device="cuda")
    g.fill_normal(a, 2.0 if fa else 1.0, seed)
    g.fill_normal(b, 2.0 if fb else 1.0, seed + 1)
    return a, b


def host_bytes(t):
    return t.view(torch.uint8).cpu().numpy()


def assert_within_tolerance(oracle, C, A, fa, B, fb, rows=None, cols=None):
    C64, S = oracle.gemm_f64(A, fa, B, fb, rows=rows, cols=cols)
    bad, worst, wi = oracle.check_tolerance(C, C64, S)
    assert bad == 0, f"{bad} elements outside tolerance, worst ratio {worst} at flat index {wi}"
    return worst


def run(g, a, b, m, k, n, **kw):
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.gemm_ex(a, b, out, **kw)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    return out


# ---------------------------------------------------------------- golden fixtures / reference API

@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "gemm_*.npz"))),
                         ids=lambda p: os.path.basename(p)[5:-4])
@pytest.mark.parametrize("entry", ["GEMM", "GEMM4"])
def test_golden_fixture_through_reference_api(g, oracle, path, entry):
    fx = np.load(path)
    A, B, Cref = fx["A"], fx["B"], fx["C"]
    fa, fb = int(fx["fmt_a"]), int(fx["fmt_b"])
    m, k = A.shape
    n = B.shape[0]
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    getattr(g, entry)(m, k, n, dev_bytes(A, fa), dev_bytes(B, fb), out)      # gemm::GEMM / gemm::GEMM4 argument order
    torch.cuda.synchronize()
    C = out.cpu().numpy()
    assert_within_tolerance(oracle, C, A, fa, B, fb)
    # the reference's own acceptance criterion against its own CPU loop (gemm_main.cpp:165-172)
    assert np.max(np.abs(C - Cref)) <= 0.25
    # and far tighter in practice: both accumulate exact products in FP32
    assert np.max(np.abs(C - Cref)) <= 1e-3 * (np.abs(oracle.decode(A, fa)) @ np.abs(oracle.decode(B, fb)).T).max()


# ---------------------------------------------------------------- exact known answers

@pytest.mark.parametrize("kernel", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("fa,fb", COMBOS)
def test_one_hot_rows_select_columns_exactly(g, oracle, kernel, fa, fb):
    m, k, n = (64, 256, 384) if kernel in SKINNY else (384, 256, 640)
    one = 0x38 if fa == 0 else 0x3C                      # 1.0 in e4m3 / e5m2
    A = np.zeros((m, k), dtype=np.uint8)
    sel = (np.arange(m) * 7 + 3) % k
    A[np.arange(m), sel] = one
    rng = np.random.default_rng(3)
    B = rng.integers(0, 0x78 if fb == 0 else 0x7C, size=(n, k), dtype=np.uint8) | (rng.integers(0, 2, size=(n, k), dtype=np.uint8) << 7)
    out = run(g, dev_bytes(A, fa), dev_bytes(B, fb), m, k, n, kernel=kernel)
    want = oracle.decode(B, fb)[:, sel].T.astype(np.float32)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("kernel", [2, 3, 4, 5, 6, 7, 8])
def test_powers_of_two_sum_exactly(g, oracle, kernel):
    m, k, n = (128, 512, 256) if kernel in SKINNY else (256, 512, 512)
    rng = np.random.default_rng(5)
    # +-2^e with e in [-2, 2]: every product and every partial sum is exactly representable in FP32
    codes = np.array([0x28, 0x30, 0x38, 0x40, 0x48], dtype=np.uint8)
    A = codes[rng.integers(0, 5, size=(m, k))] | (rng.integers(0, 2, size=(m, k), dtype=np.uint8) << 7)
    B = codes[rng.integers(0, 5, size=(n, k))] | (rng.integers(0, 2, size=(n, k), dtype=np.uint8) << 7)
    out = run(g, dev_bytes(A, 0), dev_bytes(B, 0), m, k, n, kernel=kernel).cpu().numpy()
    want = (oracle.decode(A, 0) @ oracle.decode(B, 0).T).astype(np.float32)
    assert np.array_equal(out, want)


def test_special_values_propagate(g, oracle):
    # saturated inputs (+-448 / +-57344) and signed zeros; the sum of products must match FP64 within tolerance
    m, k, n = 256, 128, 256
    A = np.full((m, k), 0x7E, dtype=np.uint8); A[::2] = 0xFE; A[:, ::3] = 0x80
    B = np.full((n, k), 0x7B, dtype=np.uint8); B[1::2] = 0xFB; B[:, ::5] = 0x00
    out = run(g, dev_bytes(A, 0), dev_bytes(B, 1), m, k, n).cpu().numpy()
    assert_within_tolerance(oracle, out, A, 0, B, 1)
    assert np.isfinite(out).all()


# ---------------------------------------------------------------- random operands, every kernel / dtype / depth

@pytest.mark.parametrize("fa,fb", COMBOS)
@pytest.mark.parametrize("kernel,depth,shape", [
    (2, 2, (256, 384, 256)), (2, 4, (384, 1040, 200)), (2, 0, (130, 48, 131)),
    (1, 2, (300, 528, 516)), (1, 4, (256, 2064, 512)), (1, 0, (129, 144, 260)),
    (3, 2, (512, 400, 512)), (3, 4, (300, 208, 516)), (3, 0, (1030, 1024, 770)),
    (5, 2, (512, 400, 1024)), (5, 4, (300, 208, 1030)), (5, 0, (1030, 1024, 1540)),
    (4, 0, (16, 1024, 1000)), (4, 2, (100, 2048, 384)), (4, 4, (128, 528, 260)),
    (8, 0, (16, 1024, 1000)), (8, 2, (100, 2048, 384)), (8, 4, (128, 528, 260)), (8, 0, (33, 8192 + 16, 130)),
    (8, 0, (64, 256, 20000)), (8, 0, (1, 128 * 150, 128)), (8, 0, (128, 4096, 2500)),
    (6, 2, (256, 400, 512)), (6, 4, (200, 208, 516)), (6, 0, (700, 1024, 900)),
    (7, 2, (256, 400, 512)), (7, 4, (200, 208, 516)), (7, 0, (700, 1024, 900)),
    (7, 0, (16, 1024, 1000)), (7, 0, (7, 8192 + 16, 520)), (7, 0, (33, 528, 260)), (7, 0, (64, 4096, 2500)), (7, 0, (1, 2048, 8192)),
    (7, 0, (32, 144, 20000)),
    (0, 0, (640, 256, 896)),
])
def test_random_operands_all_kernels(g, oracle, fa, fb, kernel, depth, shape):
    m, k, n = shape
    a, b = random_operands(g, m, k, n, fa, fb, seed=17 + kernel)
    out = run(g, a, b, m, k, n, kernel=kernel, depth=depth)
    assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), fa, host_bytes(b), fb)


@pytest.mark.parametrize("kernel,max_ctas,shape", [
    (3, 8, (512, 400, 1280)),     # 10 pair tiles on 4 pairs: the last 2 run as 4 half-width items
    (3, 8, (700, 272, 1200)),     # ragged M and N: 15 tiles, 3 left over, no split (3 > 2) ... and
    (3, 12, (700, 272, 1200)),    # ... on 6 pairs 3 left over: split into 6 halves, the last one ragged
    (1, 4, (384, 528, 768)),      # single-CTA kernel: 9 tiles on 4 CTAs, 1 left over
    (1, 6, (300, 144, 1700)),     # 21 tiles on 6 CTAs, 3 left over, ragged edges
])
@pytest.mark.parametrize("fa,fb", [(0, 0), (1, 0)])
def test_tail_round_split_into_half_width_items(g, oracle, kernel, max_ctas, shape, fa, fb):
    m, k, n = shape
    a, b = random_operands(g, m, k, n, fa, fb, seed=91)
    out = run(g, a, b, m, k, n, kernel=kernel, max_ctas=max_ctas)
    assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), fa, host_bytes(b), fb)
    whole = run(g, a, b, m, k, n, kernel=kernel)                 # all tiles at once: no tail, no split
    assert torch.equal(out, whole)                               # same K order per element either way


@pytest.mark.parametrize("m", [1, 2, 7, 16, 17, 31, 32, 33, 64, 65, 127, 128, 129, 255, 257])
def test_ragged_m(g, oracle, m):
    k, n = 272, 300
    a, b = random_operands(g, m, k, n, 0, 0, seed=m)
    out = run(g, a, b, m, k, n)
    assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 0)


@pytest.mark.parametrize("k", [16, 32, 48, 64, 112, 128, 144, 256, 4096 + 16])
@pytest.mark.parametrize("kernel", [2, 3, 4, 5, 6, 7, 8])
def test_k_sweep_including_tails(g, oracle, k, kernel):
    m, n = (48, 200) if kernel in SKINNY else (260, 520)
    a, b = random_operands(g, m, k, n, 0, 1, seed=k)
    out = run(g, a, b, m, k, n, kernel=kernel)
    assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 1)


@pytest.mark.parametrize("split", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("m", [1, 24, 128])
@pytest.mark.parametrize("kernel", SKINNY)
def test_skinny_split_k(g, oracle, split, m, kernel):
    k, n = 2048 + 128, 640
    a, b = random_operands(g, m, k, n, 0, 0, seed=split)
    out = run(g, a, b, m, k, n, kernel=kernel, split_k=split)
    assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 0)
    again = run(g, a, b, m, k, n, kernel=kernel, split_k=split)
    assert torch.equal(out, again)                       # split-K reduction order is fixed: bitwise repeatable


@pytest.mark.parametrize("m,k,n,max_pieces", [(16, 8192, 8192, 0), (128, 8192, 8192, 0), (64, 4096, 1024, 0), (5, 1024, 128, 64),
                                              (100, 128 * 37, 128 * 5 + 3, 16), (32, 8192, 57344, 0)])
def test_stream_k_pieces_sum_in_fixed_order(g, oracle, m, k, n, max_pieces):
    """The stream-K kernel cuts tiles' K ranges between CTAs wherever the even split of the unit space falls; the
    finisher adds the parked partial sums in ascending K.  Launched repeatedly (the flags a launch raises must come
    back as zero: no memset between launches) the result must not change by a bit, and it must stay within the
    path's tolerance of the FP64 oracle on sampled rows and columns."""
    a, b = random_operands(g, m, k, n, 0, 0, seed=k + n)
    outs = [run(g, a, b, m, k, n, kernel=8, split_k=max_pieces) for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    cols = np.unique(np.concatenate([np.arange(0, n, max(1, n // 61)), np.arange(max(0, n - 130), n)]))
    assert_within_tolerance(oracle, np.ascontiguousarray(outs[0][:, torch.from_numpy(cols).cuda()].cpu().numpy()), host_bytes(a), 0,
                            host_bytes(b)[cols], 0)
    # power-of-two operands: every partial sum is exact, so the clustered split-K kernel (another split of K
    # altogether) must agree bit for bit
    if n <= 8192:
        rng = np.random.default_rng(m)
        codes = np.array([0x28, 0x30, 0x38, 0x40], dtype=np.uint8)
        A = codes[rng.integers(0, 4, size=(m, k))] | (rng.integers(0, 2, size=(m, k), dtype=np.uint8) << 7)
        B = codes[rng.integers(0, 4, size=(n, k))] | (rng.integers(0, 2, size=(n, k), dtype=np.uint8) << 7)
        x = run(g, dev_bytes(A, 0), dev_bytes(B, 0), m, k, n, kernel=8, split_k=max_pieces)
        y = run(g, dev_bytes(A, 0), dev_bytes(B, 0), m, k, n, kernel=4)
        assert torch.equal(x, y)


def test_zero_k_and_empty(g):
    out = torch.full((8, 12), 3.0, dtype=torch.float32, device="cuda")
    a = torch.empty((8, 0), dtype=F8[0], device="cuda")
    b = torch.empty((12, 0), dtype=F8[0], device="cuda")
    rc = load_package()._cabi.lib().b200fp8_gemm_rowcol_f32(8, 0, 12, None, 0, None, 0, out.data_ptr(), 2, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.count_nonzero(out).item() == 0          # empty sum
    del a, b


# ---------------------------------------------------------------- extended epilogue (alpha, beta, scales, 16-bit outputs)

@pytest.mark.parametrize("out_dtype,eps", [(torch.float32, 2.0 ** -22), (torch.bfloat16, 2.0 ** -8), (torch.float16, 2.0 ** -11)])
@pytest.mark.parametrize("kernel,shape,pitch_pad", [(2, (256, 272, 384), 0), (3, (300, 528, 520), 0), (5, (512, 400, 1030), 2),
                                                    (4, (24, 1024, 520), 0), (4, (100, 2048, 384), 0), (1, (130, 144, 259), 1),
                                                    (8, (24, 1024, 520), 0), (8, (100, 8192, 384), 0), (8, (128, 2048, 2050), 2),
                                                    (3, (512, 256, 512), 8)])
@pytest.mark.parametrize("beta", [0.0, 0.75])
def test_scaled_epilogue(g, oracle, out_dtype, eps, kernel, shape, pitch_pad, beta):
    """D = alpha*sa*sb*(A B^T) + beta*D against the FP64 oracle.  Tolerance: the path's rule scaled by
    |alpha*sa*sb|, plus the output format's rounding (eps * |expected|), plus the rounding of the old D term."""
    m, k, n = shape
    a, b = random_operands(g, m, k, n, 0, 1, seed=5 + kernel)
    alpha, sa, sb = 0.5, 0.25, 3.0
    sa_t = torch.tensor([sa], dtype=torch.float32, device="cuda")
    sb_t = torch.tensor([sb], dtype=torch.float32, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(3)
    buf = torch.randn((m, n + pitch_pad), generator=gen, device="cuda").to(out_dtype)
    old = buf[:, :n].float().cpu().numpy().astype(np.float64)
    d = buf[:, :n]                                      # row pitch n + pitch_pad: exercises the non-TMA store path too
    pad_before = buf[:, n:].clone()
    g.gemm_scaled(a, b, d, alpha=alpha, beta=beta, a_scale=sa_t, b_scale=sb_t, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = oracle.gemm_f64(host_bytes(a), 0, host_bytes(b), 1)
    f = alpha * sa * sb
    want = f * C64 + beta * old
    tol = abs(f) * (1e-3 * S + 1e-6) + eps * np.abs(want) + 1e-6 * np.abs(beta * old)
    got = d.float().cpu().numpy().astype(np.float64)
    worst = np.max(np.abs(got - want) / tol)
    assert worst <= 1.0, worst
    if pitch_pad:                                       # the padding columns are untouched
        assert torch.equal(buf[:, n:], pad_before)


def test_scaled_epilogue_with_unit_factors_equals_plain_operator(g):
    m, k, n = 512, 384, 768
    a, b = random_operands(g, m, k, n, 0, 0, seed=2)
    plain = run(g, a, b, m, k, n, kernel=3)
    d = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.gemm_scaled(a, b, d, kernel=3)
    torch.cuda.synchronize()
    assert torch.equal(d, plain)


# ---------------------------------------------------------------- memory safety: canaries instead of a sanitizer

@pytest.mark.parametrize("kernel,m,n,ldc", [(2, 130, 132, 160), (3, 300, 260, 264), (1, 129, 257, 257), (4, 20, 130, 131),
                                            (3, 300, 1030, 1032), (5, 512, 1029, 1032), (1, 130, 259, 260), (2, 130, 130, 132),
                                            (5, 300, 772, 776), (5, 257, 515, 515),
                                            (4, 100, 260, 272), (8, 20, 130, 131), (8, 100, 260, 272), (8, 128, 1027, 1028),
                                            (7, 20, 130, 131), (7, 60, 260, 272), (7, 9, 1028, 1032)])
def test_no_write_outside_c(g, oracle, kernel, m, n, ldc):
    k = 192
    a, b = random_operands(g, m, k, n, 0, 0, seed=9)
    guard = 4
    buf = torch.full((m + 2 * guard, ldc), float("nan"), dtype=torch.float32, device="cuda")
    c = buf[guard:guard + m]                              # rows of pitch ldc, guard rows above and below
    g.gemm_ex(a, b, c[:, :n], kernel=kernel, ldc=ldc)
    torch.cuda.synchronize()
    h = buf.cpu().numpy()
    assert np.isnan(h[:guard]).all() and np.isnan(h[guard + m:]).all()
    assert np.isnan(h[guard:guard + m, n:]).all()
    assert_within_tolerance(oracle, np.ascontiguousarray(h[guard:guard + m, :n]), host_bytes(a), 0, host_bytes(b), 0)


def test_errors_surface_as_cuda_invalid_value(g):
    a = torch.empty((128, 72), dtype=F8[0], device="cuda")   # K not a multiple of 16
    b = torch.empty((128, 72), dtype=F8[0], device="cuda")
    out = torch.empty((128, 128), dtype=torch.float32, device="cuda")
    with pytest.raises(load_package()._cabi.B200Fp8Error) as e:
        g.GEMM(128, 72, 128, a, b, out)
    assert e.value.code == 1


# ---------------------------------------------------------------- the benchmark configurations at full size

def freivalds(a, b, c):
    """C r against A (B^T r) in FP64 on the device, with the summed per-element tolerance as bound."""
    n = b.shape[0]
    gen = torch.Generator(device="cuda").manual_seed(7)
    r = (torch.randint(0, 2, (n,), device="cuda", generator=gen).double() * 2 - 1)
    worst = 0.0
    btr = torch.zeros(b.shape[1], dtype=torch.float64, device="cuda")
    babs = torch.zeros_like(btr)
    for n0 in range(0, n, 4096):
        blk = b[n0:n0 + 4096].double()
        btr += blk.T @ r[n0:n0 + 4096]
        babs += blk.abs().sum(dim=0)
    for m0 in range(0, a.shape[0], 4096):
        ablk = a[m0:m0 + 4096].double()
        want = ablk @ btr
        bound = 1e-3 * (ablk.abs() @ babs) + 1e-6 * n
        got = c[m0:m0 + 4096].double() @ r
        worst = max(worst, float(((got - want).abs() / bound).max()))
    return worst


def sampled_check(oracle, a, b, c, fa, fb, rows=64, cols=64, points=16384):
    """Sample of a large C against the FP64 oracle, every sampled element over the full K: `rows` random full rows
    and `cols` random full columns (plus the first, the last and those next to tile edges), the four corner tiles
    of 128 x 128, and `points` random elements.  Returns the worst error as a fraction of the tolerance."""
    m, k = a.shape
    n = b.shape[0]
    A, B = host_bytes(a), host_bytes(b)
    rng = np.random.default_rng(11)
    edges = (127, 128, 255, 256, 511, 512)
    pick_m = np.array(sorted(set([0, m - 1] + [x for x in edges if x < m] + list(rng.integers(0, m, rows)))))
    pick_n = np.array(sorted(set([0, n - 1] + [x for x in edges if x < n] + list(rng.integers(0, n, cols)))))
    worst = 0.0
    got = c[torch.from_numpy(pick_m).cuda()].cpu().numpy()                 # full rows, all at once
    worst = max(worst, assert_within_tolerance(oracle, got, np.ascontiguousarray(A[pick_m]), fa, B, fb))
    got = np.ascontiguousarray(c[:, torch.from_numpy(pick_n).cuda()].cpu().numpy())   # full columns
    worst = max(worst, assert_within_tolerance(oracle, got, A, fa, np.ascontiguousarray(B[pick_n]), fb))
    for r0 in sorted({0, max(0, m - 128)}):                                # corner tiles
        for c0 in sorted({0, max(0, n - 128)}):
            got = np.ascontiguousarray(c[r0:r0 + 128, c0:c0 + 128].cpu().numpy())
            worst = max(worst, assert_within_tolerance(oracle, got, np.ascontiguousarray(A[r0:r0 + 128]), fa,
                                                       np.ascontiguousarray(B[c0:c0 + 128]), fb))
    ms, ns = rng.integers(0, m, points), rng.integers(0, n, points)
    C64, S = oracle.gemm_f64_points(A, fa, B, fb, ms, ns)
    got = c[torch.from_numpy(ms).cuda(), torch.from_numpy(ns).cuda()].cpu().numpy()
    bad, w, _ = oracle.check_tolerance(got, C64, S)
    assert bad == 0
    return max(worst, w)


def test_config1_1024_cubed_full_check(g, oracle):
    m = k = n = 1024
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 16)
    for entry in (g.GEMM, g.GEMM4):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        entry(m, k, n, a, b, out)
        torch.cuda.synchronize()
        assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 0)


@pytest.mark.parametrize("fa,fb", COMBOS)
@pytest.mark.parametrize("entry", ["GEMM", "GEMM4"])
def test_config2_4096_dtype_sweep(g, oracle, fa, fb, entry):
    m = k = n = 4096
    a, b = random_operands(g, m, k, n, fa, fb, seed=0xB200F800 + 32 + 2 * COMBOS.index((fa, fb)))
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    getattr(g, entry)(m, k, n, a, b, out)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    if (fa, fb) == (0, 0) and entry == "GEMM":
        assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), fa, host_bytes(b), fb)   # every element
    else:
        sampled_check(oracle, a, b, out, fa, fb)
    assert freivalds(a, b, out) <= 1.0


@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (8192, 8192, 28672), (8192, 28672, 8192)],
                         ids=["target-8192", "ffn-up", "ffn-down"])
def test_config3_large_shapes(g, oracle, shape):
    m, k, n = shape
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 48)
    out = run(g, a, b, m, k, n)
    sampled_check(oracle, a, b, out, 0, 0)
    assert freivalds(a, b, out) <= 1.0


@pytest.mark.parametrize("m,k,n", [(1, 8192, 8192), (16, 8192, 8192), (64, 8192, 8192), (128, 8192, 8192), (32, 8192, 57344)])
def test_config4_skinny_decode_shapes(g, oracle, m, k, n):
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 64)
    out = run(g, a, b, m, k, n)
    if m * n <= 16 * 8192:
        assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 0)   # exhaustive
    else:
        sampled_check(oracle, a, b, out, 0, 0, rows=16, cols=64)
    assert freivalds(a, b, out) <= 1.0


def test_config5_n_shards_equal_unsharded_bitwise(g, oracle):
    # the multi-GPU partition on one device: rank r's call on its slab of B must reproduce exactly the columns
    # the unsharded call produces (same kernel, same K order), written in place through ldc
    pkg = load_package()
    m, k, n = 2048, 4096, 4096
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 80)
    for kernel in (3, 5):
        full = run(g, a, b, m, k, n, kernel=kernel)
        for world in (2, 4, 8):
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            for r in range(world):
                sh = pkg.shard.column_shard(n, r, world)
                g.gemm_ex(a, b[sh.n_begin:sh.n_end], out[:, sh.n_begin:sh.n_end], kernel=kernel, ldc=n)
            torch.cuda.synchronize()
            assert torch.equal(out, full)
    sampled_check(oracle, a, b, full, 0, 0, rows=2, cols=2, points=1024)


def test_config5_full_size_one_rank_shard(g, oracle):
    # one rank's share of the 32768^3 problem at 8 GPUs: A 32768 x 32768, B slab 4096 x 32768
    m = k = 32768
    n = 4096
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 80)
    out = run(g, a, b, m, k, n)
    sampled_check(oracle, a, b, out, 0, 0, rows=16, cols=16)
    assert freivalds(a, b, out) <= 1.0


def test_config5_full_size_single_gpu_headline_problem(g, oracle):
    """The benchmark's N = 1 problem as it is timed: 32768^3 in one call (selects the 256 x 512 pair tile with tile
    pacing).  6.4 GB on the device; sampled rows, columns, corner tiles and points through the FP64 oracle, and every
    element through the randomised product check."""
    m = k = n = 32768
    a, b = random_operands(g, m, k, n, 0, 0, seed=0xB200F800 + 64)
    out = run(g, a, b, m, k, n)
    sampled_check(oracle, a, b, out, 0, 0, rows=16, cols=16, points=16384)
    assert freivalds(a, b, out) <= 1.0
    del out
    torch.cuda.empty_cache()


# ---------------------------------------------------------------- size-independent properties at large sizes

@pytest.mark.parametrize("shape", [(2048, 4096, 3072), (8192, 8192, 4096), (4096, 2048, 8192)])
@pytest.mark.parametrize("fa,fb", [(0, 0), (0, 1)])
def test_transpose_symmetry_is_bitwise(g, shape, fa, fb):
    """(A B^T)^T = B A^T: every product a*b is the same number either way round and each element sums its K products
    in the same order (k-blocks in sequence), whatever tile or kernel the swapped shape selects: identical bits."""
    m, k, n = shape
    a, b = random_operands(g, m, k, n, fa, fb, seed=31)
    c = run(g, a, b, m, k, n)
    ct = run(g, b, a, n, k, m)
    assert torch.equal(c, ct.T)


def test_row_permutation_and_row_blocks_are_bitwise(g):
    """Rows of C depend only on their own row of A: permuting A's rows permutes C's rows, and any row block computed
    alone (other tile shapes, other kernels) equals the same rows of the full result."""
    m, k, n = 4096, 4096, 4096
    a, b = random_operands(g, m, k, n, 0, 0, seed=33)
    c = run(g, a, b, m, k, n)
    perm = torch.randperm(m, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    ap = a.view(torch.uint8)[perm].contiguous().view(a.dtype)
    assert torch.equal(run(g, ap, b, m, k, n), c[perm])
    for r0, r1 in ((0, 300), (1000, 1257), (4096 - 640, 4096)):          # 300 and 257 rows pick other kernels than 4096
        assert torch.equal(run(g, a[r0:r1], b, r1 - r0, k, n), c[r0:r1])


# ---------------------------------------------------------------- host-pointer entry point, generator, drop-in binary

@pytest.mark.parametrize("shape", [(300, 272, 520), (64, 1024, 512), (2048, 2048, 4096), (8192, 4096, 4096), (4096, 4096, 8192),
                                   (4608, 2048, 12288), (5000, 3072, 9000), (12288, 1024, 12288)])
def test_host_entry_point_matches_device_entry(g, oracle, shape):
    """The host entry computes C as a grid of blocks (uploads, operator and downloads pipelined); every element still
    sums its K products in the same order, so the result equals the one-call device result bit for bit."""
    m, k, n = shape
    a, b = random_operands(g, m, k, n, 0, 1, seed=23)
    dev_out = run(g, a, b, m, k, n)
    ha, hb = a.cpu(), b.cpu()
    hc = torch.full((m, n), float("nan"), dtype=torch.float32).pin_memory()
    g.gemm_host(ha, hb, hc)
    assert torch.equal(hc, dev_out.cpu())


def test_fill_normal_matches_host_generator_and_shards(g, oracle):
    n = 1 << 20
    t = torch.empty(n, dtype=F8[0], device="cuda")
    g.fill_normal(t, 1.0, 0xB200F800)
    dev = host_bytes(t)
    host = oracle.fill_normal(n, 0, 1.0, 0xB200F800)
    # same recipe on both sides; device and host logf/cosf may differ in the last ulp, which moves a sample
    # across a rounding boundary only rarely
    assert (dev != host).mean() < 1e-3
    v = oracle.decode(dev, 0)
    assert abs(v.mean()) < 5e-3 and abs(v.std() - 1.0) < 1e-2 and np.isfinite(v).all()
    part = torch.empty(n // 4, dtype=F8[0], device="cuda")
    g.fill_normal(part, 1.0, 0xB200F800, index_offset=n // 2)
    assert np.array_equal(host_bytes(part), dev[n // 2: n // 2 + n // 4])
    e = torch.empty(n, dtype=F8[1], device="cuda")
    g.fill_normal(e, 2.0, 5)
    assert abs(oracle.decode(host_bytes(e), 1).std() - 2.0) < 3e-2


def test_reference_driver_links_and_verifies():
    """The reference's unmodified gemm_main.cpp, linked against this library (built where the reference
    tree exists), run as its `make gemm_test` does: `gemm 128 128 128 2 1 0 0`."""
    exe = os.path.join(ROOT, "oracle", "_ref", "gemm_dropin")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/gemm_dropin not built (needs the reference tree at build time)")
    for kernel in (1, 2, 3, 5, 7):
        res = subprocess.run([exe, "128", "128", "128", str(kernel), "1", "0", "0"], capture_output=True, text=True,
                             timeout=300, cwd=os.path.dirname(exe))
        assert res.returncode == 0, res.stderr
        line = [ln for ln in res.stdout.splitlines() if "MAx Error" in ln]
        assert line, res.stdout
        assert float(line[0].split()[-1]) < 1e-3, res.stdout
        assert "There are 0 errors." in res.stdout


# One shape for every branch of the automatic kernel choice (the id it must land on, asked through
# b200fp8_choose_kernel, guards the list against a rule that silently stops being reached).
PLANNER_BRANCHES = [
    ((1152, 1024, 4096), 1),     # K <= 1024: one-CTA 128 x 256 tiles
    ((4096, 512, 4096), 1),
    ((1152, 8192, 4096), 1),     # 1.5 rounds of pair tiles against one round of one-CTA tiles
    ((16384, 256, 128), 6),      # N <= 128 under a tall A: one round of 256 x 128 pair tiles
    ((4096, 1024, 96), 7),       # N <= 128, few row tiles: 128 x 64 tiles
    ((40000, 256, 128), 2),      # N <= 128, more row tiles than pairs: 128 x 128 tiles
    ((8192, 8192, 136), 6),      # two columns of tiles under a tall A, long K
    ((640, 4096, 5120), 3),      # one round either way, K >= 4096: pair tiles
    ((200, 4096, 11008), 3),
    ((2048, 2048, 2048), 1),     # one round, short K: one-CTA tiles
    ((256, 8192, 8192), 6),      # one row of 256 x 128 pair tiles
    ((8192, 28672, 8192), 5),    # long K, seven rounds of wide tiles
    ((4096, 28672, 4096), 3),    # long K but two rounds: pair tiles
    ((48, 2048, 2048), 4),       # M <= 64 with K = 2048: split-K
    ((96, 2048, 4096), 7),       # M > 64 with K <= 2048: tile kernel
    ((64, 1024, 8192), 7),       # 32 < M <= 64 with K <= 1024: tile kernel
    ((32, 512, 8192), 7),        # 16 < M <= 32 with K <= 512: tile kernel
    ((32, 1024, 2048), 4),
    ((16, 512, 2048), 4),        # M <= 16: always split-K
    ((128, 4096, 1024), 4),      # eight N tiles: splits capped by the k-blocks each would own
]


@pytest.mark.parametrize("shape,expected", PLANNER_BRANCHES)
def test_every_planner_branch_selects_its_kernel_and_computes_the_product(g, oracle, shape, expected):
    from __graft_entry__ import load_package
    m, k, n = shape
    lib = load_package()._cabi.lib()
    assert lib.b200fp8_choose_kernel(m, k, n) == expected
    a, b = random_operands(g, m, k, n, 0, 1, seed=0xB200F800 + 300 + expected)
    out = run(g, a, b, m, k, n)
    if m * n <= 1 << 22 and m * n * k <= 1 << 33:
        assert_within_tolerance(oracle, out.cpu().numpy(), host_bytes(a), 0, host_bytes(b), 1)
    else:
        sampled_check(oracle, a, b, out, 0, 1, rows=8, cols=8, points=4096)
    assert freivalds(a, b, out) <= 1.0
    # and the forced kernel gives the same bits as the automatic call: the choice is only a choice
    forced = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.gemm_ex(a, b, forced, kernel=expected)
    torch.cuda.synchronize()
    assert torch.equal(forced, out)
