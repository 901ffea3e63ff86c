"""GPU tests of the full epilogue entry point (b200fp8_gemm_rowcol_epilogue) against the CPU oracle:

    t = alpha * sa * sb * (A B^T) + beta * D + bias[n];   amax = max |t|;   D = convert(sd * t)

with D in FP32 / BF16 / FP16 / E4M3 / E5M2.  The FP64 oracle gives t; the path's tolerance
(1e-3 * sum|a b| + 1e-6, scaled by |alpha sa sb|) bounds the error of t, and because the
8-bit conversion is monotone the stored byte must decode to a value between the oracle's
encodings of the two ends of that interval (this covers rounding, subnormals and saturation
with the oracle's own encoder, which is pinned to the toolkit's).  Known-answer cases whose
results are exactly representable must match bit for bit.
"""
import numpy as np
import pytest
import torch

from __graft_entry__ import load_package

pytestmark = pytest.mark.gpu

F8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}
OUT8 = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
EPS = {torch.float32: 2.0 ** -22, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


@pytest.fixture(scope="module")
def g():
    assert torch.cuda.is_available()
    pkg = load_package()
    pkg._cabi.lib()          # the library must be present: there is no fallback
    torch.cuda.set_device(0)
    return pkg.gemm


def operands(g, m, k, n, fa=0, fb=0, seed=1):
    a = torch.empty((m, k), dtype=F8[fa], device="cuda")
    b = torch.empty((n, k), dtype=F8[fb], device="cuda")
    g.fill_normal(a, 2.0 if fa else 1.0, seed)
    g.fill_normal(b, 2.0 if fb else 1.0, seed + 1)
    return a, b


def host_bytes(t):
    return t.view(torch.uint8).cpu().numpy()


def scalar(x):
    return torch.tensor([x], dtype=torch.float32, device="cuda")


SHAPES = [(2, (256, 272, 384), 0), (3, (300, 528, 528), 0), (5, (512, 400, 1040), 16), (4, (24, 1024, 528), 0),
          (4, (100, 2048, 384), 0), (1, (130, 144, 259), 1), (3, (512, 256, 517), 3)]


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("kernel,shape,pitch_pad", SHAPES)
@pytest.mark.parametrize("beta,with_bias", [(0.0, False), (0.5, True)])
def test_fp8_output_with_scale_amax_and_bias(g, oracle, out_dtype, kernel, shape, pitch_pad, beta, with_bias):
    m, k, n = shape
    a, b = operands(g, m, k, n, 0, 1, seed=11 + kernel)
    alpha, sa, sb, sd = 0.5, 0.25, 3.0, 0.125
    gen = torch.Generator(device="cuda").manual_seed(5)
    buf = (4 * torch.randn((m, n + pitch_pad), generator=gen, device="cuda")).to(out_dtype)
    fmt = OUT8[out_dtype]
    old = oracle.decode(host_bytes(buf[:, :n].contiguous()), fmt).astype(np.float64)
    d = buf[:, :n]
    pad_before = buf[:, n:].clone().view(torch.uint8)
    bias = (3 * torch.randn(n, generator=gen, device="cuda")).to(torch.bfloat16) if with_bias else None
    amax = scalar(-1.0)                                   # the library zeroes it before the kernel
    g.gemm_epilogue(a, b, d, alpha=alpha, beta=beta, a_scale=scalar(sa), b_scale=scalar(sb), d_scale=scalar(sd),
                    amax_d=amax, bias=bias, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = oracle.gemm_f64(host_bytes(a), 0, host_bytes(b), 1)
    f = alpha * sa * sb
    t = f * C64 + beta * old
    if with_bias:
        t = t + bias.float().cpu().numpy().astype(np.float64)[None, :]
    tol = abs(f) * (1e-3 * S + 1e-6) + 2.0 ** -22 * (np.abs(t) + np.abs(beta * old))
    lo = oracle.decode(oracle.encode((sd * (t - tol)).astype(np.float32), fmt), fmt)
    hi = oracle.decode(oracle.encode((sd * (t + tol)).astype(np.float32), fmt), fmt)
    got = oracle.decode(host_bytes(d.contiguous()), fmt)
    bad = ~((got >= lo) & (got <= hi))
    assert not bad.any(), (int(bad.sum()), np.argwhere(bad)[:4], got[bad][:4], lo[bad][:4], hi[bad][:4])
    # the maximum is taken before the output scale, over the valid part only
    am = float(amax.item())
    assert abs(am - np.abs(t).max()) <= tol.max(), (am, np.abs(t).max())
    if pitch_pad:
        assert torch.equal(buf[:, n:].view(torch.uint8), pad_before)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kernel,shape,pitch_pad", [SHAPES[1], SHAPES[2], SHAPES[3], SHAPES[5]])
def test_wide_outputs_with_bias_and_amax(g, oracle, out_dtype, kernel, shape, pitch_pad):
    m, k, n = shape
    a, b = operands(g, m, k, n, 0, 0, seed=21 + kernel)
    alpha, sd, beta = 0.75, 2.0, 0.25
    gen = torch.Generator(device="cuda").manual_seed(6)
    buf = torch.randn((m, n + pitch_pad), generator=gen, device="cuda").to(out_dtype)
    old = buf[:, :n].float().cpu().numpy().astype(np.float64)
    d = buf[:, :n]
    bias = torch.randn(n, generator=gen, device="cuda")
    amax = scalar(1e30)
    g.gemm_epilogue(a, b, d, alpha=alpha, beta=beta, d_scale=scalar(sd), amax_d=amax, bias=bias, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = oracle.gemm_f64(host_bytes(a), 0, host_bytes(b), 0)
    t = alpha * C64 + beta * old + bias.cpu().numpy().astype(np.float64)[None, :]
    tol_t = alpha * (1e-3 * S + 1e-6) + 2.0 ** -22 * (np.abs(t) + np.abs(old))
    want = sd * t
    got = d.float().cpu().numpy().astype(np.float64)
    worst = np.max(np.abs(got - want) / (sd * tol_t + EPS[out_dtype] * np.abs(want)))
    assert worst <= 1.0, worst
    assert abs(float(amax.item()) - np.abs(t).max()) <= tol_t.max()


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("kernel,m,n", [(2, 128, 128), (3, 256, 512), (5, 300, 1040), (4, 16, 256), (1, 130, 272)])
def test_fp8_output_exact_known_answers(g, oracle, out_dtype, kernel, m, n):
    """0/1 operands with K = 16: every sum is an integer <= 16, exact in FP32, and the power-of-two output scale
    keeps it exact, so the conversion sees the same float on both sides: the output bytes (ties to even, and
    saturation at 448 for E4M3 with d_scale = 64) and the maximum must equal the oracle's bit for bit."""
    k = 16
    rng = np.random.default_rng(kernel)
    one = {0: 0x38, 1: 0x3C}
    A = (rng.random((m, k)) < 0.6)
    B = (rng.random((n, k)) < 0.6)
    a = torch.from_numpy(np.where(A, one[0], 0).astype(np.uint8)).cuda().view(F8[0])
    b = torch.from_numpy(np.where(B, one[1], 0).astype(np.uint8)).cuda().view(F8[1])
    sums = A.astype(np.float32) @ B.astype(np.float32).T
    fmt = OUT8[out_dtype]
    for sd in (1.0, 0.25, 64.0):
        d = torch.zeros((m, n), dtype=torch.uint8, device="cuda").view(out_dtype)
        amax = scalar(0.0)
        g.gemm_epilogue(a, b, d, d_scale=scalar(sd), amax_d=amax, kernel=kernel)
        torch.cuda.synchronize()
        assert g.device_status() == 0
        want = oracle.encode((sd * sums).astype(np.float32), fmt)
        assert np.array_equal(host_bytes(d), want), sd
        assert float(amax.item()) == float(sums.max())


def test_epilogue_with_unit_factors_equals_plain_operator(g):
    m, k, n = 512, 384, 768
    a, b = operands(g, m, k, n, 0, 0, seed=2)
    plain = torch.empty((m, n), dtype=torch.float32, device="cuda")
    g.gemm_ex(a, b, plain, kernel=3)
    d = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    amax = scalar(0.0)
    g.gemm_epilogue(a, b, d, amax_d=amax, kernel=3)
    torch.cuda.synchronize()
    assert torch.equal(d, plain)
    assert float(amax.item()) == float(plain.abs().max().item())


def test_epilogue_rejects_bad_arguments(g):
    pkg = load_package()
    a, b = operands(g, 64, 64, 64)
    d = torch.empty((64, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(TypeError):
        g.gemm_epilogue(a, b, d, bias=torch.zeros(63, device="cuda"))
    with pytest.raises(TypeError):
        g.gemm_epilogue(a, b, d.to(torch.int32))
    lib = pkg._cabi.lib()
    ep = pkg._cabi.EpilogueDesc()
    ep.struct_bytes = 4                                   # wrong size: refused before anything is launched
    rc = lib.b200fp8_gemm_rowcol_epilogue(64, 64, 64, a.data_ptr(), 0, 64, b.data_ptr(), 0, 64, d.data_ptr(), 0, 64,
                                          ep, None, None)
    assert rc == 1
    rc = lib.b200fp8_gemm_rowcol_epilogue(64, 64, 64, a.data_ptr(), 0, 64, b.data_ptr(), 0, 64, d.data_ptr(), 9, 64,
                                          None, None, None)
    assert rc == 1
