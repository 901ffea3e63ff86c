"""GPU tests of the full epilogue entry point (b200fp8_gemm_rowcol_epilogue) against the CPU oracle:

    t = act(alpha * sa * sb * ra[m] * rb[n] * (A B^T) + beta * D + bias[n]);   amax = max |t|;   D = convert(sd * t)

with D in FP32 / BF16 / FP16 / E4M3 / E5M2, optional per-row scale vectors ra / rb and act in none / ReLU / GELU.  The FP64 oracle gives t; the path's tolerance
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


def activation_f64(t, name):
    """The activations in FP64 and a bound on |act'| (how far an error of t can move the result)."""
    from scipy.special import erf
    if name == "relu":
        return np.maximum(t, 0.0), 1.0
    if name == "gelu":
        return 0.5 * t * (1.0 + erf(t / np.sqrt(2.0))), 1.13
    if name == "gelu_tanh":
        return 0.5 * t * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (t + 0.044715 * t ** 3))), 1.13
    return t, 1.0


ROW_SCALE_SHAPES = [(3, (300, 528, 528)), (5, (512, 400, 1040)), (4, (24, 1024, 528)), (4, (100, 2048, 384)),
                    (8, (16, 1024, 640)), (1, (130, 144, 259)), (7, (48, 512, 200)), (0, (1, 4096, 1024))]


@pytest.mark.parametrize("activation", ["none", "relu", "gelu", "gelu_tanh"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kernel,shape", ROW_SCALE_SHAPES)
def test_row_scales_and_activations(g, oracle, kernel, shape, out_dtype, activation):
    """Per-row scales of A and of B (row-wise quantised operands) and the activation after the bias, against FP64.
    The activations' slopes are at most 1.13, so the tolerance of t, widened by that factor plus a few FP32 ulps
    for erff / tanhf, bounds the result."""
    m, k, n = shape
    a, b = operands(g, m, k, n, 0, 1, seed=31 + kernel)
    gen = torch.Generator(device="cuda").manual_seed(7)
    ra = torch.rand(m, generator=gen, device="cuda") * 0.2 + 0.01
    rb = torch.rand(n, generator=gen, device="cuda") * 0.05 + 0.001
    bias = torch.randn(n, generator=gen, device="cuda") * 0.5
    alpha, sa, beta = 1.5, 0.5, 0.25
    old_t = torch.randn((m, n), generator=gen, device="cuda").to(out_dtype)
    d = old_t.clone()
    amax = scalar(-1.0)
    g.gemm_epilogue(a, b, d, alpha=alpha, beta=beta, a_scale=scalar(sa), amax_d=amax, bias=bias, a_row_scale=ra,
                    b_row_scale=rb, activation=activation, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = oracle.gemm_f64(host_bytes(a), 0, host_bytes(b), 1)
    f = alpha * sa * ra.cpu().numpy().astype(np.float64)[:, None] * rb.cpu().numpy().astype(np.float64)[None, :]
    old = old_t.float().cpu().numpy().astype(np.float64)
    pre = f * C64 + beta * old + bias.cpu().numpy().astype(np.float64)[None, :]
    tol_pre = f * (1e-3 * S + 1e-6) + 2.0 ** -21 * (np.abs(pre) + np.abs(beta * old) + np.abs(f * C64))
    want, slope = activation_f64(pre, activation)
    tol = slope * tol_pre + 2.0 ** -20 * np.abs(want) + 1e-7
    got = d.float().cpu().numpy().astype(np.float64)
    worst = np.max(np.abs(got - want) / (tol + EPS[out_dtype] * np.abs(want)))
    assert worst <= 1.0, worst
    # the maximum is of the activated value
    assert abs(float(amax.item()) - np.abs(want).max()) <= tol.max()
    # and the vectors really entered: without them the result differs
    if activation == "none" and out_dtype == torch.float32:
        d2 = old_t.clone()
        g.gemm_epilogue(a, b, d2, alpha=alpha, beta=beta, a_scale=scalar(sa), bias=bias, kernel=kernel)
        torch.cuda.synchronize()
        assert not torch.equal(d, d2)


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("kernel,shape", [ROW_SCALE_SHAPES[0], ROW_SCALE_SHAPES[2], ROW_SCALE_SHAPES[5]])
def test_fp8_output_with_row_scales_and_relu(g, oracle, out_dtype, kernel, shape):
    """8-bit output after row scales, bias and ReLU: the stored byte decodes to a value between the oracle's encodings
    of the two ends of the tolerance interval (ReLU is monotone, like the conversion)."""
    m, k, n = shape
    a, b = operands(g, m, k, n, 0, 0, seed=41 + kernel)
    gen = torch.Generator(device="cuda").manual_seed(8)
    ra = torch.rand(m, generator=gen, device="cuda") * 0.5 + 0.05
    rb = torch.rand(n, generator=gen, device="cuda") * 0.5 + 0.05
    bias = (2 * torch.randn(n, generator=gen, device="cuda")).to(torch.float16)
    sd = 0.5
    fmt = OUT8[out_dtype]
    d = torch.zeros((m, n), dtype=torch.uint8, device="cuda").view(out_dtype)
    amax = scalar(0.0)
    g.gemm_epilogue(a, b, d, d_scale=scalar(sd), amax_d=amax, bias=bias, a_row_scale=ra, b_row_scale=rb,
                    activation="relu", kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = oracle.gemm_f64(host_bytes(a), 0, host_bytes(b), 0)
    f = ra.cpu().numpy().astype(np.float64)[:, None] * rb.cpu().numpy().astype(np.float64)[None, :]
    pre = f * C64 + bias.float().cpu().numpy().astype(np.float64)[None, :]
    tol = f * (1e-3 * S + 1e-6) + 2.0 ** -21 * (np.abs(pre) + np.abs(f * C64))
    lo = oracle.decode(oracle.encode((sd * np.maximum(pre - tol, 0.0)).astype(np.float32), fmt), fmt)
    hi = oracle.decode(oracle.encode((sd * np.maximum(pre + tol, 0.0)).astype(np.float32), fmt), fmt)
    got = oracle.decode(host_bytes(d), fmt)
    bad = ~((got >= lo) & (got <= hi))
    assert not bad.any(), (int(bad.sum()), np.argwhere(bad)[:4], got[bad][:4], lo[bad][:4], hi[bad][:4])
    assert abs(float(amax.item()) - np.maximum(pre, 0.0).max()) <= tol.max()


@pytest.mark.parametrize("kernel,m,n", [(3, 256, 512), (4, 16, 256), (8, 32, 384), (1, 130, 272)])
def test_relu_and_power_of_two_row_scales_exact(g, kernel, m, n):
    """0/1 operands (K = 16), power-of-two row scales and an integer bias: every intermediate is exact in FP32, so
    the result of scale, bias and ReLU must equal the integer arithmetic bit for bit."""
    k = 16
    rng = np.random.default_rng(100 + kernel)
    A = (rng.random((m, k)) < 0.5)
    B = (rng.random((n, k)) < 0.5)
    a = torch.from_numpy(np.where(A, 0x38, 0).astype(np.uint8)).cuda().view(F8[0])
    b = torch.from_numpy(np.where(B, 0x38, 0).astype(np.uint8)).cuda().view(F8[0])
    ra = 2.0 ** rng.integers(-2, 3, m)
    rb = 2.0 ** rng.integers(-2, 3, n)
    bias = rng.integers(-6, 2, n).astype(np.float64)
    sums = A.astype(np.float64) @ B.astype(np.float64).T
    want = np.maximum(ra[:, None] * rb[None, :] * sums + bias[None, :], 0.0)
    d = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    amax = scalar(0.0)
    g.gemm_epilogue(a, b, d, amax_d=amax, bias=torch.from_numpy(bias.astype(np.float32)).cuda(),
                    a_row_scale=torch.from_numpy(ra.astype(np.float32)).cuda(),
                    b_row_scale=torch.from_numpy(rb.astype(np.float32)).cuda(), activation="relu", kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    assert np.array_equal(d.cpu().numpy().astype(np.float64), want)
    assert float(amax.item()) == float(want.max())


@pytest.mark.parametrize("activation", ["gelu", "gelu_tanh"])
@pytest.mark.parametrize("kernel,m,n", [(3, 256, 512), (4, 16, 384), (1, 130, 272)])
def test_gelu_accuracy_on_exact_arguments(g, kernel, m, n, activation):
    """0/1 operands, power-of-two row scales and multiples of 1/4 as bias: the argument of the activation is exact in
    FP32 and spreads over [-9, 9], so the difference to the FP64 function is the formula's own error: at most 2e-6
    relative right of zero and 1e-6 |t| absolute left of it (the bound the header states)."""
    k = 16
    rng = np.random.default_rng(200 + kernel)
    A = (rng.random((m, k)) < 0.5)
    B = (rng.random((n, k)) < 0.5)
    a = torch.from_numpy(np.where(A, 0x38, 0).astype(np.uint8)).cuda().view(F8[0])
    b = torch.from_numpy(np.where(B, 0x38, 0).astype(np.uint8)).cuda().view(F8[0])
    ra = 2.0 ** rng.integers(-4, 0, m)
    rb = 2.0 ** rng.integers(-1, 2, n)
    bias = rng.integers(-36, 4, n) / 4.0
    pre = ra[:, None] * rb[None, :] * (A.astype(np.float64) @ B.astype(np.float64).T) + bias[None, :]
    assert pre.min() < -6 and pre.max() > 3
    want, _ = activation_f64(pre, activation)
    d = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.gemm_epilogue(a, b, d, bias=torch.from_numpy(bias.astype(np.float32)).cuda(),
                    a_row_scale=torch.from_numpy(ra.astype(np.float32)).cuda(),
                    b_row_scale=torch.from_numpy(rb.astype(np.float32)).cuda(), activation=activation, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    got = d.cpu().numpy().astype(np.float64)
    bound = np.where(pre >= 0, 2e-6 * np.abs(want), 1e-6 * np.abs(pre)) + 1e-30
    worst = np.max(np.abs(got - want) / bound)
    assert worst <= 1.0, worst


def test_shorter_epilogue_struct_of_older_callers_is_accepted(g):
    """A caller compiled before the activation and row-scale fields existed passes the shorter struct size: the
    library must not look at the fields behind it (set here to values that would change the result) and gives the
    plain scaled result."""
    import ctypes
    pkg = load_package()
    lib = pkg._cabi.lib()
    m, k, n = 256, 256, 384
    a, b = operands(g, m, k, n, seed=3)
    want = torch.empty((m, n), dtype=torch.float32, device="cuda")
    g.gemm_epilogue(a, b, want, alpha=0.5, kernel=3)
    ep = pkg._cabi.EpilogueDesc()
    class OldEpilogue(ctypes.Structure):                  # the struct as older callers were compiled against it
        _fields_ = pkg._cabi.EpilogueDesc._fields_[:9]
    assert OldEpilogue._fields_[-1][0] == "bias_dtype" and ctypes.sizeof(OldEpilogue) == 64
    ep.struct_bytes = ctypes.sizeof(OldEpilogue)
    ep.alpha, ep.beta = 0.5, 0.0
    wrong_m = torch.full((m,), 1000.0, device="cuda")
    wrong_n = torch.full((n,), 1000.0, device="cuda")
    ep.activation = 1                                    # behind the declared size: must not be looked at
    ep.a_row_scale = wrong_m.data_ptr()
    ep.b_row_scale = wrong_n.data_ptr()
    got = torch.empty_like(want)
    opt = pkg.gemm.Options(ctypes.sizeof(pkg.gemm.Options), 0, 3, 0, 0)
    rc = lib.b200fp8_gemm_rowcol_epilogue(m, k, n, a.data_ptr(), 0, k, b.data_ptr(), 0, k, got.data_ptr(), 0, n,
                                          ctypes.byref(ep), ctypes.byref(opt), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    ep.struct_bytes = ctypes.sizeof(pkg._cabi.EpilogueDesc)   # full size: an unknown activation is refused, nothing launched
    ep.activation = 77
    before = lib.b200fp8_launch_count()
    rc = lib.b200fp8_gemm_rowcol_epilogue(m, k, n, a.data_ptr(), 0, k, b.data_ptr(), 0, k, got.data_ptr(), 0, n,
                                          ctypes.byref(ep), ctypes.byref(opt), None)
    assert rc == 1 and lib.b200fp8_launch_count() == before


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
    with pytest.raises(TypeError):
        g.gemm_epilogue(a, b, d, a_row_scale=torch.zeros(63, device="cuda"))
    with pytest.raises(TypeError):
        g.gemm_epilogue(a, b, d, b_row_scale=torch.zeros(64, device="cuda", dtype=torch.float16))
    with pytest.raises(ValueError):
        g.gemm_epilogue(a, b, d, activation="swish")
    lib = pkg._cabi.lib()
    ep = pkg._cabi.EpilogueDesc()
    ep.struct_bytes = 4                                   # wrong size: refused before anything is launched
    rc = lib.b200fp8_gemm_rowcol_epilogue(64, 64, 64, a.data_ptr(), 0, 64, b.data_ptr(), 0, 64, d.data_ptr(), 0, 64,
                                          ep, None, None)
    assert rc == 1
    rc = lib.b200fp8_gemm_rowcol_epilogue(64, 64, 64, a.data_ptr(), 0, 64, b.data_ptr(), 0, 64, d.data_ptr(), 9, 64,
                                          None, None, None)
    assert rc == 1
