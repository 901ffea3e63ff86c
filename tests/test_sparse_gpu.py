"""GPU tests of GEMV, blocked-ELL SpMM and SpMV (the kernels after GEMM on the reference's roadmap, README.md:7)
against the CPU oracle: the blocked-ELL operand is expanded to a dense byte matrix on the host and the FP64 oracle
and the path's tolerance |C - C_ref| <= 1e-3 * sum|a b| + 1e-6 judge the result.  Where the summation order is the
same as the dense kernel's (SpMM with ascending block columns: absent blocks only add exact zeros) the result must
equal the dense operator's bit for bit."""
import numpy as np
import pytest
import torch

from __graft_entry__ import load_package

pytestmark = pytest.mark.gpu

F8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}


@pytest.fixture(scope="module")
def g():
    assert torch.cuda.is_available()
    pkg = load_package()
    pkg._cabi.lib()          # the library must be present: there is no fallback
    torch.cuda.set_device(0)
    return pkg.gemm


def dev(x_np, fmt):
    return torch.from_numpy(np.ascontiguousarray(x_np)).cuda().view(F8[fmt])


def check(oracle, C, A, fa, B, fb):
    C64, S = oracle.gemm_f64(A, fa, B, fb)
    bad, worst, wi = oracle.check_tolerance(C, C64, S)
    assert bad == 0, f"{bad} elements outside tolerance, worst ratio {worst} at flat index {wi}"


@pytest.mark.parametrize("fa,fb", [(0, 0), (1, 0), (0, 1)])
@pytest.mark.parametrize("kernel,m,k,n,blocks", [(0, 384, 1024, 640, 3), (1, 300, 1040, 500, 4), (2, 130, 2048, 129, 16),
                                                 (1, 256, 128 * 80, 256, 70), (2, 128, 256, 128, 2), (0, 1024, 4096, 2048, 8)])
def test_spmm_against_oracle_and_dense_operator(g, oracle, fa, fb, kernel, m, k, n, blocks):
    vals, ind = oracle.make_bell_uniform(m, k, blocks, fa, seed=100 + m + blocks, sigma=2.0 if fa else 1.0)
    B = oracle.fill_normal(n * k, fb, 2.0 if fb else 1.0, 7).reshape(n, k)
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.spmm_bell(dev(vals, fa), torch.from_numpy(ind).cuda(), dev(B, fb), out, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    dense = oracle.bell_to_dense(vals, ind, k)
    check(oracle, out.cpu().numpy(), dense, fa, B, fb)
    # same kernel on the expanded matrix: identical summation order, so identical bits
    kdense = kernel if kernel else (1 if ((m + 127) // 128) * ((n + 255) // 256) >= 74 else 2)
    ref = torch.empty_like(out)
    g.gemm_ex(dev(dense, fa), dev(B, fb), ref, kernel=kdense)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_spmm_padding_blocks_contribute_nothing(g, oracle):
    m, k, n, blocks = 384, 1024, 256, 4
    vals, ind = oracle.make_bell_uniform(m, k, blocks, 0, seed=5)
    ind[0, 3] = -1                      # a padding block in the cuSPARSE convention
    ind[1, 2] = ind[1, 3]; ind[1, 3] = 1 << 20      # far beyond K: also padding
    ind[2, 3] = -7
    vals[0:128, 3 * 128:] = 0x7F        # NaN bytes in a padding block must not reach C
    vals[256:384, 3 * 128:] = 0x7E      # 448, the largest finite value
    B = oracle.fill_normal(n * k, 0, 1.0, 9).reshape(n, k)
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.spmm_bell(dev(vals, 0), torch.from_numpy(ind).cuda(), dev(B, 0), out)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    check(oracle, out.cpu().numpy(), oracle.bell_to_dense(vals, ind, k), 0, B, 0)


def test_spmm_without_blocks_is_zero_and_bad_arguments_are_refused(g, oracle):
    pkg = load_package()
    m, k, n = 256, 512, 128
    B = dev(oracle.fill_normal(n * k, 0, 1.0, 9).reshape(n, k), 0)
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    vals = torch.empty((m, 0), dtype=F8[0], device="cuda")
    ind = torch.empty((2, 0), dtype=torch.int32, device="cuda")
    g.spmm_bell(vals, ind, B, out)
    torch.cuda.synchronize()
    assert not out.any()
    vals, ind_np = oracle.make_bell_uniform(m, k, 2, 0, seed=1)
    with pytest.raises(pkg._cabi.B200Fp8Error):          # a CTA pair cannot follow two block rows
        g.spmm_bell(dev(vals, 0), torch.from_numpy(ind_np).cuda(), B, out, kernel=3)
    with pytest.raises(ValueError):
        g.spmm_bell(dev(vals, 0), torch.from_numpy(ind_np[:1]).cuda(), B, out)
    with pytest.raises(TypeError):
        g.spmm_bell(dev(vals, 0), torch.from_numpy(ind_np.astype(np.int64)).cuda(), B, out)


@pytest.mark.parametrize("fa,fx", [(0, 0), (1, 1), (0, 1)])
@pytest.mark.parametrize("m,k,blocks,split_k", [(1024, 4096, 8, 0), (300, 1040, 5, 0), (128, 128 * 80, 70, 1), (8192, 8192, 16, 0),
                                                (130, 256, 1, 0), (4096, 128 * 96, 96, 2)])
@pytest.mark.parametrize("kernel", [0, 8], ids=["clustered", "stream-k"])
def test_spmv_against_oracle(g, oracle, fa, fx, m, k, blocks, split_k, kernel):
    vals, ind = oracle.make_bell_uniform(m, k, blocks, fa, seed=m + blocks, sigma=2.0 if fa else 1.0)
    if blocks > 2:
        ind[0, -1] = -1                 # one padding block
    x = oracle.fill_normal(k, fx, 2.0 if fx else 1.0, 3).reshape(1, k)
    y = torch.full((m,), float("nan"), dtype=torch.float32, device="cuda")
    g.spmv_bell(dev(vals, fa), torch.from_numpy(ind).cuda(), dev(x, fx).reshape(k), y, split_k=split_k, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    dense = oracle.bell_to_dense(vals, ind, k)
    check(oracle, y.cpu().numpy().reshape(m, 1), dense, fa, x, fx)


@pytest.mark.parametrize("fb,fx", [(0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("n,k", [(8192, 8192), (1000, 1040), (130, 16), (57344, 2048)])
def test_gemv_against_oracle_and_m1_operator(g, oracle, fb, fx, n, k):
    B = oracle.fill_normal(n * k, fb, 2.0 if fb else 1.0, 5).reshape(n, k)
    x = oracle.fill_normal(k, fx, 2.0 if fx else 1.0, 6).reshape(1, k)
    y = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    g.gemv(dev(B, fb), dev(x, fx).reshape(k), y)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    check(oracle, y.cpu().numpy().reshape(1, n), x, fx, B, fb)
    ref = torch.empty((1, n), dtype=torch.float32, device="cuda")
    g.gemm_ex(dev(x, fx), dev(B, fb), ref)
    torch.cuda.synchronize()
    assert torch.equal(y.reshape(1, n), ref)
