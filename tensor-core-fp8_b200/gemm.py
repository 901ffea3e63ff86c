"""Host-side mirror of the reference's operator API for the FP8 GEMM path.

Reference: ``gemm::GEMM`` / ``gemm::GEMM4`` (GEMM/include/gemm.cuh:12-55), called
by ``BmFN`` (GEMM/gemm_main.cpp:77, :123).  Same names, same argument order
``(m, k, n, a, b, out)``, same layouts: ``a`` is row-major M x K, ``b`` is
"column-major K x N" = N rows of K elements, ``out`` is row-major M x N FP32.  The dtype
pair is taken from the tensors (``torch.float8_e4m3fn`` / ``torch.float8_e5m2``), which
is what the C++ overload set does with the pointer types.

torch is used only for device memory and streams; the computation is the CUDA library
behind include/b200fp8.h.  Errors surface as ``B200Fp8Error`` carrying the cudaError_t
value the reference's functions would have returned.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi
from ._cabi import (E4M3, E5M2, KERNEL_AUTO, KERNEL_CTA1_N128, KERNEL_CTA1_N256, KERNEL_PAIR_N256,  # noqa: F401
                    KERNEL_CTA1_N64, KERNEL_PAIR_N128, KERNEL_PAIR_N512, KERNEL_SKINNY, KERNEL_SKINNY_STREAMK,
                    B200Fp8Error, Options)

_DTYPES = {torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"expected float8_e4m3fn or float8_e5m2, got {t.dtype}") from None


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_extent(name: str, t: torch.Tensor, rows: int, cols: int, ld: int) -> None:
    """The C ABI sees only pointers: a matrix that is too small, transposed or strided along its rows would make a
    kernel read or write outside the allocation, so the extents are proven here, before the call."""
    if rows < 0 or cols < 0:
        raise ValueError(f"{name}: negative extent")
    if rows == 0 or cols == 0:
        return
    if t.dim() > 2 or (t.dim() >= 1 and t.stride(-1) != 1 and t.shape[-1] > 1):
        raise ValueError(f"{name}: the last dimension must be contiguous (stride 1), got strides {tuple(t.stride())}")
    if ld < cols:
        raise ValueError(f"{name}: leading dimension {ld} is smaller than its {cols} columns")
    need = (rows - 1) * ld + cols
    # elements reachable from data_ptr() through the tensor's own shape and strides (a view of a wider buffer has a pitch)
    span = 1 + sum((sz - 1) * st for sz, st in zip(t.shape, t.stride())) if t.numel() else 0
    if need > span:
        raise ValueError(f"{name}: needs {need} elements ({rows} rows of {cols}, pitch {ld}) but the tensor spans {span}")


def _check_operands(m, k, n, a, b, out, lda, ldb, ldc, out_name="out"):
    if not (a.is_cuda and b.is_cuda and out.is_cuda):
        raise ValueError("a, b and out must be CUDA tensors (device pointers, as in the reference)")
    if not (a.device == b.device == out.device):
        raise ValueError(f"a, b and {out_name} must live on one device, got {a.device}, {b.device}, {out.device}")
    _check_extent("a", a, m, k, lda)
    _check_extent("b", b, n, k, ldb)
    _check_extent(out_name, out, m, n, ldc)


def _gemm(m, k, n, a, b, out, depth, kernel=KERNEL_AUTO, split_k=0, max_ctas=0, lda=None, ldb=None, ldc=None):
    if out.dtype != torch.float32:
        raise TypeError("out must be float32")
    _check_operands(m, k, n, a, b, out, k if lda is None else lda, k if ldb is None else ldb, n if ldc is None else ldc)
    opt = Options(ctypes.sizeof(Options), depth, kernel, split_k, max_ctas)
    with torch.cuda.device(out.device):
        rc = _cabi.lib().b200fp8_gemm_rowcol_f32_ex(
            m, k, n, a.data_ptr(), dtype_code(a), k if lda is None else lda, b.data_ptr(), dtype_code(b),
            k if ldb is None else ldb, out.data_ptr(), n if ldc is None else ldc, ctypes.byref(opt),
            _stream_ptr(out.device))
    _cabi.check(rc, f"GEMM m={m} k={k} n={n}")
    return out


def GEMM(m: int, k: int, n: int, a_matrix: torch.Tensor, b_matrix: torch.Tensor, output_matrix: torch.Tensor):
    """``gemm::GEMM`` (GEMM/include/gemm.cuh:12-15 and its three dtype overloads): the "2-stage" entry."""
    return _gemm(m, k, n, a_matrix, b_matrix, output_matrix, depth=2)


def GEMM4(m: int, k: int, n: int, a_matrix: torch.Tensor, b_matrix: torch.Tensor, output_matrix: torch.Tensor):
    """``gemm::GEMM4`` (GEMM/include/gemm.cuh:18-21 and overloads): the "4-stage" entry."""
    return _gemm(m, k, n, a_matrix, b_matrix, output_matrix, depth=4)


def gemm_ex(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, depth: int = 0,
            kernel: int = KERNEL_AUTO, split_k: int = 0, max_ctas: int = 0, ldc: int | None = None):
    """Extended form: shapes from the tensors (a: [M, K], b: [N, K]); ring depth 0 = as deep as fits."""
    m, k = a.shape
    n, k2 = b.shape
    if k != k2:
        raise ValueError("a and b disagree on K")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    if tuple(out.shape) != (m, n):
        raise ValueError(f"out must be [{m}, {n}], got {tuple(out.shape)}")
    return _gemm(m, k, n, a, b, out, depth, kernel, split_k, max_ctas, a.stride(0) if m > 1 else k,
                 b.stride(0) if n > 1 else k, ldc if ldc is not None else (out.stride(0) if m > 1 else n))


OUT_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def gemm_scaled(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, *, alpha: float = 1.0, beta: float = 0.0,
                a_scale: torch.Tensor | None = None, b_scale: torch.Tensor | None = None, depth: int = 0,
                kernel: int = KERNEL_AUTO, split_k: int = 0, max_ctas: int = 0):
    """D = alpha * a_scale * b_scale * (A B^T) + beta * D, D float32 / bfloat16 / float16 (updated in place).

    The epilogue of the reference's cuBLASLt comparator (GEMM/src/cublas.cu:37-53): alpha, beta and
    per-tensor scale pointers (one-element float32 CUDA tensors here, or None).
    """
    m, k = a.shape
    n, k2 = b.shape
    if k != k2 or d.shape != (m, n):
        raise ValueError("shape mismatch")
    if d.dtype not in OUT_DTYPES:
        raise TypeError("d must be float32, bfloat16 or float16")
    for s_ in (a_scale, b_scale):
        if s_ is not None and (s_.dtype != torch.float32 or not s_.is_cuda or s_.numel() != 1):
            raise TypeError("scales are one-element float32 CUDA tensors")
    _check_operands(m, k, n, a, b, d, a.stride(0) if m > 1 else k, b.stride(0) if n > 1 else k, d.stride(0) if m > 1 else n, "d")
    opt = Options(ctypes.sizeof(Options), depth, kernel, split_k, max_ctas)
    with torch.cuda.device(d.device):
        rc = _cabi.lib().b200fp8_gemm_rowcol_scaled(
            m, k, n, a.data_ptr(), dtype_code(a), a.stride(0) if m > 1 else k, b.data_ptr(), dtype_code(b),
            b.stride(0) if n > 1 else k, d.data_ptr(), OUT_DTYPES[d.dtype], d.stride(0) if m > 1 else n,
            float(alpha), float(beta), a_scale.data_ptr() if a_scale is not None else None,
            b_scale.data_ptr() if b_scale is not None else None, ctypes.byref(opt), _stream_ptr(d.device))
    _cabi.check(rc, "gemm_scaled")
    return d


EPILOGUE_OUT_DTYPES = {**OUT_DTYPES, torch.float8_e4m3fn: 3, torch.float8_e5m2: 4}


ACTIVATIONS = {"none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3}     # B200FP8_ACT_* of include/b200fp8.h


def gemm_epilogue(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, *, alpha: float = 1.0, beta: float = 0.0,
                  a_scale: torch.Tensor | None = None, b_scale: torch.Tensor | None = None,
                  d_scale: torch.Tensor | None = None, amax_d: torch.Tensor | None = None,
                  bias: torch.Tensor | None = None, a_row_scale: torch.Tensor | None = None,
                  b_row_scale: torch.Tensor | None = None, activation: str | int = 0, depth: int = 0,
                  kernel: int = KERNEL_AUTO, split_k: int = 0, max_ctas: int = 0):
    """t = act(alpha * a_scale * b_scale * a_row_scale[m] * b_row_scale[n] * (A B^T) + beta * D + bias[n]);
    amax_d = max |t|;  D = convert(d_scale * t).

    a_row_scale (M float32 values) and b_row_scale (N) are per-row scales of row-wise quantised operands;
    activation is "none", "relu", "gelu" (erf form) or "gelu_tanh", applied after the bias.

    The whole epilogue of the reference's cuBLASLt comparator (GEMM/src/cublas.cu:37-53; amax and scale slots in
    GEMM/include/helper.h:59-66).  D may be float32, bfloat16, float16, float8_e4m3fn or float8_e5m2 (8-bit outputs
    round to nearest even and saturate to finite).  Scales and amax_d are one-element float32 CUDA tensors; bias has
    N elements of float32, bfloat16 or float16.
    """
    m, k = a.shape
    n, k2 = b.shape
    if k != k2 or d.shape != (m, n):
        raise ValueError("shape mismatch")
    if d.dtype not in EPILOGUE_OUT_DTYPES:
        raise TypeError("d must be float32, bfloat16, float16, float8_e4m3fn or float8_e5m2")
    for s_ in (a_scale, b_scale, d_scale, amax_d):
        if s_ is not None and (s_.dtype != torch.float32 or not s_.is_cuda or s_.numel() != 1):
            raise TypeError("scales and amax are one-element float32 CUDA tensors")
    if bias is not None and (bias.dtype not in OUT_DTYPES or not bias.is_cuda or bias.numel() != n or not bias.is_contiguous()):
        raise TypeError("bias is a contiguous CUDA vector of N float32 / bfloat16 / float16 values")
    for v_, rows, what in ((a_row_scale, m, "a_row_scale has M"), (b_row_scale, n, "b_row_scale has N")):
        if v_ is not None and (v_.dtype != torch.float32 or not v_.is_cuda or v_.numel() != rows or not v_.is_contiguous()
                               or v_.device != d.device):
            raise TypeError(f"{what} contiguous float32 values on the device of d")
    if isinstance(activation, str):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation is one of {sorted(ACTIVATIONS)}")
        activation = ACTIVATIONS[activation]
    if activation not in ACTIVATIONS.values():
        raise ValueError("unknown activation")
    _check_operands(m, k, n, a, b, d, a.stride(0) if m > 1 else k, b.stride(0) if n > 1 else k, d.stride(0) if m > 1 else n, "d")
    ptr = lambda t: t.data_ptr() if t is not None else None
    ep = _cabi.EpilogueDesc(ctypes.sizeof(_cabi.EpilogueDesc), float(alpha), float(beta), ptr(a_scale), ptr(b_scale),
                            ptr(d_scale), ptr(amax_d), ptr(bias), OUT_DTYPES[bias.dtype] if bias is not None else 0,
                            int(activation), ptr(a_row_scale), ptr(b_row_scale))
    opt = Options(ctypes.sizeof(Options), depth, kernel, split_k, max_ctas)
    with torch.cuda.device(d.device):
        rc = _cabi.lib().b200fp8_gemm_rowcol_epilogue(
            m, k, n, a.data_ptr(), dtype_code(a), a.stride(0) if m > 1 else k, b.data_ptr(), dtype_code(b),
            b.stride(0) if n > 1 else k, d.data_ptr(), EPILOGUE_OUT_DTYPES[d.dtype], d.stride(0) if m > 1 else n,
            ctypes.byref(ep), ctypes.byref(opt), _stream_ptr(d.device))
    _cabi.check(rc, "gemm_epilogue")
    return d


ELL_BLOCK = 128     # rows and columns of a blocked-ELL block


def gemv(b: torch.Tensor, x: torch.Tensor, y: torch.Tensor):
    """y[n] = sum_k B[n][k] x[k]: the GEMV of the reference's roadmap (README.md:7) = the operator with M = 1."""
    n, k = b.shape
    if x.numel() != k or y.numel() != n or y.dtype != torch.float32 or not (x.is_contiguous() and y.is_contiguous()):
        raise ValueError("x has K elements, y has N float32 elements, both contiguous")
    if b.dim() != 2 or (k > 1 and b.stride(1) != 1) or not (b.is_cuda and x.is_cuda and y.is_cuda) or not (b.device == x.device == y.device):
        raise ValueError("b is a CUDA matrix [N][K] with contiguous rows, on the device of x and y")
    with torch.cuda.device(y.device):
        rc = _cabi.lib().b200fp8_gemv_f32(n, k, b.data_ptr(), dtype_code(b), b.stride(0) if n > 1 else k, x.data_ptr(),
                                           dtype_code(x), y.data_ptr(), _stream_ptr(y.device))
    _cabi.check(rc, f"gemv n={n} k={k}")
    return y


def _check_bell(values: torch.Tensor, col_ind: torch.Tensor, m: int):
    if col_ind.dtype != torch.int32 or not col_ind.is_cuda or not col_ind.is_contiguous() or col_ind.dim() != 2:
        raise TypeError("col_ind is a contiguous int32 CUDA matrix [ceil(M/128)][blocks per row]")
    blocks = col_ind.shape[1]
    if col_ind.shape[0] != (m + ELL_BLOCK - 1) // ELL_BLOCK or values.shape[1] != blocks * ELL_BLOCK:
        raise ValueError("values is [M][blocks * 128], col_ind is [ceil(M/128)][blocks]")
    return blocks


def spmm_bell(values: torch.Tensor, col_ind: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, depth: int = 0,
              kernel: int = KERNEL_AUTO, max_ctas: int = 0):
    """C = A_sparse B^T with A in blocked-ELL form, 128 x 128 blocks (the format of GenerateUniformBlockedELLIndex,
    GEMM/include/bm_test_utils.h:48-70): values [M][blocks * 128] FP8, col_ind [ceil(M/128)][blocks] int32
    block-column indices (negative = padding block), b [N][K] FP8, out [M][N] float32."""
    m = values.shape[0]
    n, k = b.shape
    blocks = _check_bell(values, col_ind, m)
    if out.shape != (m, n) or out.dtype != torch.float32:
        raise ValueError("out is [M][N] float32")
    opt = Options(ctypes.sizeof(Options), depth, kernel, 0, max_ctas)
    with torch.cuda.device(out.device):
        rc = _cabi.lib().b200fp8_spmm_bell_rowcol_f32(
            m, k, n, values.data_ptr(), dtype_code(values), values.stride(0) if m > 1 else blocks * ELL_BLOCK,
            col_ind.data_ptr(), blocks, b.data_ptr(), dtype_code(b), b.stride(0) if n > 1 else k, out.data_ptr(),
            out.stride(0) if m > 1 else n, ctypes.byref(opt), _stream_ptr(out.device))
    _cabi.check(rc, f"spmm_bell m={m} k={k} n={n} blocks={blocks}")
    return out


def spmv_bell(values: torch.Tensor, col_ind: torch.Tensor, x: torch.Tensor, y: torch.Tensor, *, split_k: int = 0,
              kernel: int = KERNEL_AUTO):
    """y = A_sparse x with A in blocked-ELL form as in spmm_bell; x has K FP8 elements, y has M float32 elements."""
    m = values.shape[0]
    k = x.numel()
    blocks = _check_bell(values, col_ind, m)
    if y.numel() != m or y.dtype != torch.float32 or not (x.is_contiguous() and y.is_contiguous()):
        raise ValueError("y has M float32 elements; x and y are contiguous")
    opt = Options(ctypes.sizeof(Options), 0, kernel, split_k, 0)
    with torch.cuda.device(y.device):
        rc = _cabi.lib().b200fp8_spmv_bell_f32(
            m, k, values.data_ptr(), dtype_code(values), values.stride(0) if m > 1 else blocks * ELL_BLOCK,
            col_ind.data_ptr(), blocks, x.data_ptr(), dtype_code(x), y.data_ptr(), ctypes.byref(opt), _stream_ptr(y.device))
    _cabi.check(rc, f"spmv_bell m={m} k={k} blocks={blocks}")
    return y


def gemm_host(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, depth: int = 0):
    """BmFN's whole sequence with HOST tensors (GEMM/gemm_main.cpp:56-64, :77, :161): upload, run, download."""
    if a.is_cuda or b.is_cuda or out.is_cuda:
        raise ValueError("gemm_host takes host tensors")
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("a is [M][K], b is [N][K]")
    m, k = a.shape
    n, k2 = b.shape
    if k != k2:
        raise ValueError("a and b disagree on K")
    if out.dtype != torch.float32 or tuple(out.shape) != (m, n):
        raise ValueError(f"out must be float32 [{m}, {n}], got {out.dtype} {tuple(out.shape)}")
    if not (a.is_contiguous() and b.is_contiguous() and out.is_contiguous()):
        raise ValueError("gemm_host takes contiguous tensors (lda = ldb = K, ldc = N)")
    rc = _cabi.lib().b200fp8_gemm_rowcol_f32_host(m, k, n, a.data_ptr(), dtype_code(a), b.data_ptr(), dtype_code(b),
                                                   out.data_ptr(), depth)
    _cabi.check(rc, f"gemm_host m={m} k={k} n={n}")
    return out


def fill_normal(t: torch.Tensor, sigma: float, seed: int, index_offset: int = 0):
    """Seeded synthetic operand: t[i] = fp8(sigma * N(0,1)), RNE + saturate-to-finite, keyed by (seed, index)."""
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    with torch.cuda.device(t.device):
        rc = _cabi.lib().b200fp8_fill_normal(t.data_ptr(), t.numel(), dtype_code(t), float(sigma), int(seed),
                                              int(index_offset), _stream_ptr(t.device))
    _cabi.check(rc, "fill_normal")
    return t


def device_status(reset: bool = True) -> int:
    """0 unless a bounded wait inside one of the kernels ran out on the current device."""
    st = ctypes.c_int(-1)
    _cabi.check(_cabi.lib().b200fp8_device_status(ctypes.byref(st), 1 if reset else 0), "device_status")
    return st.value


def launch_count() -> int:
    return int(_cabi.lib().b200fp8_launch_count())
