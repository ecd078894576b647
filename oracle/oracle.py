"""ORACLE -- TEST INFRASTRUCTURE ONLY.

CPU checkers for the FP32 GEMM path. Only tests/, __graft_entry__.smoke() and
the CPU-baseline leg of bench.py may import this module, and only to CHECK or
to time a baseline; the product never routes through it.

Three checkers:
  * host_gemm / host_gemm_f64: the C restatement in oracle/host_gemm.c of the
    reference kernel's arithmetic (src/primitive/hygon/gemm/fp32_gemm.hip:24-30,
    tests/api/gemm_numerics_test.cpp:30-51 of the reference).
  * torch_reference: the reference's own PyTorch reference expression
    `alpha * (a @ b) + beta * c` (tests/python/torch_gemm_test.py:40,
    benchmarks/ftrain_bench/ops/gemm.py:39 of the reference), on CPU tensors.
  * reference_library: the reference's own C++/kernel sources compiled for the
    CPU (oracle/_ref, built by oracle/build_oracle.py where the reference
    checkout exists).

Parity is pinned: tests/test_oracle.py checks host_gemm against the golden
vectors of the reference's tests and against outputs of reference_library
committed under tests/golden/.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


class _Strides(ctypes.Structure):
    _fields_ = [("row", ctypes.c_int64), ("col", ctypes.c_int64)]


def _library() -> ctypes.CDLL:
    path = HERE / "libftoracle.so"
    if not path.exists():
        from . import build_oracle

        build_oracle.build_restatement()
    lib = ctypes.CDLL(str(path))
    pointer = ctypes.c_void_p
    common = [pointer, _Strides, pointer, _Strides, pointer, _Strides]
    lib.ftoracle_gemm_f32.argtypes = common + [pointer, _Strides] + [ctypes.c_int64] * 3 + [ctypes.c_float] * 2
    lib.ftoracle_gemm_f32_fma.argtypes = lib.ftoracle_gemm_f32.argtypes
    lib.ftoracle_gemm_f64.argtypes = common + [pointer] + [ctypes.c_int64] * 3 + [ctypes.c_float] * 2
    lib.ftoracle_fill.argtypes = [pointer, ctypes.c_uint64, ctypes.c_uint64]
    lib.ftoracle_element_value.argtypes = [ctypes.c_uint64]
    lib.ftoracle_element_value.restype = ctypes.c_float
    for name in ("ftoracle_gemm_f32", "ftoracle_gemm_f32_fma", "ftoracle_gemm_f64", "ftoracle_fill"):
        getattr(lib, name).restype = None
    return lib


_lib = _library()


def _strides(array: np.ndarray) -> _Strides:
    assert array.dtype == np.float32 and array.ndim == 2
    return _Strides(array.strides[0] // 4, array.strides[1] // 4)


def fill(count: int, offset: int = 0) -> np.ndarray:
    """The reference test's deterministic values in [-0.5, 0.5): element i = value(i + offset)."""
    out = np.empty(count, dtype=np.float32)
    _lib.ftoracle_fill(out.ctypes.data, count, offset)
    return out


def grid_inputs(m: int, k: int, n: int):
    """a, b, c of the reference's numerics grid (gemm_numerics_test.cpp:72-78)."""
    return (fill(m * k).reshape(m, k), fill(k * n, 7919).reshape(k, n), fill(m * n, 104729).reshape(m, n))


def host_gemm(a: np.ndarray, b: np.ndarray, c: np.ndarray | None, alpha: float, beta: float,
              fma: bool = False) -> np.ndarray:
    """FP32, sequential over k. Accepts any 2-D float32 views (strides honoured)."""
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    d = np.empty((m, n), dtype=np.float32)
    function = _lib.ftoracle_gemm_f32_fma if fma else _lib.ftoracle_gemm_f32
    c_pointer = c.ctypes.data if c is not None else None
    c_strides = _strides(c) if c is not None else _Strides(0, 0)
    function(a.ctypes.data, _strides(a), b.ctypes.data, _strides(b), c_pointer, c_strides, d.ctypes.data, _strides(d),
             m, n, k, alpha, beta)
    return d


def host_gemm_f64(a: np.ndarray, b: np.ndarray, c: np.ndarray | None, alpha: float, beta: float) -> np.ndarray:
    m, k = a.shape
    _, n = b.shape
    d = np.empty((m, n), dtype=np.float64)
    c_pointer = c.ctypes.data if c is not None else None
    c_strides = _strides(c) if c is not None else _Strides(0, 0)
    _lib.ftoracle_gemm_f64(a.ctypes.data, _strides(a), b.ctypes.data, _strides(b), c_pointer, c_strides,
                           d.ctypes.data, m, n, k, alpha, beta)
    return d


def torch_reference(a, b, c=None, alpha: float = 1.0, beta: float = 0.0):
    """The reference's PyTorch expression; dtype and device follow the inputs."""
    out = alpha * (a @ b)
    if c is not None:
        out = out + beta * c
    return out


def scaled_error(x, exact64, a, b, c=None, beta: float = 0.0) -> float:
    """max_ij |x_ij - exact_ij| / (||a_i,:||_2 * ||b_:,j||_2 + |beta| |c_ij|).

    The yardstick of the accuracy bar: a kernel passes when its scaled error is
    at most twice that of torch's FP32 matmul on the same inputs. Works on
    numpy arrays or torch tensors (any device); norms are taken in float64.
    """
    import torch

    def as_tensor(value):
        return value if isinstance(value, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(value))

    x, exact64, a, b = (as_tensor(v) for v in (x, exact64, a, b))
    row_norms = a.double().norm(dim=1, keepdim=True)
    col_norms = b.double().norm(dim=0, keepdim=True)
    scale = row_norms * col_norms
    if c is not None and beta != 0.0:
        scale = scale + abs(beta) * as_tensor(c).double().abs()
    scale = scale + 1e-300
    return float(((x.double() - exact64.double()).abs() / scale).max())


def within_reference_tolerance(actual: np.ndarray, expected: np.ndarray, rel: float = 2e-5, abs_: float = 2e-5):
    """The reference numerics test's criterion (tests/support/numerics.hpp:72-101):
    |actual - expected| <= abs + rel * |expected| element-wise. Returns (ok, worst ratio)."""
    diff = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    allowed = abs_ + rel * np.abs(expected.astype(np.float64))
    ratio = float((diff / allowed).max()) if diff.size else 0.0
    return ratio <= 1.0, ratio


def reference_library_path() -> str | None:
    """Path of the CPU build of the reference's own sources, if it exists."""
    path = HERE / "_ref" / "libflash_train_ref.so"
    return str(path) if path.exists() else None
