"""Pins the CPU oracle: against the reference tests' known answers, against
outputs of the reference's own code (tests/golden/reference_grid.npz, and live
when oracle/_ref exists) and against the reference's PyTorch expression."""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).parent / "golden"
GRID = [(1, 1, 1), (3, 4, 2), (16, 16, 16), (64, 48, 32), (129, 65, 17), (33, 257, 65), (256, 128, 64)]


def test_known_answer_2x2(oracle):
    # ftrainGemm known answer of the reference, tests/api/gemm_api_test.cpp:392-438.
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    c = np.zeros((2, 2), np.float32)
    for fma in (False, True):
        d = oracle.host_gemm(a, b, c, 2.0, 0.5, fma=fma)
        assert d.tolist() == [[38.0, 44.0], [86.0, 100.0]]


def test_fill_rule(oracle):
    # tests/api/gemm_numerics_test.cpp:30-32: ((i * 2654435761) % 199) / 199 - 0.5.
    values = oracle.fill(1000, offset=7919)
    expected = np.array([np.float32(((i + 7919) * 2654435761 % 2**64) % 199) / np.float32(199.0) - np.float32(0.5)
                         for i in range(1000)], np.float32)
    assert np.array_equal(values, expected)
    assert values.min() >= -0.5 and values.max() < 0.5


@pytest.mark.parametrize("shape", GRID, ids=lambda s: "x".join(map(str, s)))
def test_matches_committed_reference_outputs(oracle, shape):
    m, k, n = shape
    golden = np.load(GOLDEN / "reference_grid.npz")
    a, b, c = oracle.grid_inputs(m, k, n)
    for key, c_operand, beta in ((f"fresh_{m}x{k}x{n}", None, 0.0), (f"accumulated_{m}x{k}x{n}", c, 1.25)):
        reference = golden[key]
        ok, ratio = oracle.within_reference_tolerance(oracle.host_gemm(a, b, c_operand, 1.5, beta), reference)
        assert ok, f"{key}: worst ratio {ratio}"
        # One of the two rounding variants is the reference build's arithmetic, bit for bit.
        exact = [np.array_equal(oracle.host_gemm(a, b, c_operand, 1.5, beta, fma=fma), reference) for fma in (False, True)]
        assert any(exact), f"{key}: neither the fused nor the unfused variant reproduces the reference bits"


def test_matches_live_reference_library(oracle, reference_capi, capi):
    if reference_capi is None:
        pytest.skip("no reference checkout in this environment (golden fixtures cover it)")
    binding = capi.GemmBinding(lib=reference_capi)
    rng = np.random.default_rng(5)
    for m, k, n in [(5, 7, 3), (31, 64, 33)]:
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)
        c = rng.standard_normal((m, n), dtype=np.float32)
        d = np.zeros((m, n), np.float32)
        op = lambda x: (x.ctypes.data, x.shape, None)  # noqa: E731
        plan = binding.make_plan(op(a), op(b), op(c), op(d), -0.75, 2.0)
        assert plan.primitive_names() == ["Fp32Gemm"]
        plan.execute()
        ok, ratio = oracle.within_reference_tolerance(oracle.host_gemm(a, b, c, -0.75, 2.0), d, 1e-6, 1e-6)
        assert ok, ratio


def test_strided_views_and_float64(oracle):
    rng = np.random.default_rng(1)
    buffer = rng.standard_normal((9, 6), dtype=np.float32)
    a = buffer.T  # 6 x 9 view with strides (1, 6)
    b = rng.standard_normal((9, 4), dtype=np.float32)
    expected = a.astype(np.float64) @ b.astype(np.float64)
    assert np.allclose(oracle.host_gemm(a, b, None, 1.0, 0.0), expected, atol=1e-5)
    assert np.allclose(oracle.host_gemm_f64(a, b, None, 1.0, 0.0), expected, atol=1e-12)


def test_torch_expression_on_config1(oracle):
    # Config 1: m=128 k=64 n=96, N(0,1) from seed 0, alpha=1, beta=0, no C.
    torch = pytest.importorskip("torch")
    golden = np.load(GOLDEN / "torch_config1.npz")
    a = torch.from_numpy(golden["a"])
    b = torch.from_numpy(golden["b"])
    d = oracle.torch_reference(a, b)
    assert torch.allclose(d, torch.from_numpy(golden["d32"]), rtol=1e-5, atol=1e-5)
    ours = oracle.host_gemm(golden["a"], golden["b"], None, 1.0, 0.0)
    error_ours = oracle.scaled_error(ours, golden["d64"], golden["a"], golden["b"])
    error_torch = oracle.scaled_error(golden["d32"], golden["d64"], golden["a"], golden["b"])
    assert error_ours < 1e-6 and error_torch < 1e-6
    # Empty and degenerate shapes.
    assert oracle.host_gemm(np.zeros((0, 3), np.float32), np.zeros((3, 4), np.float32), None, 1.0, 0.0).shape == (0, 4)
    c = np.full((2, 2), 3.0, np.float32)
    assert np.array_equal(oracle.host_gemm(np.zeros((2, 0), np.float32), np.zeros((0, 2), np.float32), c, 1.0, 0.5),
                          np.full((2, 2), 1.5, np.float32))
