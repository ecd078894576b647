"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU
oracle, the committed golden vectors and a float64 reference.

Tolerances
  * exact-FP32 kernels vs the oracle: the reference's own criterion,
    |d - ref| <= 2e-5 + 2e-5 |ref| (tests/api/gemm_numerics_test.cpp:55-59 there).
  * every kernel vs float64: scaled error
        max |d - d64| / (||a_row|| * ||b_col|| + |beta c|)
    at most 2x that of torch's FP32 matmul on the same inputs (with a floor of
    2^-24 so that a lucky torch result on a tiny case cannot fail the test).
"""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).parent / "golden"
GRID = [(1, 1, 1), (3, 4, 2), (16, 16, 16), (64, 48, 32), (129, 65, 17), (33, 257, 65), (256, 128, 64)]
ERROR_FLOOR = 2.0 ** -24


@pytest.fixture(scope="module")
def gpu(capi):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    torch.backends.cuda.matmul.allow_tf32 = False
    import gpu_support

    return gpu_support


def platform_gemm(capi, gpu, kernel, a, b, c, alpha, beta, d=None):
    """Runs one kernel family through ftcuda_gemm_configure / ftcuda_gemm_launch."""
    import os

    if kernel in (capi.KERNEL_TF32X3, capi.KERNEL_TF32X3_SPLITK, capi.KERNEL_TF32X3_ROWS) and os.environ.get("FT_SKIP_TENSOR"):
        return None, "tensor-core kernels switched off by FT_SKIP_TENSOR"
    m, n = a.shape[0], b.shape[1]
    if d is None:
        d = torch.full((m, n), float("nan"), device="cuda")
    c_operand = gpu.operand(c) if c is not None else capi.null_operand(m, n)
    desc = capi.make_desc(gpu.operand(a), gpu.operand(b), c_operand, gpu.operand(d), alpha, beta,
                          torch.cuda.current_device())
    reason = capi.platform_supports(kernel, desc)
    if reason is not None:
        return None, reason
    launch = capi.PlatformGemm(kernel, desc)
    workspace = torch.empty(max(launch.workspace_bytes, 1), dtype=torch.uint8, device="cuda")
    launch.run(workspace.data_ptr(), launch.workspace_bytes, gpu.current_stream())
    torch.cuda.synchronize()
    return d, None


def check_against_float64(oracle, d, a, b, c, alpha, beta, what):
    exact = alpha * (a.double() @ b.double())
    if c is not None:
        exact = exact + beta * c.double()
    plain = alpha * (a @ b)
    if c is not None:
        plain = plain + beta * c
    # alpha scales both the numerator and the row norms' product.
    ours = oracle.scaled_error(d, exact, a * abs(alpha), b, c, beta)
    torch_error = oracle.scaled_error(plain, exact, a * abs(alpha), b, c, beta)
    assert torch.isfinite(d).all(), f"{what}: non-finite output"
    assert ours <= 2.0 * max(torch_error, ERROR_FLOOR), f"{what}: scaled error {ours:.3e} vs torch FP32 {torch_error:.3e}"
    return ours, torch_error


# --------------------------------------------------------------- golden vectors

def test_known_answer_one_shot(capi, gpu):
    # tests/api/gemm_api_test.cpp:392-438 of the reference: exact equality.
    a = torch.tensor([[1.0, 2.0], [3.0, 4.0]], device="cuda")
    b = torch.tensor([[5.0, 6.0], [7.0, 8.0]], device="cuda")
    c = torch.zeros(2, 2, device="cuda")
    d = torch.empty(2, 2, device="cuda")
    capi.gemm_once(gpu.operand(a), gpu.operand(b), gpu.operand(c), gpu.operand(d), 2.0, 0.5, stream=gpu.current_stream())
    torch.cuda.synchronize()
    assert d.cpu().tolist() == [[38.0, 44.0], [86.0, 100.0]]
    assert capi.last_status() == capi.STATUS_SUCCESS and capi.last_message() == ""


@pytest.mark.parametrize("shape", GRID, ids=lambda s: "x".join(map(str, s)))
def test_reference_grid_selected_primitive(capi, gpu, oracle, shape):
    """The reference's numerics test, run as it runs it: staged API, primitive 0."""
    m, k, n = shape
    golden = np.load(GOLDEN / "reference_grid.npz")
    a_h, b_h, c_h = oracle.grid_inputs(m, k, n)
    a, b, c = (torch.from_numpy(x).cuda() for x in (a_h, b_h, c_h))
    fresh, names = gpu.gemm(a, b, None, 1.5, 0.0)
    assert names[-1] == "Fp32Gemm"
    ok, ratio = oracle.within_reference_tolerance(fresh.cpu().numpy(), golden[f"fresh_{m}x{k}x{n}"])
    assert ok, f"fresh {names[0]}: worst ratio {ratio}"
    accumulated, _ = gpu.gemm(a, b, c, 1.5, 1.25)
    ok, ratio = oracle.within_reference_tolerance(accumulated.cpu().numpy(), golden[f"accumulated_{m}x{k}x{n}"])
    assert ok, f"accumulated {names[0]}: worst ratio {ratio}"


@pytest.mark.parametrize("kernel", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("shape", GRID + [(128, 64, 96), (255, 512, 260), (17, 2304, 64), (384, 4100, 516)],
                         ids=lambda s: "x".join(map(str, s)))
def test_every_kernel_family_against_oracle(capi, gpu, oracle, kernel, shape):
    m, k, n = shape
    a_h, b_h, c_h = oracle.grid_inputs(m, k, n)
    a, b, c = (torch.from_numpy(x).cuda() for x in (a_h, b_h, c_h))
    d, reason = platform_gemm(capi, gpu, kernel, a, b, c, 1.5, 1.25)
    if d is None:
        pytest.skip(f"{capi.KERNEL_NAMES[kernel]} declines {shape}: {reason}")
    expected = oracle.host_gemm(a_h, b_h, c_h, 1.5, 1.25, fma=True)
    # K up to 4100 here: the sequential-sum rounding of the oracle itself grows
    # with K, so the absolute part of the reference's tolerance is scaled by
    # sqrt(K / 257) beyond the reference grid's largest K.
    slack = max(1.0, (k / 257.0) ** 0.5)
    ok, ratio = oracle.within_reference_tolerance(d.cpu().numpy(), expected, 2e-5 * slack, 2e-5 * slack)
    assert ok, f"{capi.KERNEL_NAMES[kernel]} {shape}: worst ratio {ratio}"
    # No C: beta must not matter and C must not be read.
    d, _ = platform_gemm(capi, gpu, kernel, a, b, None, -2.0, 7.0)
    expected = oracle.host_gemm(a_h, b_h, None, -2.0, 7.0, fma=True)
    ok, ratio = oracle.within_reference_tolerance(d.cpu().numpy(), expected, 2e-5 * slack, 2e-5 * slack)
    assert ok, f"{capi.KERNEL_NAMES[kernel]} {shape} without C: worst ratio {ratio}"


# --------------------------------------------------------------- API behaviour on a device

def test_rebinding_and_plan_outlives_args(capi, gpu):
    # tests/api/gemm_api_test.cpp:22-138 of the reference: 3x2x4, two data sets, negative beta.
    torch.manual_seed(11)
    a1, b1, c1 = torch.randn(3, 2, device="cuda"), torch.randn(2, 4, device="cuda"), torch.randn(3, 4, device="cuda")
    a2, b2, c2 = torch.randn(3, 2, device="cuda"), torch.randn(2, 4, device="cuda"), torch.randn(3, 4, device="cuda")
    d1, d2 = torch.empty(3, 4, device="cuda"), torch.empty(3, 4, device="cuda")
    plan1 = gpu.make_plan(a1, b1, c1, d1, 1.25, -0.5)
    plan2 = gpu.make_plan(a2, b2, c2, d2, -2.0, 0.75)
    assert plan1.handle.value != plan2.handle.value
    gpu.run_plan(plan2)
    gpu.run_plan(plan1)
    torch.cuda.synchronize()
    assert torch.allclose(d1, 1.25 * (a1 @ b1) - 0.5 * c1, rtol=1e-5, atol=1e-5)
    assert torch.allclose(d2, -2.0 * (a2 @ b2) + 0.75 * c2, rtol=1e-5, atol=1e-5)


def test_in_place_accumulation(capi, gpu):
    # tests/api/gemm_api_test.cpp:330-390: C and D are the same buffer, alpha 2, beta 3.
    torch.manual_seed(12)
    for kernel, shape in ((0, (3, 2, 4)), (0, (200, 96, 136)), (1, (256, 128, 512)), (3, (4, 512, 64))):
        m, k, n = shape
        a, b, cd = torch.randn(m, k, device="cuda"), torch.randn(k, n, device="cuda"), torch.randn(m, n, device="cuda")
        expected = 2.0 * (a.double() @ b.double()) + 3.0 * cd.double()
        d, reason = platform_gemm(capi, gpu, kernel, a, b, cd, 2.0, 3.0, d=cd)
        assert d is not None, reason
        assert torch.allclose(cd.double(), expected, rtol=1e-4, atol=1e-3), capi.KERNEL_NAMES[kernel]


def test_empty_output_and_zero_depth(capi, gpu):
    # Empty output: succeeds with no storage at all (gemm_api_test.cpp:140-165).
    plan = gpu.binding().make_plan(capi.null_operand(0, 5), capi.null_operand(5, 7), capi.null_operand(0, 7),
                                   capi.null_operand(0, 7), 1.0, 0.0)
    assert plan.num_primitives >= 1 and plan.workspace_bytes(0) == 0
    plan.execute(0, 0, 0, gpu.current_stream())
    # K == 0 with null A and B: D = beta * C (fp32_gemm_test.cpp:138-145, fp32_gemm.cpp:57-60).
    c = torch.randn(6, 9, device="cuda")
    d = torch.empty(6, 9, device="cuda")
    plan = gpu.binding().make_plan(capi.null_operand(6, 0), capi.null_operand(0, 9), gpu.operand(c), gpu.operand(d),
                                   3.0, 0.5)
    gpu.run_plan(plan)
    torch.cuda.synchronize()
    assert torch.equal(d, 0.5 * c)


def test_status_codes(capi, gpu):
    b = gpu.binding()
    a_t, b_t = torch.zeros(4, 3, device="cuda"), torch.zeros(3, 5, device="cuda")
    c_t, d_t = torch.zeros(4, 5, device="cuda"), torch.zeros(4, 5, device="cuda")
    op = gpu.operand
    # Shape mismatch -> INVALID_ARGUMENT (gemm_api_test.cpp:186-250).
    with pytest.raises(capi.FTrainError) as info:
        b.make_plan(op(a_t), op(torch.zeros(4, 5, device="cuda")), op(c_t), op(d_t))
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT
    # INT64_MAX extents -> OVERFLOW (gemm_api_test.cpp:167-184).
    big = 2 ** 63 - 1
    with pytest.raises(capi.FTrainError) as info:
        b.make_plan((0, (big, big), None), (0, (big, big), None), (0, (big, big), None), (0, (big, big), None))
    assert info.value.status == capi.STATUS_OVERFLOW
    # Null A with work to do -> UNSUPPORTED, naming the primitive (gemm_api_test.cpp:252-328).
    with pytest.raises(capi.FTrainError) as info:
        b.make_plan(capi.null_operand(4, 3), op(b_t), op(c_t), op(d_t))
    assert info.value.status == capi.STATUS_UNSUPPORTED
    assert "Fp32Gemm" in info.value.message and "a required operand address is null" in info.value.message
    # FP16 A -> UNSUPPORTED "an operand is not fp32"; FP64 compute type -> UNSUPPORTED.
    args = capi.Args(b.ops)
    keep = []
    for name, tensor, numeric in (("a", a_t, capi.NUMERIC_FP16), ("b", b_t, capi.NUMERIC_FP32),
                                  ("c", c_t, capi.NUMERIC_FP32), ("d", d_t, capi.NUMERIC_FP32)):
        view, alive = capi.make_view(tensor.data_ptr(), tensor.shape, numeric_type=numeric)
        keep.append(alive)
        args.set_tensor(b.roles[name], view)
    import ctypes

    scalar = ctypes.c_float(1.0)
    for name in ("alpha", "beta"):
        view, alive = capi.make_view(ctypes.addressof(scalar), (), host=True)
        keep.append(alive)
        args.set_tensor(b.roles[name], view)
    args.set_gemm(b.gemm, capi.NUMERIC_FP32)
    with pytest.raises(capi.FTrainError) as info:
        capi.Plan(args)
    assert info.value.status == capi.STATUS_UNSUPPORTED
    assert "Fp32Gemm" in info.value.message and "an operand is not fp32" in info.value.message
    view, alive = capi.make_view(a_t.data_ptr(), a_t.shape)
    args.set_tensor(b.roles["a"], view)
    args.set_gemm(b.gemm, capi.NUMERIC_FP64)
    with pytest.raises(capi.FTrainError) as info:
        capi.Plan(args)
    assert info.value.status == capi.STATUS_UNSUPPORTED and "compute type is not fp32" in info.value.message
    # Workspace too small / bad index -> INVALID_ARGUMENT without dispatch.
    plan = b.make_plan(op(a_t), op(b_t), op(c_t), op(d_t))
    with pytest.raises(capi.FTrainError) as info:
        plan.execute(plan.num_primitives, 0, 0, gpu.current_stream())
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT


def test_selection_cache_and_workspace_walk(capi, gpu):
    # Tall K with few tiles: the split-K kernel is recommended and asks for a
    # workspace; a later index needs none (usage: walk indices by budget).
    a, b = torch.randn(256, 16384, device="cuda"), torch.randn(16384, 256, device="cuda")
    d = torch.empty(256, 256, device="cuda")
    plan = gpu.make_plan(a, b, None, d)
    names = plan.primitive_names()
    assert names[0] == "Fp32Gemm3xTf32SplitK" and plan.workspace_bytes(0) > 0
    assert names[-1] == "Fp32Gemm" and plan.workspace_bytes(len(names) - 1) == 0
    with pytest.raises(capi.FTrainError) as info:
        plan.execute(0, 0, 0, gpu.current_stream())
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT
    # Same problem description, other addresses: same ordered selection (cache hit).
    a2, b2, d2 = a.clone(), b.clone(), torch.empty_like(d)
    again = gpu.make_plan(a2, b2, None, d2)
    assert again.primitive_names() == names and again.handle.value != plan.handle.value
    exact = a.double() @ b.double()
    for index in range(len(names)):
        d.fill_(float("nan"))
        gpu.run_plan(plan, index)
        torch.cuda.synchronize()
        assert torch.allclose(d.double(), exact, rtol=1e-4, atol=2e-2), names[index]


# --------------------------------------------------------------- the benchmark configurations

def test_config1_small_default(capi, gpu, oracle):
    golden = np.load(GOLDEN / "torch_config1.npz")
    a, b = torch.from_numpy(golden["a"]).cuda(), torch.from_numpy(golden["b"]).cuda()
    d, names = gpu.gemm(a, b)
    error = oracle.scaled_error(d.cpu(), golden["d64"], golden["a"], golden["b"])
    torch_error = oracle.scaled_error(golden["d32"], golden["d64"], golden["a"], golden["b"])
    assert error <= 2.0 * max(torch_error, ERROR_FLOOR), (names, error, torch_error)


def test_config2_4096_cubed_with_addend(capi, gpu, oracle):
    torch.manual_seed(1)
    a, b, c = (torch.randn(4096, 4096, device="cuda") for _ in range(3))
    report = {}
    for kernel in (0, 1):
        d, reason = platform_gemm(capi, gpu, kernel, a, b, c, 1.5, 0.5)
        assert d is not None, reason
        report[capi.KERNEL_NAMES[kernel]] = check_against_float64(oracle, d, a, b, c, 1.5, 0.5, capi.KERNEL_NAMES[kernel])
    print("config2 scaled errors (ours, torch fp32):", report)


@pytest.mark.parametrize("m", [1, 17, 255, 4097])
def test_config3_tail_sweep_contiguous_and_transposed(capi, gpu, oracle, m):
    k = n = 4096
    generator = torch.Generator(device="cuda").manual_seed(2)
    a = torch.rand(m, k, device="cuda", generator=generator) * 2 - 1
    b = torch.rand(k, n, device="cuda", generator=generator) * 2 - 1
    buffer = a.t().contiguous()  # k x m; its transpose is an (m, k) view with strides (1, m)
    for label, a_view in (("contiguous", a), ("transposed view", buffer.t())):
        d, names = gpu.gemm(a_view, b)
        check_against_float64(oracle, d, a, b, None, 1.0, 0.0, f"m={m} {label} via {names[0]}")
        # A second Plan for the same description reproduces the selection.
        assert gpu.make_plan(a_view, b, None, d).primitive_names() == names
    if m <= 17:
        assert gpu.make_plan(a, b, None, d).primitive_name(0) == ("Fp32GemmSkinny" if m == 1 else "Fp32Gemm3xTf32FewRows")
    if m >= 17:
        # The transposed view of a k x m buffer with an odd m has a pitch TMA cannot take; the tensor-core
        # Primitives still come first: they stage A in the workspace (and ask for one).
        staged = gpu.make_plan(buffer.t(), b, None, d)
        assert staged.primitive_name(0).startswith("Fp32Gemm3xTf32") and staged.workspace_bytes(0) >= m * k * 4
    # The one-shot call takes no workspace here and must still succeed.
    once = torch.empty(m, n, device="cuda")
    capi.gemm_once(gpu.operand(a), gpu.operand(b), capi.null_operand(m, n), gpu.operand(once), 1.0, 0.0,
                   stream=gpu.current_stream())
    torch.cuda.synchronize()
    check_against_float64(oracle, once, a, b, None, 1.0, 0.0, f"m={m} one-shot")


def check_whole_matrix_in_row_blocks(oracle, d, a, b, what, block_rows):
    """Every element of d against a float64 product, `block_rows` rows at a time (to bound memory): the
    scaled error is taken per block and the worst block has to meet the bar against the worst block of
    torch's FP32 product."""
    b64 = b.double()
    col_norms = b64.norm(dim=0, keepdim=True)
    ours = torch_error = 0.0
    for start in range(0, a.shape[0], block_rows):
        rows = slice(start, min(start + block_rows, a.shape[0]))
        a64 = a[rows].double()
        exact = a64 @ b64
        scale = a64.norm(dim=1, keepdim=True) * col_norms + 1e-300
        assert torch.isfinite(d[rows]).all(), f"{what}: non-finite output in rows {rows}"
        ours = max(ours, float(((d[rows].double() - exact).abs() / scale).max()))
        torch_error = max(torch_error, float((((a[rows] @ b).double() - exact).abs() / scale).max()))
        del a64, exact, scale
    assert ours <= 2.0 * max(torch_error, ERROR_FLOOR), f"{what}: scaled error {ours:.3e} vs torch FP32 {torch_error:.3e}"
    return ours, torch_error


def test_config4_training_shape_whole_matrix(capi, gpu, oracle):
    m, k, n = 16384, 4096, 14336
    torch.manual_seed(3)
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(k, n, device="cuda") / (k ** 0.5)
    d, names = gpu.gemm(a, b)
    assert names[0] == "Fp32Gemm3xTf32"
    # All 128 x 75 output tiles of every band, not a sample of rows.
    report = check_whole_matrix_in_row_blocks(oracle, d, a, b, "config 4, all rows", 2048)
    print("config4 scaled errors (ours, torch fp32):", report)


def test_config5_tall_k_split_whole_matrix(capi, gpu, oracle):
    m = n = 2048
    k = 262144
    generator = torch.Generator(device="cuda").manual_seed(4)
    a = torch.rand(m, k, device="cuda", generator=generator) * 2 - 1
    b = torch.rand(k, n, device="cuda", generator=generator) * 2 - 1
    d, names = gpu.gemm(a, b)
    assert names[0] == "Fp32Gemm3xTf32SplitK"
    # The float64 copy of B alone is 4 GiB; 256 rows of A at a time keep the rest small.
    report = check_whole_matrix_in_row_blocks(oracle, d, a, b, "config 5, all rows", 256)
    print("config5 scaled errors (ours, torch fp32):", report)


def test_plan_reuse_many_executions(capi, gpu):
    a, b = torch.randn(1024, 1024, device="cuda"), torch.randn(1024, 1024, device="cuda")
    d = torch.empty(1024, 1024, device="cuda")
    plan = gpu.make_plan(a, b, None, d)
    size = plan.workspace_bytes(0)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device="cuda")
    stream = gpu.current_stream()
    before = capi.launch_count()
    for _ in range(1000):
        plan.execute(0, workspace.data_ptr() if size else 0, size, stream)
    torch.cuda.synchronize()
    assert capi.launch_count() - before >= 1000
    assert torch.allclose(d.double(), a.double() @ b.double(), rtol=1e-4, atol=1e-2)


@pytest.mark.parametrize("kernel", [0, 1, 2, 4])
def test_transposed_view_of_a(capi, gpu, oracle, kernel):
    """A given as the transpose of a contiguous k x m buffer: dims (m, k), strides (1, m)."""
    torch.manual_seed(31)
    # K is kept short: a strictly sequential FP32 sum over thousands of N(0,1) products is
    # by itself further from float64 than twice torch's blocked sum.
    shapes = [(256, 320, 2304), (132, 200, 4128)]
    if kernel in (capi.KERNEL_TF32X3, capi.KERNEL_TF32X3_SPLITK):
        shapes.append((256, 2304, 384))  # long K: the tensor kernels sum in blocks
    for m, k, n in shapes:
        buffer = torch.randn(k, m, device="cuda")
        a_view = buffer.t()
        b = torch.randn(k, n, device="cuda")
        c = torch.randn(m, n, device="cuda")
        d, reason = platform_gemm(capi, gpu, kernel, a_view, b, c, 0.75, -1.5)
        if d is None:
            pytest.skip(f"{capi.KERNEL_NAMES[kernel]} declines: {reason}")
        check_against_float64(oracle, d, a_view.contiguous(), b, c, 0.75, -1.5, f"{capi.KERNEL_NAMES[kernel]} {m}x{k}x{n}")


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16, 17, 31, 32])
def test_few_rows_kernel_row_counts_and_ragged_strips(capi, gpu, oracle, m):
    """Every row-count variant of the few-rows kernel; n off the 128-column strip and, through a
    view of a wider buffer, off the multiple of four; K off the 32-row box and long enough for
    several A stages per CTA."""
    torch.manual_seed(m)
    for k, n, pitch in ((1000, 200, 200), (4096 + 36, 130, 132), (8192, 4096, 4096), (257, 517, 520)):
        a = torch.randn(m, k, device="cuda") / 8
        wide = torch.randn(k, pitch, device="cuda")
        b = wide[:, :n]
        c = torch.randn(m, n, device="cuda")
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_SKINNY, a, b, c, 1.5, -0.25)
        assert d is not None, reason
        check_against_float64(oracle, d, a, b.contiguous(), c, 1.5, -0.25, f"few rows m={m} k={k} n={n}")
        # Transposed view of A (k x m buffer).
        a_view = (torch.randn(k, m, device="cuda") / 8).t()
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_SKINNY, a_view, b, None, 1.0, 0.0)
        assert d is not None, reason
        check_against_float64(oracle, d, a_view.contiguous(), b.contiguous(), None, 1.0, 0.0,
                              f"few rows, transposed A, m={m} k={k} n={n}")


@pytest.mark.parametrize("kernel", [0, 1, 2, 4])
@pytest.mark.parametrize("a_transposed", [False, True])
def test_transposed_view_of_b(capi, gpu, oracle, kernel, a_transposed):
    """B given as the transpose of a contiguous n x k buffer (the weight of a Linear layer):
    dims (k, n), strides (1, k); alone and together with a transposed view of A."""
    torch.manual_seed(37)
    shapes = [(256, 320, 2304), (132, 200, 4128)]
    if kernel in (capi.KERNEL_TF32X3, capi.KERNEL_TF32X3_SPLITK):
        shapes.append((384, 2304, 256))
    for m, k, n in shapes:
        a = (torch.randn(k, m, device="cuda").t() if a_transposed else torch.randn(m, k, device="cuda"))
        b_view = torch.randn(n, k, device="cuda").t()
        c = torch.randn(m, n, device="cuda")
        d, reason = platform_gemm(capi, gpu, kernel, a, b_view, c, -1.25, 0.5)
        if d is None:
            pytest.skip(f"{capi.KERNEL_NAMES[kernel]} declines: {reason}")
        check_against_float64(oracle, d, a.contiguous(), b_view.contiguous(), c, -1.25, 0.5,
                              f"{capi.KERNEL_NAMES[kernel]} {m}x{k}x{n} B^T{' A^T' if a_transposed else ''}")


def test_training_layouts_select_a_tensor_kernel(capi, gpu, oracle):
    """The three products of a Linear layer y = x W^T with x: tokens x in, W: out x in.
    forward  y  = x  @ W^T   (B is a transposed view)
    dgrad    dx = dy @ W     (plain)
    wgrad    dW = dy^T @ x   (A is a transposed view)"""
    tokens, features_in, features_out = 1024, 768, 1536
    torch.manual_seed(41)
    x = torch.randn(tokens, features_in, device="cuda")
    w = torch.randn(features_out, features_in, device="cuda") / features_in ** 0.5
    dy = torch.randn(tokens, features_out, device="cuda")
    for label, a, b in (("forward", x, w.t()), ("dgrad", dy, w), ("wgrad", dy.t(), x)):
        d, names = gpu.gemm(a, b)
        assert names[0] in ("Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK"), f"{label}: {names}"
        check_against_float64(oracle, d, a.contiguous(), b.contiguous(), None, 1.0, 0.0, f"{label} via {names[0]}")


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16, 17, 24, 32])
def test_few_rows_kernel_with_b_contiguous_along_k(capi, gpu, oracle, m):
    """x @ W^T for few rows of x: B is the transposed view of an n x k weight matrix (dims (k, n),
    strides (1, pitch)). n off the 32-row strip, K off the 128-value box, pitch wider than K, A plain
    and as a transposed view."""
    torch.manual_seed(100 + m)
    for k, n, pitch in ((1000, 200, 1000), (4096 + 36, 130, 4136), (8192, 4096, 8192), (260, 517, 264)):
        a = torch.randn(m, k, device="cuda") / 8
        wide = torch.randn(n, pitch, device="cuda")
        b = wide[:, :k].t()
        c = torch.randn(m, n, device="cuda")
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_SKINNY, a, b, c, 1.5, -0.25)
        assert d is not None, reason
        check_against_float64(oracle, d, a, b.contiguous(), c, 1.5, -0.25, f"few rows, W^T, m={m} k={k} n={n}")
        a_view = (torch.randn(k, m, device="cuda") / 8).t()
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_SKINNY, a_view, b, None, 1.0, 0.0)
        assert d is not None, reason
        check_against_float64(oracle, d, a_view.contiguous(), b.contiguous(), None, 1.0, 0.0,
                              f"few rows, W^T, transposed A, m={m} k={k} n={n}")
    # Through the Plan: the Finder's first choice for this layout is a few-rows kernel, the exact one up to 16 rows.
    x = torch.randn(m, 2048, device="cuda")
    w = torch.randn(1024, 2048, device="cuda")
    d, names = gpu.gemm(x, w.t())
    assert names[0] == ("Fp32GemmSkinny" if m <= 16 else "Fp32Gemm3xTf32FewRows"), names
    check_against_float64(oracle, d, x, w.t().contiguous(), None, 1.0, 0.0, f"x @ W^T via {names[0]}")


@pytest.mark.parametrize("kernel", [1, 2])
def test_scatter_launch_adds_rows_into_owner_buffers(capi, gpu, oracle, kernel):
    """ftcuda_gemm_launch_scatter with the owners' buffers on this GPU: two K shards ("ranks") add
    their products into three owners' row blocks that were initialised with beta * C."""
    import os

    if os.environ.get("FT_SKIP_TENSOR"):
        pytest.skip("tensor-core kernels switched off by FT_SKIP_TENSOR")
    torch.manual_seed(47)
    m, k, n, owners = 384, 4608, 400, 3
    rows = m // owners
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(k, n, device="cuda")
    c = torch.randn(m, n, device="cuda")
    alpha, beta = 0.75, -1.25
    for with_workspace in (False, True):  # every K slice adds directly / slices combined locally first
        blocks = [(beta * c[i * rows:(i + 1) * rows]).contiguous() for i in range(owners)]
        for k_start, k_stop in ((0, 2304), (2304, 4608)):
            a_cols = a[:, k_start:k_stop].contiguous()
            b_rows = b[k_start:k_stop].contiguous()
            unused = torch.empty(m, n, device="cuda")
            desc = capi.make_desc(gpu.operand(a_cols), gpu.operand(b_rows), capi.null_operand(m, n), gpu.operand(unused), alpha, 0.0,
                                  torch.cuda.current_device())
            reason = capi.platform_supports(kernel, desc)
            if reason is not None:
                pytest.skip(reason)
            launch = capi.PlatformGemm(kernel, desc)
            size = launch.workspace_bytes if with_workspace else 0
            workspace = torch.empty(max(size, 1), dtype=torch.uint8, device="cuda")
            # The pointer is never null: a workspace of fewer bytes than the launch asks for (here 0, also for
            # the cluster form of the single-launch kernel, which asks for none) must be ignored, not written.
            launch.run_scatter([block.data_ptr() for block in blocks], rows, gpu.current_stream(), workspace.data_ptr(), size)
        torch.cuda.synchronize()
        check_against_float64(oracle, torch.cat(blocks), a, b, c, alpha, beta,
                              f"scatter launch, {capi.KERNEL_NAMES[kernel]}, workspace={with_workspace}")
    # Argument checks: owners must cover m, buffers must exist, only tensor-core families scatter.
    with pytest.raises(capi.FTrainError, match="do not cover"):
        launch.run_scatter([blocks[0].data_ptr()], rows, gpu.current_stream())
    with pytest.raises(capi.FTrainError, match="no buffer"):
        launch.run_scatter([blocks[0].data_ptr(), 0, blocks[2].data_ptr()], rows, gpu.current_stream())
    simt = capi.PlatformGemm(capi.KERNEL_SIMT, desc)
    with pytest.raises(capi.FTrainError, match="tensor-core kernels only"):
        simt.run_scatter([block.data_ptr() for block in blocks], rows, gpu.current_stream())


def test_seeded_random_shapes_layouts_and_scalars_every_family(capi, gpu, oracle):
    """Eighty seeded random problems (the last twenty with few rows of a row-major A and a K of 256 or
    more, the few-rows tensor kernel's domain): extents off every tile size, A and B plain or as transposed views
    (pitches padded to keep them 16-byte aligned or deliberately not), C present or not, assorted
    scalars. Every family that accepts a problem must meet the float64 bar on it; the exact-FP32
    families are also held to the reference's tolerance against the sequential oracle when K is short."""
    import random

    rng = random.Random(20240611)
    torch.manual_seed(53)
    ran = {name: 0 for name in capi.KERNEL_NAMES.values()}
    for case in range(80):
        few_rows = case >= 60
        m = rng.choice([1, 2, 7, 17, 31, 33, 64] if few_rows else [1, 2, 7, 17, 31, 33, 64, 100, 129, 200, 257, 384, 513])
        n = rng.choice([1, 5, 32, 96, 100, 128, 131, 192, 260, 384, 500, 777])
        k = rng.choice([256, 300, 512, 1000, 2048, 4100] if few_rows else [1, 8, 31, 32, 33, 64, 100, 256, 300, 512, 1000, 2048, 4100])
        a_t, b_t = rng.random() < 0.35 and not few_rows, rng.random() < 0.35
        pad_a, pad_b = rng.choice([0, 0, 4, 3]), rng.choice([0, 0, 4, 1])
        a = (torch.randn(k, m + pad_a, device="cuda")[:, :m].t() if a_t else torch.randn(m, k + pad_a, device="cuda")[:, :k])
        b = (torch.randn(n, k + pad_b, device="cuda")[:, :k].t() if b_t else torch.randn(k, n + pad_b, device="cuda")[:, :n])
        c = torch.randn(m, n, device="cuda") if rng.random() < 0.6 else None
        alpha = rng.choice([1.0, -0.5, 2.25])
        beta = rng.choice([0.0, 1.0, -1.75]) if c is not None else 0.0
        for kernel, name in capi.KERNEL_NAMES.items():
            d, reason = platform_gemm(capi, gpu, kernel, a, b, c, alpha, beta)
            if d is None:
                continue
            ran[name] += 1
            what = f"case {case}: {name} {m}x{k}x{n} a_t={a_t} b_t={b_t} pads=({pad_a},{pad_b}) alpha={alpha} beta={beta}"
            if k <= 300 or kernel in (capi.KERNEL_TF32X3, capi.KERNEL_TF32X3_SPLITK, capi.KERNEL_TF32X3_ROWS, capi.KERNEL_SKINNY,
                                      capi.KERNEL_SIMT_SPLITK):
                # Blocked sums (or short K): the float64 bar applies as it stands.
                check_against_float64(oracle, d, a.contiguous(), b.contiguous(), c, alpha, beta, what)
            else:
                # A strictly sequential FP32 sum over a long K: the reference's own tolerance, scaled as in the smoke test.
                exact = alpha * (a.double() @ b.double()) + (beta * c.double() if c is not None else 0.0)
                slack = 2e-5 * max(1.0, (k / 257.0) ** 0.5)
                scale = (a.double().abs() @ b.double().abs()) * abs(alpha) + (abs(beta) * c.double().abs() if c is not None else 0.0)
                assert ((d.double() - exact).abs() <= slack * (1.0 + scale)).all(), what
    # The draw must actually have exercised every family.
    assert all(count >= 5 for count in ran.values()), ran


def test_random_problems_through_the_plan_api_with_the_finders_choice(capi, gpu, oracle):
    """Two hundred seeded random problems through the staged API, primitive 0 as the Finder ranks it -- the
    seeded test above forces every family; this one walks the selection rules: few rows, mid-size shapes
    that take the cluster form or split-K, small outputs, arbitrary extents, A and B plain or as
    transposed views. Blocked sums are held to the float64 bar, a strictly sequential exact sum
    (the reference's arithmetic) over more than a hundred K values to the reference's own tolerance."""
    import random

    rng = random.Random(0)
    torch.manual_seed(1)
    chosen = {}
    for case in range(200):
        kind = rng.random()
        if kind < 0.3:
            m = rng.choice([1, 2, 5, 8, 9, 12, 16, 17, 31, 32, 33, 48, 64])
            k = rng.choice([256, 512, 1000, 1024, 2048, 4096, 8192])
            n = rng.choice([128, 192, 500, 1024, 2048, 4096])
        elif kind < 0.7:
            m, k, n = rng.randint(65, 1100), rng.choice([128, 300, 512, 1000, 2048, 3072, 4096, 5000]), rng.randint(128, 2400)
        else:
            m, k, n = rng.randint(1, 700), rng.randint(1, 700), rng.randint(1, 700)
        a = torch.randn(k, m, device="cuda").t() if rng.random() < 0.3 else torch.randn(m, k, device="cuda")
        b = torch.randn(n, k, device="cuda").t() if rng.random() < 0.3 else torch.randn(k, n, device="cuda")
        c = torch.randn(m, n, device="cuda") if rng.random() < 0.5 else None
        alpha, beta = (1.0, 0.0) if c is None else (rng.uniform(-2, 2), rng.uniform(-2, 2))
        d, names = gpu.gemm(a, b, c, alpha, beta)
        chosen[names[0]] = chosen.get(names[0], 0) + 1
        what = f"case {case}: {names[0]} {m}x{k}x{n} a plain={a.is_contiguous()} b plain={b.is_contiguous()} alpha={alpha:.3f} beta={beta:.3f}"
        if names[0] == "Fp32Gemm" and k > 100:
            exact = alpha * (a.double() @ b.double()) + (beta * c.double() if c is not None else 0.0)
            slack = 2e-5 * max(1.0, (k / 257.0) ** 0.5)
            scale = (a.double().abs() @ b.double().abs()) * abs(alpha) + (abs(beta) * c.double().abs() if c is not None else 0.0)
            assert ((d.double() - exact).abs() <= slack * (1.0 + scale)).all(), what
        else:
            check_against_float64(oracle, d, a.contiguous(), b.contiguous(), c, alpha, beta, what)
    # The draw reaches every family the Finder ranks first somewhere.
    for name in ("Fp32Gemm", "Fp32GemmSkinny", "Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK", "Fp32Gemm3xTf32FewRows"):
        assert chosen.get(name, 0) >= 3, chosen


@pytest.mark.parametrize("m,k,n,ranks", [
    (256, 3072, 384, 6),     # 4 tiles, six K slices
    (384, 1024, 1152, 4),    # 18 tiles
    (1024, 1024, 1024, 3),   # 48 tiles
    (1024, 512, 1536, 2),    # 64 tiles, slices of 256
    (300, 1000, 500, 3),     # ragged in m, n and K; the last slice is shorter
    (130, 4100, 200, 6),     # one column of tiles off both tile extents, K off the K block
])
def test_tensor_kernel_splits_k_over_a_cluster(capi, gpu, oracle, m, k, n, ranks):
    """Few tiles and a long enough K: the single-launch 3xTF32 family cuts K over a thread-block cluster
    (one launch, no workspace) and the slices meet through distributed shared memory. With and without C,
    B plain and as a transposed view, D written through a row pitch; results repeat bit for bit."""
    import os

    if os.environ.get("FT_SKIP_TENSOR"):
        pytest.skip("tensor-core kernels switched off by FT_SKIP_TENSOR")
    del ranks  # documents the expected cluster size; the library's choice is not visible through the ABI
    torch.manual_seed(m + k + n)
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(k, n, device="cuda")
    c = torch.randn(m, n, device="cuda")
    for b_view in (b, b.t().contiguous().t()):
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3, a, b_view, c, 1.5, -0.25)
        assert d is not None, reason
        check_against_float64(oracle, d, a, b, c, 1.5, -0.25, f"cluster split {m}x{k}x{n}")
        again, _ = platform_gemm(capi, gpu, capi.KERNEL_TF32X3, a, b_view, c, 1.5, -0.25)
        assert torch.equal(d, again), "the slices are added in rank order: results must repeat bit for bit"
    d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3, a, b, None, 1.0, 0.0)
    assert d is not None, reason
    check_against_float64(oracle, d, a, b, None, 1.0, 0.0, f"cluster split, no C, {m}x{k}x{n}")
    desc = capi.make_desc(gpu.operand(a), gpu.operand(b), capi.null_operand(m, n), gpu.operand(d), 1.0, 0.0, 0)
    assert capi.PlatformGemm(capi.KERNEL_TF32X3, desc).workspace_bytes == 0


@pytest.mark.parametrize("m", [1, 9, 16, 17, 32, 33, 64])
def test_tensor_few_rows_kernel(capi, gpu, oracle, m):
    """The 3xTF32 kernel with B as the tensor core's 128-row operand: every padded row count (16, 32,
    64), n off the 128-column strip, K off the K block and long enough for several drains and for the
    cluster to split it, B wider than n, with and without C."""
    import os

    if os.environ.get("FT_SKIP_TENSOR"):
        pytest.skip("tensor-core kernels switched off by FT_SKIP_TENSOR")
    torch.manual_seed(200 + m)
    for k, n, pitch in ((1000, 200, 200), (4096 + 36, 130, 132), (8192, 4096, 4096), (260, 517, 520), (16384, 1024, 1024)):
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(k, pitch, device="cuda")[:, :n]
        c = torch.randn(m, n, device="cuda")
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, a, b, c, 1.5, -0.25)
        assert d is not None, reason
        check_against_float64(oracle, d, a, b.contiguous(), c, 1.5, -0.25, f"tensor few rows m={m} k={k} n={n}")
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, a, b, None, 1.0, 0.0)
        assert d is not None, reason
        check_against_float64(oracle, d, a, b.contiguous(), None, 1.0, 0.0, f"tensor few rows, no C, m={m} k={k} n={n}")
        # B handed over as the transposed view of an [n][k] matrix (x @ W.T): its strip tile is a K-major operand.
        bt = torch.randn(n, k + 4, device="cuda")[:, :k].t()
        d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, a, bt, c, 1.5, -0.25)
        assert d is not None, reason
        check_against_float64(oracle, d, a, bt.contiguous(), c, 1.5, -0.25, f"tensor few rows, B along K, m={m} k={k} n={n}")
    # Declined: too many rows, short K.
    wide = torch.randn(65, 512, device="cuda")
    assert platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, wide, torch.randn(512, 256, device="cuda"), None, 1.0, 0.0)[0] is None
    # A stored by columns (the transposed view of a k x m buffer, whatever its pitch) is copied into the
    # workspace as a row-major matrix first: accepted, with a workspace.
    a_t = torch.randn(512, m, device="cuda").t()
    b = torch.randn(512, 256, device="cuda")
    d, reason = platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, a_t, b, None, 1.0, 0.0)
    assert d is not None, reason
    check_against_float64(oracle, d, a_t.contiguous(), b, None, 1.0, 0.0, f"tensor few rows, A staged, m={m}")
    assert platform_gemm(capi, gpu, capi.KERNEL_TF32X3_ROWS, torch.randn(8, 64, device="cuda"), torch.randn(64, 256, device="cuda"),
                         None, 1.0, 0.0)[0] is None


@pytest.mark.parametrize("kernel", [1, 2, 5])
def test_split_precision_kernels_keep_ieee_behaviour_at_the_edge_of_the_range(capi, gpu, oracle, kernel):
    """Infinities, NaN and +-FLT_MAX in A and B: the 3xTF32 kernels must give what the exact FFMA kernel
    (FTCUDA_GEMM_SIMT, the reference's arithmetic) gives -- +-inf where it gives +-inf, NaN where it gives
    NaN (inf - inf, inf * 0, NaN), finite and close where it is finite. The high part of the split
    saturates at the largest finite TF32 number, so FLT_MAX neither rounds up to infinity nor turns into
    a NaN inside the split."""
    import os

    if os.environ.get("FT_SKIP_TENSOR"):
        pytest.skip("tensor-core kernels switched off by FT_SKIP_TENSOR")
    flt_max = torch.finfo(torch.float32).max
    torch.manual_seed(61)
    m, k, n = (48, 1024, 384) if kernel == 5 else (256, 1024, 384)
    a = torch.rand(m, k, device="cuda") * 0.5 + 0.25
    b = torch.rand(k, n, device="cuda") * 0.25 + 0.125   # positive, so that a row's infinities do not cancel
    a[1, 5] = float("inf")
    a[2, 700] = float("-inf")
    a[3, 9], a[3, 600] = float("inf"), float("-inf")       # inf - inf -> NaN
    a[4, 33] = float("nan")
    a[5, 100] = flt_max                                     # times at most 0.375: finite
    a[6, 1000] = -flt_max
    a[7, 64] = float("inf")
    b[64, 17] = 0.0                                         # inf * 0 -> NaN in column 17 of row 7
    b[200, 40] = float("inf")                               # a whole column of +inf
    b[300, 41] = -flt_max * 0.5                             # times at most 0.75: finite
    expected, reason = platform_gemm(capi, gpu, capi.KERNEL_SIMT, a, b, None, 1.0, 0.0)
    assert expected is not None, reason
    d, reason = platform_gemm(capi, gpu, kernel, a, b, None, 1.0, 0.0)
    if d is None:
        pytest.skip(f"{capi.KERNEL_NAMES[kernel]} declines: {reason}")
    name = capi.KERNEL_NAMES[kernel]
    assert torch.equal(torch.isnan(d), torch.isnan(expected)), f"{name}: NaN pattern differs from the FFMA kernel's"
    infinite = torch.isinf(expected)
    assert torch.equal(torch.isinf(d), infinite), f"{name}: infinity pattern differs from the FFMA kernel's"
    assert torch.equal(d[infinite], expected[infinite]), f"{name}: an infinity has the wrong sign"
    finite = torch.isfinite(expected)
    ordinary = torch.ones(n, dtype=torch.bool, device="cuda")
    ordinary[40] = False  # the column of +inf
    assert finite[5][ordinary].all() and finite[6][ordinary].all() and finite[:, 41].sum() >= m - 6, \
        "the FLT_MAX lines are meant to stay finite"
    assert torch.allclose(d[finite], expected[finite], rtol=2e-5, atol=1e-3), f"{name}: finite entries are off"


def test_a_wait_that_runs_out_is_reported_once_and_the_device_stays_usable(capi, gpu):
    """The give-up path of the kernels' bounded waits, made to happen without a fault: one warp waits
    200 microseconds on a barrier nothing arrives on, returns, and leaves code 2 in the device's status
    word. The next launch reports it (once), the one after runs and is correct; a reset clears it too."""
    device = torch.cuda.current_device()
    a, b = torch.randn(256, 512, device="cuda"), torch.randn(512, 384, device="cuda")
    d = torch.empty(256, 384, device="cuda")
    desc = capi.make_desc(gpu.operand(a), gpu.operand(b), capi.null_operand(256, 384), gpu.operand(d), 1.0, 0.0, device)
    launch = capi.PlatformGemm(capi.KERNEL_SIMT, desc)
    launch.run(0, 0, gpu.current_stream())
    torch.cuda.synchronize()
    assert capi.device_status(device) == 0
    capi.selftest_bounded_wait(device, 200_000, gpu.current_stream())
    torch.cuda.synchronize()  # the kernel returned by itself
    assert capi.device_status(device) == 2
    with pytest.raises(capi.FTrainError, match="timed-out wait"):
        launch.run(0, 0, gpu.current_stream())
    assert capi.device_status(device) == 0
    d.fill_(float("nan"))
    launch.run(0, 0, gpu.current_stream())
    torch.cuda.synchronize()
    assert torch.allclose(d, a @ b, rtol=1e-4, atol=1e-3)
    # Through the public API the same condition is INTERNAL_ERROR, then clean again.
    capi.selftest_bounded_wait(device, 200_000, gpu.current_stream())
    torch.cuda.synchronize()
    plan = gpu.make_plan(a, b, None, d)
    with pytest.raises(capi.FTrainError) as info:
        gpu.run_plan(plan)
    assert info.value.status == capi.STATUS_INTERNAL_ERROR and "timed-out wait" in info.value.message
    gpu.run_plan(plan)
    torch.cuda.synchronize()
    capi.selftest_bounded_wait(device, 200_000, gpu.current_stream())
    torch.cuda.synchronize()
    capi.device_status_reset(device)
    assert capi.device_status(device) == 0
    gpu.run_plan(plan)
    torch.cuda.synchronize()
    assert torch.allclose(d, a @ b, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("kernel", [1, 2, 5])
def test_operands_tma_cannot_fetch_are_staged_in_the_workspace(capi, gpu, oracle, kernel):
    """A and/or B with layouts no TMA descriptor describes -- transposed views with odd pitches, a base in
    the middle of a row, two non-unit strides -- run on the tensor-core families through a copy at the head
    of the workspace; with split-K the partial sums follow the copies in the same workspace."""
    import os

    if os.environ.get("FT_SKIP_TENSOR"):
        pytest.skip("tensor-core kernels switched off by FT_SKIP_TENSOR")
    torch.manual_seed(83)
    rows_kernel = kernel == capi.KERNEL_TF32X3_ROWS
    m, k, n = (33, 2048, 513) if rows_kernel else (255, 2304, 517)
    cases = {
        "A transposed, odd pitch": (torch.randn(k, m, device="cuda").t(), torch.randn(k, n + 3, device="cuda")[:, :n + 3][:, :n]),
        "A off a 16-byte boundary": (torch.randn(m, k + 5, device="cuda")[:, 1:k + 1], torch.randn(k, n + 3, device="cuda")[:, :n]),
        "A every other column, B transposed with odd pitch": (torch.randn(m, 2 * k, device="cuda")[:, ::2],
                                                             torch.randn(n, k + 1, device="cuda")[:, :k].t()),
        "only B staged": (torch.randn(m, k, device="cuda"), torch.randn(k, n, device="cuda")),
    }
    c = torch.randn(m, n, device="cuda")
    for label, (a, b) in cases.items():
        d = torch.full((m, n), float("nan"), device="cuda")
        desc = capi.make_desc(gpu.operand(a), gpu.operand(b), gpu.operand(c), gpu.operand(d), 1.25, -0.5, torch.cuda.current_device())
        reason = capi.platform_supports(kernel, desc)
        assert reason is None, f"{label}: {reason}"
        launch = capi.PlatformGemm(kernel, desc)
        assert launch.workspace_bytes > 0, label
        # An oddly aligned workspace must do: the copies are aligned inside it.
        workspace = torch.empty(launch.workspace_bytes + 8, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            d.fill_(float("nan"))
            launch.run(workspace.data_ptr() + 4, launch.workspace_bytes, gpu.current_stream())
            torch.cuda.synchronize()
            check_against_float64(oracle, d, a.contiguous(), b.contiguous(), c, 1.25, -0.5, f"{capi.KERNEL_NAMES[kernel]}, {label}")
        with pytest.raises(capi.FTrainError, match="workspace"):
            launch.run(0, 0, gpu.current_stream())
