"""GroupedABCDGemm on the GPU, through the public C API: D_g = alpha * A_g * B_g + beta * C_g over ragged
groups, an empty group among them, against the reference's PyTorch expression evaluated group by group
(in float64 for the accuracy bar: scaled error at most twice that of a plain FP32 product)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ERROR_FLOOR = 2.0 ** -24


@pytest.fixture(scope="module")
def binding(capi):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    torch.backends.cuda.matmul.allow_tf32 = False
    return capi.GroupedGemmBinding(order=("d", "beta", "b", "a", "alpha", "c"))


def packed(matrices):
    """The groups stored one after another, dense row-major: (flat tensor, rows, cols)."""
    flat = torch.cat([m.reshape(-1) for m in matrices]) if matrices else torch.empty(0, device="cuda")
    return flat, [m.shape[0] for m in matrices], [m.shape[1] for m in matrices]


def operand(flat, rows, cols, **extra):
    return {"address": flat.data_ptr() if flat is not None else 0, "rows": rows, "cols": cols, **extra}


def run(capi, plan, index):
    size = plan.workspace_bytes(index)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device="cuda")
    plan.execute(index, workspace.data_ptr() if size else 0, size, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()


def check_groups(oracle, d_flat, shapes, a_list, b_list, c_list, alpha, beta, what, exact_kernel=False):
    at = 0
    for g, (m, k, n) in enumerate(shapes):
        d = d_flat[at:at + m * n].reshape(m, n)
        at += m * n
        if m * n == 0:
            continue
        a, b = a_list[g], b_list[g]
        c = c_list[g] if c_list is not None else None
        exact = alpha * (a.double() @ b.double()) + (beta * c.double() if c is not None else 0.0)
        plain = oracle.torch_reference(a, b, c, alpha, beta)
        ours = oracle.scaled_error(d, exact, a * abs(alpha), b, c, beta)
        other = oracle.scaled_error(plain, exact, a * abs(alpha), b, c, beta)
        assert torch.isfinite(d).all(), f"{what}: group {g} has non-finite output"
        if exact_kernel and k > 300:
            # A strictly sequential FP32 sum over a long K (the reference kernel's arithmetic) is by itself further
            # from float64 than a blocked sum: the reference's own tolerance, scaled with sqrt(K) as in the other tests.
            slack = 2e-5 * max(1.0, (k / 257.0) ** 0.5)
            scale = (a.double().abs() @ b.double().abs()) * abs(alpha) + (abs(beta) * c.double().abs() if c is not None else 0.0)
            assert ((d.double() - exact).abs() <= slack * (1.0 + scale)).all(), f"{what}: group {g} ({m}x{k}x{n})"
        else:
            assert ours <= 2.0 * max(other, ERROR_FLOOR), f"{what}: group {g} ({m}x{k}x{n}) scaled error {ours:.3e} vs FP32 {other:.3e}"


RAGGED = [(256, 512, 384), (0, 512, 384), (130, 260, 200), (1, 128, 4), (513, 1024, 196), (64, 4096, 388)]


@pytest.mark.parametrize("with_c", [True, False])
def test_ragged_groups_with_an_empty_one(capi, binding, oracle, with_c):
    torch.manual_seed(71)
    a_list = [torch.randn(m, k, device="cuda") for m, k, n in RAGGED]
    b_list = [torch.randn(k, n, device="cuda") for m, k, n in RAGGED]
    c_list = [torch.randn(m, n, device="cuda") for m, k, n in RAGGED] if with_c else None
    alpha, beta = 1.5, (-0.75 if with_c else 0.0)
    a_flat, a_rows, a_cols = packed(a_list)
    b_flat, b_rows, b_cols = packed(b_list)
    d_rows, d_cols = [m for m, k, n in RAGGED], [n for m, k, n in RAGGED]
    c_flat = packed(c_list)[0] if with_c else None
    d_flat = torch.full((sum(m * n for m, k, n in RAGGED),), float("nan"), device="cuda")
    plan = binding.make_plan(operand(a_flat, a_rows, a_cols), operand(b_flat, b_rows, b_cols), operand(c_flat, d_rows, d_cols),
                             operand(d_flat, d_rows, d_cols), alpha, beta)
    names = plan.primitive_names()
    assert names == ["GroupedFp32Gemm3xTf32", "GroupedFp32Gemm"], names
    assert plan.workspace_bytes(0) > 0 and plan.workspace_bytes(1) == 0
    before = capi.launch_count()
    for index, name in enumerate(names):
        d_flat.fill_(float("nan"))
        run(capi, plan, index)
        check_groups(oracle, d_flat, RAGGED, a_list, b_list, c_list, alpha, beta, name, exact_kernel=name == "GroupedFp32Gemm")
    # One launch for all groups on the tensor cores; one per non-empty group on the exact path.
    assert capi.launch_count() - before == 1 + sum(1 for m, k, n in RAGGED if m * n)
    # The tensor-core Primitive needs its workspace.
    with pytest.raises(capi.FTrainError) as info:
        plan.execute(0, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT


def test_explicit_offsets_strides_and_transposed_weights(capi, binding, oracle):
    """MoE-style: the tokens of all experts in one (tokens, hidden) matrix, every expert's weight stored
    (out, in) and used as its transposed view, outputs written into one (tokens, out) matrix."""
    torch.manual_seed(73)
    hidden, out = 768, 1152
    counts = [300, 0, 129, 515, 64]
    tokens = torch.randn(sum(counts), hidden, device="cuda")
    weights = torch.randn(len(counts), out, hidden, device="cuda") / hidden ** 0.5
    result = torch.full((sum(counts), out), float("nan"), device="cuda")
    starts = [sum(counts[:g]) for g in range(len(counts))]
    groups = len(counts)
    a = operand(tokens, counts, [hidden] * groups, offsets=[s * hidden for s in starts], row_strides=[hidden] * groups,
                col_strides=[1] * groups)
    # B_g = W_g^T: (hidden, out) with strides (1, hidden).
    b = operand(weights, [hidden] * groups, [out] * groups, offsets=[g * out * hidden for g in range(groups)],
                row_strides=[1] * groups, col_strides=[hidden] * groups)
    d = operand(result, counts, [out] * groups, offsets=[s * out for s in starts], row_strides=[out] * groups, col_strides=[1] * groups)
    c = operand(None, counts, [out] * groups, offsets=[s * out for s in starts], row_strides=[out] * groups, col_strides=[1] * groups)
    plan = binding.make_plan(a, b, c, d, 1.0, 0.0)
    names = plan.primitive_names()
    assert names[0] == "GroupedFp32Gemm3xTf32", names
    shapes = [(count, hidden, out) for count in counts]
    a_list = [tokens[s:s + count] for s, count in zip(starts, counts)]
    b_list = [weights[g].t().contiguous() for g in range(groups)]
    for index, name in enumerate(names):
        result.fill_(float("nan"))
        run(capi, plan, index)
        check_groups(oracle, result.reshape(-1), shapes, a_list, b_list, None, 1.0, 0.0, f"{name}, transposed weights",
                     exact_kernel=name == "GroupedFp32Gemm")
    # An equal description again: the cached selection, a new Plan.
    again = binding.make_plan(a, b, c, d, 1.0, 0.0)
    assert again.primitive_names() == names and again.handle.value != plan.handle.value


def test_shallow_groups_fall_to_the_exact_primitive_and_zero_depth_scales_c(capi, binding, oracle):
    torch.manual_seed(79)
    shapes = [(40, 64, 72), (33, 0, 20), (7, 300, 9)]  # K < 128, K = 0, and a small one
    a_list = [torch.randn(m, k, device="cuda") for m, k, n in shapes]
    b_list = [torch.randn(k, n, device="cuda") for m, k, n in shapes]
    c_list = [torch.randn(m, n, device="cuda") for m, k, n in shapes]
    a_flat, a_rows, a_cols = packed(a_list)
    b_flat, b_rows, b_cols = packed(b_list)
    c_flat, d_rows, d_cols = packed(c_list)
    d_flat = torch.full_like(c_flat, float("nan"))
    plan = binding.make_plan(operand(a_flat, a_rows, a_cols), operand(b_flat, b_rows, b_cols), operand(c_flat, d_rows, d_cols),
                             operand(d_flat, d_rows, d_cols), 2.0, 0.5)
    assert plan.primitive_names() == ["GroupedFp32Gemm"]
    run(capi, plan, 0)
    check_groups(oracle, d_flat, shapes, a_list, b_list, c_list, 2.0, 0.5, "exact grouped", exact_kernel=True)
    # K = 0: D = beta * C exactly.
    at = 40 * 72
    assert torch.equal(d_flat[at:at + 33 * 20], 0.5 * c_list[1].reshape(-1))


def test_description_errors(capi, binding):
    flat = torch.zeros(4096, device="cuda")
    good = operand(flat, [4, 4], [8, 8])
    with pytest.raises(capi.FTrainError) as info:  # a's columns (8) against b's rows (9) in group 1
        binding.make_plan(good, operand(flat, [8, 9], [4, 4]), operand(flat, [4, 4], [4, 4]), operand(flat, [4, 4], [4, 4]))
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT and "group 1" in info.value.message
    with pytest.raises(capi.FTrainError) as info:  # another number of groups
        binding.make_plan(good, operand(flat, [8], [4]), operand(flat, [4, 4], [4, 4]), operand(flat, [4, 4], [4, 4]))
    assert info.value.status == capi.STATUS_INVALID_ARGUMENT


@pytest.mark.parametrize("kind", ["GroupedBCDGemm", "GroupedABGemm"])
def test_tensor_list_variants(capi, oracle, kind):
    """GroupedBCDGemm (a is a TensorList: every group's A is a tensor of its own) and GroupedABGemm (c and d are
    TensorLists: every group's result goes to its own tensor; here the last group has no addend at all)."""
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(89)
    shapes = [(200, 512, 384), (0, 512, 384), (129, 256, 196), (33, 1024, 260)]
    a_list = [torch.randn(m, k, device="cuda") for m, k, n in shapes]
    b_list = [torch.randn(k, n, device="cuda") for m, k, n in shapes]
    c_list = [torch.randn(m, n, device="cuda") for m, k, n in shapes]
    d_list = [torch.full((m, n), float("nan"), device="cuda") for m, k, n in shapes]
    alpha, beta = -1.25, 0.5
    as_list = lambda tensors, drop_last=False: [(0 if drop_last and i == len(tensors) - 1 else t.data_ptr(), tuple(t.shape), None)  # noqa: E731
                                                for i, t in enumerate(tensors)]
    b_flat, b_rows, b_cols = packed(b_list)
    binding = capi.GroupedGemmBinding(kind=kind)
    if kind == "GroupedBCDGemm":
        c_flat, d_rows, d_cols = packed(c_list)
        d_flat = torch.full_like(c_flat, float("nan"))
        plan = binding.make_plan(as_list(a_list), operand(b_flat, b_rows, b_cols), operand(c_flat, d_rows, d_cols),
                                 operand(d_flat, d_rows, d_cols), alpha, beta)
        expected_c = c_list
    else:
        a_flat, a_rows, a_cols = packed(a_list)
        plan = binding.make_plan(operand(a_flat, a_rows, a_cols), operand(b_flat, b_rows, b_cols), as_list(c_list, drop_last=True),
                                 as_list(d_list), alpha, beta)
        expected_c = c_list[:-1] + [None]
    names = plan.primitive_names()
    assert names == ["GroupedFp32Gemm3xTf32", "GroupedFp32Gemm"], names
    for index, name in enumerate(names):
        if kind == "GroupedBCDGemm":
            d_flat.fill_(float("nan"))
        else:
            for d in d_list:
                d.fill_(float("nan"))
        run(capi, plan, index)
        results = d_flat if kind == "GroupedBCDGemm" else torch.cat([d.reshape(-1) for d in d_list])
        at = 0
        for g, (m, k, n) in enumerate(shapes):
            if m * n == 0:
                continue
            d = results[at:at + m * n].reshape(m, n)
            at += m * n
            c = expected_c[g]
            exact = alpha * (a_list[g].double() @ b_list[g].double()) + (beta * c.double() if c is not None else 0.0)
            plain = oracle.torch_reference(a_list[g], b_list[g], c, alpha, beta if c is not None else 0.0)
            ours = oracle.scaled_error(d, exact, a_list[g] * abs(alpha), b_list[g], c, beta)
            other = oracle.scaled_error(plain, exact, a_list[g] * abs(alpha), b_list[g], c, beta)
            assert torch.isfinite(d).all(), f"{kind} {name}: group {g} has non-finite output"
            if name == "GroupedFp32Gemm" and k > 300:
                slack = 2e-5 * max(1.0, (k / 257.0) ** 0.5)
                scale = (a_list[g].double().abs() @ b_list[g].double().abs()) * abs(alpha) + (abs(beta) * c.double().abs() if c is not None else 0.0)
                assert ((d.double() - exact).abs() <= slack * (1.0 + scale)).all(), f"{kind} {name}: group {g}"
            else:
                assert ours <= 2.0 * max(other, ERROR_FLOOR), f"{kind} {name}: group {g} scaled error {ours:.3e} vs {other:.3e}"
