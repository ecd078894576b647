"""ftcuda_gemm_splitk_static: the split-K GEMM that uses the library's own
static scratch instead of a caller-supplied workspace (for callers that cannot
allocate one; see include/ftcuda/ftcuda.h). Checked against the ordinary
split-K entry point, which gets its workspace from the caller, on two calls in
a row that share the scratch. The file name makes pytest collect it last."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu(capi):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    import gpu_support

    return gpu_support


def reference_split_k(capi, gpu, a, b, c, alpha, beta):
    """The existing entry point: FTCUDA_GEMM_SIMT_SPLITK with a workspace from the caller."""
    m, n = a.shape[0], b.shape[1]
    d = torch.full((m, n), float("nan"), device="cuda")
    desc = capi.make_desc(gpu.operand(a), gpu.operand(b), gpu.operand(c), gpu.operand(d), alpha, beta,
                          torch.cuda.current_device())
    launch = capi.PlatformGemm(capi.KERNEL_SIMT_SPLITK, desc)
    assert launch.workspace_bytes > 0
    workspace = torch.empty(launch.workspace_bytes, dtype=torch.uint8, device="cuda")
    launch.run(workspace.data_ptr(), launch.workspace_bytes, gpu.current_stream())
    torch.cuda.synchronize()
    return d


def test_static_scratch_matches_workspace_variant_twice(capi, gpu):
    assert capi.splitk_static_capacity() == 16 << 20
    torch.manual_seed(21)
    # Two different problems back to back: the second must not see the first one's partial sums.
    for m, k, n, alpha, beta in ((192, 4096, 320, 1.5, 0.75), (77, 8200, 130, -0.5, 2.0)):
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(k, n, device="cuda")
        c = torch.randn(m, n, device="cuda")
        expected = reference_split_k(capi, gpu, a, b, c, alpha, beta)
        d = torch.full((m, n), float("nan"), device="cuda")
        desc = capi.make_desc(gpu.operand(a), gpu.operand(b), gpu.operand(c), gpu.operand(d), alpha, beta,
                              torch.cuda.current_device())
        # A first call may load the kernel's module and resolve the scratch address; the check that
        # nothing is allocated is made around a second call. torch's own counter only sees torch's
        # caching allocator, so the driver's free-memory figure (cudaMemGetInfo) is compared as well.
        capi.splitk_static(desc, gpu.current_stream())
        torch.cuda.synchronize()
        d.fill_(float("nan"))
        torch.cuda.synchronize()
        reserved_before = torch.cuda.memory_reserved()
        free_before = torch.cuda.mem_get_info()[0]
        capi.splitk_static(desc, gpu.current_stream())
        torch.cuda.synchronize()
        assert torch.cuda.memory_reserved() == reserved_before
        assert torch.cuda.mem_get_info()[0] >= free_before  # an allocation inside the call would lower it
        # Both sum FP32 partial slices in order, possibly with another slice
        # count: the tolerance is the one of the exact-FP32 tests, scaled for K.
        slack = (k / 257.0) ** 0.5
        tolerance = 2e-5 * slack
        assert torch.isfinite(d).all()
        assert torch.all((d - expected).abs() <= tolerance + tolerance * expected.abs()), (m, k, n)
        exact = alpha * (a.double() @ b.double()) + beta * c.double()
        assert torch.allclose(d.double(), exact, rtol=1e-4, atol=1e-2)


def test_static_scratch_refuses_what_does_not_fit(capi, gpu):
    m = n = 2048  # 4 Mi outputs: two slices would need 32 MiB
    a = torch.zeros(m, 1024, device="cuda")
    b = torch.zeros(1024, n, device="cuda")
    d = torch.zeros(m, n, device="cuda")
    desc = capi.make_desc(gpu.operand(a), gpu.operand(b), capi.null_operand(m, n), gpu.operand(d), 1.0, 0.0,
                          torch.cuda.current_device())
    with pytest.raises(capi.FTrainError) as info:
        capi.splitk_static(desc, gpu.current_stream())
    assert "do not fit" in info.value.message
