"""flash_train.torch.gemm on a device: the reference's Python test
(tests/python/torch_gemm_test.py:15-71 there), case for case."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPE_GRID = [(1, 1, 1), (3, 4, 2), (16, 16, 16), (64, 48, 32), (129, 65, 17), (33, 257, 65), (256, 128, 64)]


@pytest.fixture(scope="module")
def binding(native_library):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    from conftest import load_build_module

    load_build_module().build_torch_binding(verbose=False)
    torch.backends.cuda.matmul.allow_tf32 = False
    import flash_train.torch

    return flash_train.torch


def make_inputs(shape=(128, 64, 96)):
    generator = torch.Generator(device="cuda").manual_seed(7)
    m, k, n = shape
    a = torch.randn(m, k, device="cuda", generator=generator)
    b = torch.randn(k, n, device="cuda", generator=generator)
    c = torch.randn(m, n, device="cuda", generator=generator)
    return a, b, c


@pytest.mark.parametrize("shape", SHAPE_GRID)
def test_gemm_matches_matmul(binding, shape):
    a, b, c = make_inputs(shape)
    d = binding.gemm(a, b, c, alpha=1.5, beta=0.25)
    torch.testing.assert_close(d, 1.5 * (a @ b) + 0.25 * c, rtol=1e-4, atol=1e-3)


def test_gemm_without_c_and_defaults(binding):
    a, b, _ = make_inputs()
    torch.testing.assert_close(binding.gemm(a, b, alpha=1.5), 1.5 * (a @ b), rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(binding.gemm(a, b), a @ b, rtol=1e-4, atol=1e-3)


def test_runs_on_the_current_stream(binding):
    a, b, _ = make_inputs((512, 256, 384))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        d = binding.gemm(a, b)
    side.synchronize()
    torch.testing.assert_close(d, a @ b, rtol=1e-4, atol=1e-3)


def test_rejections_raise_runtime_error(binding):
    a, b, _ = make_inputs()
    with pytest.raises(RuntimeError):
        binding.gemm(a, torch.randn(3, 3, device="cuda"))
    with pytest.raises(RuntimeError):
        binding.gemm(a.cpu(), b)
    with pytest.raises(RuntimeError):
        binding.gemm(a.to(torch.float64), b)
    with pytest.raises(RuntimeError):
        binding.gemm(a.t(), b)  # not contiguous: rejected by the binding, as in the reference
