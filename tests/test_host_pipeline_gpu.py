"""flash_train.torch.HostGemm: operands in host memory, bands of rows in flight."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ERROR_FLOOR = 2.0 ** -24


@pytest.fixture(scope="module")
def binding(native_library):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    from conftest import load_build_module

    load_build_module().build_torch_binding(verbose=False)
    torch.backends.cuda.matmul.allow_tf32 = False
    import flash_train.torch

    return flash_train.torch


def check(oracle, out, a, b, c, alpha, beta, what):
    """Scaled error against float64 at most twice that of a plain FP32 product (on the CPU here)."""
    exact = alpha * (a.double() @ b.double())
    plain = alpha * (a @ b)
    if c is not None:
        exact = exact + beta * c.double()
        plain = plain + beta * c
    ours = oracle.scaled_error(out, exact, a * abs(alpha), b, c, beta)
    other = oracle.scaled_error(plain, exact, a * abs(alpha), b, c, beta)
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    assert ours <= 2.0 * max(other, ERROR_FLOOR), f"{what}: scaled error {ours:.3e} vs FP32 {other:.3e}"


@pytest.mark.parametrize("m,n,k,band_rows,with_c", [
    (640, 384, 512, 256, False),   # two full bands and a ragged one
    (300, 200, 96, 128, True),     # SIMT-sized, addend, ragged end
    (17, 256, 512, 2048, False),   # one band, few rows
    (512, 384, 256, 64, True),     # many bands: every buffer pair is reused several times
])
def test_host_gemm_matches_float64(binding, oracle, m, n, k, band_rows, with_c):
    generator = torch.Generator().manual_seed(m * 7 + n)
    a = torch.randn(m, k, generator=generator).pin_memory()
    b = torch.randn(k, n, generator=generator).pin_memory()
    c = torch.randn(m, n, generator=generator).pin_memory() if with_c else None
    alpha, beta = 1.25, (-0.5 if with_c else 0.0)
    pipeline = binding.HostGemm(m, n, k, band_rows=band_rows, with_c=with_c)
    out = torch.empty(m, n).pin_memory()
    for call in range(2):  # the second call reuses buffers the first one has just used
        out.fill_(float("nan"))
        result = pipeline(a, b, c, alpha=alpha, beta=beta, out=out)
        torch.cuda.synchronize()
        assert result is out
        check(oracle, out, a, b, c, alpha, beta, f"{m}x{n}x{k} bands of {band_rows}, call {call}")


def test_overlapping_calls_write_their_results_in_call_order(binding, oracle):
    """overlap_calls=True: the next call's copy-in runs while the previous call's result is still leaving; every
    call's result must still be complete and right after synchronize()."""
    generator = torch.Generator().manual_seed(5)
    m, n, k = 1024, 640, 512
    b = torch.randn(k, n, generator=generator).pin_memory()
    inputs = [torch.randn(m, k, generator=generator).pin_memory() for _ in range(4)]
    outputs = [torch.full((m, n), float("nan")).pin_memory() for _ in range(4)]
    pipeline = binding.HostGemm(m, n, k, band_rows=128)
    for a, out in zip(inputs, outputs):
        pipeline(a, b, out=out, overlap_calls=True)
    pipeline.synchronize()
    for index, (a, out) in enumerate(zip(inputs, outputs)):
        check(oracle, out, a, b, None, 1.0, 0.0, f"overlapping call {index}")
    # join(): the current stream waits for the copy-outs, so an event recorded on it comes after them.
    out = torch.full((m, n), float("nan")).pin_memory()
    pipeline(inputs[0], b, out=out, overlap_calls=True)
    pipeline.join()
    torch.cuda.current_stream().synchronize()
    check(oracle, out, inputs[0], b, None, 1.0, 0.0, "joined call")


def test_one_shot_form_and_checks(binding, oracle):
    a = torch.randn(130, 64).pin_memory()
    b = torch.randn(64, 72).pin_memory()
    out = binding.gemm_host(a, b, band_rows=64)
    torch.cuda.synchronize()
    check(oracle, out, a, b, None, 1.0, 0.0, "one-shot")
    with pytest.raises(RuntimeError, match="host tensor"):
        binding.gemm_host(a.cuda(), b)
    with pytest.raises(RuntimeError, match="reduction depth"):
        binding.gemm_host(a, torch.randn(65, 72))
    with pytest.raises(RuntimeError, match="FP32"):
        binding.gemm_host(a.double(), b)


def test_band_ranges():
    from flash_train.torch import band_ranges

    assert band_ranges(0, 128) == []
    assert band_ranges(100, 128) == [(0, 100)]
    assert band_ranges(300, 128) == [(0, 128), (128, 256), (256, 300)]
    with pytest.raises(ValueError):
        band_ranges(10, 0)
