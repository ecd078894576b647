"""Accuracy of the 3xTF32 tensor-core kernel as a function of how often its
accumulator is drained into a round-to-nearest FP32 running sum, against
float64, relative to an FP32 FFMA GEMM (torch with TF32 off). Run with -s to
see the table that profiles/tensorGemm3xTf32_accuracy_vs_drain.md records."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [(2048, 4096, 2048, "normal"), (1024, 65536, 1024, "uniform"), (512, 512, 512, "normal")]


def run_case(capi, oracle, m, k, n, distribution, chunk):
    torch.manual_seed(0)
    if distribution == "normal":
        a, b = torch.randn(m, k, device="cuda"), torch.randn(k, n, device="cuda")
    else:
        a, b = torch.rand(m, k, device="cuda") * 2 - 1, torch.rand(k, n, device="cuda") * 2 - 1
    d = torch.empty(m, n, device="cuda")
    operand = lambda t: (t.data_ptr(), tuple(t.shape), None)  # noqa: E731
    desc = capi.make_desc(operand(a), operand(b), (0, (m, n), None), operand(d), 1.0, 0.0, torch.cuda.current_device())
    previous = os.environ.get("FTCUDA_TF32_CHUNK_K_BLOCKS")
    try:
        if chunk is None:
            os.environ.pop("FTCUDA_TF32_CHUNK_K_BLOCKS", None)
        else:
            os.environ["FTCUDA_TF32_CHUNK_K_BLOCKS"] = str(chunk)
        launch = capi.PlatformGemm(capi.KERNEL_TF32X3, desc)  # the knob is read here
    finally:
        if previous is None:
            os.environ.pop("FTCUDA_TF32_CHUNK_K_BLOCKS", None)
        else:
            os.environ["FTCUDA_TF32_CHUNK_K_BLOCKS"] = previous
    stream = torch.cuda.current_stream().cuda_stream
    launch.run(0, 0, stream)
    torch.cuda.synchronize()
    exact = a.double() @ b.double()
    ours = oracle.scaled_error(d, exact, a, b)
    plain = oracle.scaled_error(a @ b, exact, a, b)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        launch.run(0, 0, stream)
    start.record()
    for _ in range(10):
        launch.run(0, 0, stream)
    stop.record()
    torch.cuda.synchronize()
    return ours, plain, 2.0 * m * n * k / (start.elapsed_time(stop) / 10 * 1e-3) / 1e12


def test_default_drain_interval_meets_the_accuracy_bar(capi, oracle):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    torch.backends.cuda.matmul.allow_tf32 = False
    for m, k, n, distribution in CASES:
        ours, plain, _ = run_case(capi, oracle, m, k, n, distribution, None)
        assert ours <= 2.0 * plain, (m, k, n, ours, plain)


def test_drain_interval_sweep_table(capi, oracle):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    torch.backends.cuda.matmul.allow_tf32 = False
    print("\nK blocks between drains | shape | scaled error / FFMA GEMM's | TFLOP/s")
    worst_without = 0.0
    for chunk in (2, 4, 8, 16, 32, 1 << 20):
        for m, k, n, distribution in CASES:
            ours, plain, tflops = run_case(capi, oracle, m, k, n, distribution, chunk)
            print(f"{chunk:>8} | {m}x{k}x{n} {distribution:<7} | {ours / plain:6.2f} | {tflops:6.1f}")
            if chunk == 1 << 20:
                worst_without = max(worst_without, ours / plain)
    # Without drains the truncating accumulation shows clearly; this is why the drains exist.
    assert worst_without > 4.0
