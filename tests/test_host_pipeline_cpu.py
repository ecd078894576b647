"""Host-side logic of flash_train.torch.host_pipeline that needs no device: the band partition and the
argument checks (the module file is loaded on its own, without the compiled binding)."""
import importlib.util
from pathlib import Path

import pytest
import torch

MODULE = Path(__file__).resolve().parents[1] / "flash-train_b200" / "python" / "flash_train" / "torch" / "host_pipeline.py"


@pytest.fixture(scope="module")
def host_pipeline():
    spec = importlib.util.spec_from_file_location("host_pipeline_under_test", MODULE)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_band_ranges_cover_rows_once(host_pipeline):
    assert host_pipeline.band_ranges(0, 128) == []
    assert host_pipeline.band_ranges(100, 128) == [(0, 100)]
    assert host_pipeline.band_ranges(300, 128) == [(0, 128), (128, 256), (256, 300)]
    for m, band in ((1, 1), (17, 5), (4096, 512), (4097, 512)):
        ranges = host_pipeline.band_ranges(m, band)
        assert ranges[0][0] == 0 and ranges[-1][1] == m
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert all(0 < stop - start <= band for start, stop in ranges)
    with pytest.raises(ValueError):
        host_pipeline.band_ranges(10, 0)


def test_host_matrix_checks(host_pipeline):
    check = host_pipeline._check_host_matrix
    check(torch.zeros(3, 4), "a")
    with pytest.raises(RuntimeError, match="FP32"):
        check(torch.zeros(3, 4, dtype=torch.float64), "a")
    with pytest.raises(RuntimeError, match="rank two"):
        check(torch.zeros(3), "a")
    with pytest.raises(RuntimeError, match="contiguous"):
        check(torch.zeros(4, 3).t(), "a")
