"""PyTorch binding: `gemm(a, b, c=None, alpha=1.0, beta=0.0) -> Tensor`, plus
`HostGemm` / `gemm_host` for operands in pinned host memory (host_pipeline.py).

Signature, defaults, checks and error type (RuntimeError) are those of the
reference binding (python/flash_train/torch/csrc/flash_train_torch.cpp:34-75
there). The work is done by libflash_train.so through ftrainGemm; there is no
fallback: a missing extension or library is an error.
"""
import ctypes
import os

# The extension links against libtorch, which enters the process with torch.
import torch  # noqa: F401

_package_root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_native_library = os.path.join(_package_root, "libflash_train.so")
if not os.path.exists(_native_library):
    raise RuntimeError(
        f"{_native_library} is missing: build it with `python flash-train_b200/build.py` "
        "(there is no pure-Python or CPU fallback)"
    )
# Loading by absolute path pins this copy over anything on LD_LIBRARY_PATH.
ctypes.CDLL(_native_library, mode=ctypes.RTLD_GLOBAL)

try:
    from ._flash_train_torch import gemm, last_message
except ModuleNotFoundError as exc:
    if exc.name != "flash_train.torch._flash_train_torch":
        raise
    raise RuntimeError(
        "the torch binding has not been built: run `python flash-train_b200/build.py`"
    ) from exc

from .host_pipeline import HostGemm, band_ranges, gemm_host  # noqa: E402

__all__ = ["gemm", "last_message", "HostGemm", "gemm_host", "band_ranges"]
