"""flash_train: FP32 GEMM operator library for NVIDIA B200 (sm_100a).

Same package surface as the reference (python/flash_train/__init__.py:10-15
there): the framework bindings are submodules imported on first use, so
`import flash_train` itself needs neither PyTorch nor a GPU.
"""
import importlib
import typing

__version__ = "0.1.0"

_LAZY_SUBMODULES = ("torch", "capi", "sharded")


def __getattr__(name: str) -> typing.Any:
    # A plain `from . import torch` here would recurse through this hook.
    if name in _LAZY_SUBMODULES:
        return importlib.import_module(f".{name}", __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = list(_LAZY_SUBMODULES)
