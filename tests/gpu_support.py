"""Helpers for the GPU tests: torch tensors as device memory, the library's
C ABI (through flash_train.capi) as the thing under test."""
from __future__ import annotations

import torch

from flash_train import capi

ALL_PRIMITIVES = ("Fp32Gemm", "Fp32Gemm3xTf32", "Fp32GemmSkinny", "Fp32Gemm3xTf32SplitK", "Fp32GemmSplitK",
                  "Fp32Gemm3xTf32FewRows")
EXACT_PRIMITIVES = ("Fp32Gemm", "Fp32GemmSkinny", "Fp32GemmSplitK")

_binding = None


def binding() -> capi.GemmBinding:
    global _binding
    if _binding is None:
        # Roles added in another order than the library's own supported Pattern,
        # like the reference's staged test fixture (tests/api/gemm_staged_fixture.hpp:20-29).
        _binding = capi.GemmBinding(order=("d", "beta", "a", "alpha", "c", "b"))
    return _binding


def operand(tensor: torch.Tensor):
    dims = tuple(tensor.shape)
    strides = None if tensor.is_contiguous() else tuple(tensor.stride())
    return tensor.data_ptr(), dims, strides


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def make_plan(a, b, c, d, alpha=1.0, beta=0.0) -> capi.Plan:
    m, n = d.shape
    c_operand = operand(c) if c is not None else capi.null_operand(m, n)
    return binding().make_plan(operand(a), operand(b), c_operand, operand(d), alpha, beta)


def run_plan(plan: capi.Plan, index: int = 0, device=None):
    """Executes one primitive with exactly the workspace it asks for. Returns the workspace tensor."""
    size = plan.workspace_bytes(index)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device or "cuda")
    plan.execute(index, workspace.data_ptr() if size else 0, size, current_stream())
    return workspace


def gemm(a, b, c=None, alpha=1.0, beta=0.0, primitive: str | None = None, out=None):
    """D = alpha * A @ B + beta * C through Plan create/execute. `primitive`
    names the kernel to run; None runs index 0 (the Finder's choice).
    Returns (d, names) after synchronising."""
    m, n = a.shape[0], b.shape[1]
    d = out if out is not None else torch.full((m, n), float("nan"), device=a.device, dtype=torch.float32)
    plan = make_plan(a, b, c, d, alpha, beta)
    names = plan.primitive_names()
    index = 0 if primitive is None else names.index(primitive)
    workspace = run_plan(plan, index, a.device)
    torch.cuda.synchronize()
    del workspace
    return d, names


def float64_reference(a, b, c=None, alpha=1.0, beta=0.0):
    out = alpha * (a.double() @ b.double())
    if c is not None:
        out = out + beta * c.double()
    return out
