"""Regenerates tests/golden/*.npz. Needs the reference checkout (to build
oracle/_ref) and is therefore run by hand in the development container:

    python oracle/build_oracle.py && python tests/golden/make_golden.py

Two fixtures:
  reference_grid.npz   outputs of the REFERENCE's own code (its C++ pipeline and
                       its kernel source, compiled for the CPU) on the 7-shape
                       grid of its numerics test, alpha 1.5, beta 0 with a null
                       C and beta 1.25 (tests/api/gemm_numerics_test.cpp:55-137).
  torch_config1.npz    the reference's PyTorch expression on the 128x64x96
                       seed-0 case, in float32 and float64, computed on the CPU.
"""
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "flash-train_b200" / "python"))

from flash_train import capi  # noqa: E402
from oracle import oracle  # noqa: E402

GRID = [(1, 1, 1), (3, 4, 2), (16, 16, 16), (64, 48, 32), (129, 65, 17), (33, 257, 65), (256, 128, 64)]


def operand(array):
    return array.ctypes.data, array.shape, None


def main() -> None:
    path = oracle.reference_library_path()
    if path is None:
        raise SystemExit("oracle/_ref is not built: run oracle/build_oracle.py where the reference checkout exists")
    ref = capi.bind(path)
    binding = capi.GemmBinding(lib=ref)
    out = {}
    for m, k, n in GRID:
        a, b, c = oracle.grid_inputs(m, k, n)
        d = np.zeros((m, n), np.float32)
        plan = binding.make_plan(operand(a), operand(b), capi.null_operand(m, n), operand(d), 1.5, 0.0)
        plan.execute()
        out[f"fresh_{m}x{k}x{n}"] = d.copy()
        plan = binding.make_plan(operand(a), operand(b), operand(c), operand(d), 1.5, 1.25)
        plan.execute()
        out[f"accumulated_{m}x{k}x{n}"] = d.copy()
    np.savez_compressed(Path(__file__).with_name("reference_grid.npz"), **out)

    import torch

    torch.manual_seed(0)
    a = torch.randn(128, 64)
    b = torch.randn(64, 96)
    np.savez_compressed(Path(__file__).with_name("torch_config1.npz"), a=a.numpy(), b=b.numpy(),
                        d32=(a @ b).numpy(), d64=(a.double() @ b.double()).numpy())
    print("wrote", sorted(p.name for p in Path(__file__).parent.glob("*.npz")))


if __name__ == "__main__":
    main()
