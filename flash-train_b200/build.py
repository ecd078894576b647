"""Builds the native pieces in-tree.

  python flash-train_b200/build.py            # libflash_train.so + torch binding
  python flash-train_b200/build.py --no-torch # library only

Outputs (next to the Python package, the layout of the reference wheel,
python/flash_train/torch/__init__.py:15-18 there):
  flash-train_b200/python/flash_train/libflash_train.so
  flash-train_b200/python/flash_train/torch/_flash_train_torch*.so
  flash-train_b200/python/flash_train/bin/plan_reuse_bench

Host C++ is compiled with g++, CUDA sources with nvcc for sm_100a only
(-gencode arch=compute_100a,code=sm_100a); the CUDA runtime is linked
statically so the library does not depend on which libcudart a host process
(for instance PyTorch) has loaded. Object files are cached under
flash-train_b200/build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
INCLUDE = REPO / "include"
OBJ = ROOT / "build"
PACKAGE = ROOT / "python" / "flash_train"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-DFTRAIN_BUILDING", "-Wall", "-Wextra",
              f"-I{CSRC}", f"-I{INCLUDE}"]
CUDA_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{CSRC / 'cuda'}", f"-I{INCLUDE}"]


def _newest_header() -> float:
    stamps = [p.stat().st_mtime for pattern in ("*.h", "*.hpp", "*.cuh")
              for base in (CSRC, INCLUDE) for p in base.rglob(pattern)]
    stamps.append(Path(__file__).stat().st_mtime)
    return max(stamps)


def _stale(target: Path, sources: list[Path], headers: float) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return stamp < headers or any(stamp < s.stat().st_mtime for s in sources)


def _run(command: list[str]) -> None:
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(command) + "\n" + result.stdout + result.stderr)


def host_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cpp") if p.relative_to(CSRC).parts[0] not in ("cuda", "bench"))


def cuda_sources() -> list[Path]:
    return sorted((CSRC / "cuda").glob("*.cu"))


def _object_for(source: Path) -> Path:
    return OBJ / (str(source.relative_to(CSRC)).replace(os.sep, "__") + ".o")


def compile_objects(sources: list[Path], verbose: bool) -> list[Path]:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = _newest_header()
    jobs = []
    for source in sources:
        target = _object_for(source)
        if not _stale(target, [source], headers):
            continue
        if source.suffix == ".cu":
            jobs.append([NVCC, *CUDA_FLAGS, "-c", str(source), "-o", str(target)])
        else:
            jobs.append(["g++", *HOST_FLAGS, "-c", str(source), "-o", str(target)])
    if verbose and jobs:
        print(f"[build] compiling {len(jobs)} translation units", flush=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_run, jobs))
    return [_object_for(s) for s in sources]


def build_library(verbose: bool = True) -> Path:
    """libflash_train.so: host pipeline + CUDA platform subtree."""
    sources = host_sources() + cuda_sources()
    objects = compile_objects(sources, verbose)
    target = PACKAGE / "libflash_train.so"
    if _stale(target, objects, 0.0):
        _run([NVCC, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
              "-o", str(target), *map(str, objects), "-Xlinker", "--exclude-libs,ALL", "-lpthread", "-ldl"])
        if verbose:
            print(f"[build] linked {target.relative_to(REPO)}", flush=True)
    return target


def build_plan_bench(verbose: bool = True) -> Path:
    """bin/plan_reuse_bench: host cost of Plan reuse measured from C++ (no binding in the way)."""
    library = build_library(verbose)
    source = CSRC / "bench" / "plan_reuse_bench.cpp"
    target = PACKAGE / "bin" / "plan_reuse_bench"
    target.parent.mkdir(exist_ok=True)
    if _stale(target, [source, library], _newest_header()):
        _run([NVCC, "-std=c++17", "-O2", "-cudart", "static", f"-I{INCLUDE}", str(source), "-o", str(target),
              f"-L{PACKAGE}", "-lflash_train", "-Xlinker", "-rpath,$ORIGIN/.."])
        if verbose:
            print(f"[build] built {target.relative_to(REPO)}", flush=True)
    return target


def build_torch_binding(verbose: bool = True) -> Path:
    """The pybind11 module behind flash_train.torch.gemm."""
    import torch
    from torch.utils import cpp_extension

    library = build_library(verbose)
    source = PACKAGE / "torch" / "csrc" / "flash_train_torch.cpp"
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = PACKAGE / "torch" / ("_flash_train_torch" + suffix)
    if not _stale(target, [source, library], _newest_header()):
        return target
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    includes = [f"-I{p}" for p in cpp_extension.include_paths()]
    includes += [f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}", f"-I{CUDA_HOME / 'include'}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
          "-DTORCH_EXTENSION_NAME=_flash_train_torch", "-DTORCH_API_INCLUDE_EXTENSION_H",
          f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *includes, str(source), "-o", str(target),
          f"-L{PACKAGE}", "-lflash_train", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10",
          "-lc10_cuda", "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{torch_lib}"])
    if verbose:
        print(f"[build] built {target.relative_to(REPO)}", flush=True)
    return target


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--no-torch", action="store_true", help="skip the PyTorch binding")
    parser.add_argument("--quiet", action="store_true")
    options = parser.parse_args()
    build_library(not options.quiet)
    build_plan_bench(not options.quiet)
    if not options.no_torch:
        build_torch_binding(not options.quiet)
    return 0


if __name__ == "__main__":
    sys.exit(main())
