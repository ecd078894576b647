"""ORACLE -- TEST INFRASTRUCTURE ONLY. Builds the checkers.

  oracle/libftoracle.so             the C restatement (oracle/host_gemm.c)
  oracle/_ref/libflash_train_ref.so the REFERENCE's own sources, compiled for the
                                    CPU where they lie (never copied): every
                                    src/**/*.cpp plus the kernel file
                                    src/primitive/hygon/gemm/fp32_gemm.hip,
                                    against the stand-in HIP headers in
                                    oracle/hip_shim/. Built only where the
                                    reference checkout exists; the result
                                    exports the same 29 ftrain* symbols.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# The reference checkout: $FTRAIN_REFERENCE, else a directory named "reference" beside this repository.
REFERENCE = Path(os.environ["FTRAIN_REFERENCE"]) if os.environ.get("FTRAIN_REFERENCE") else HERE.parent.parent / "reference"


def _run(command: list[str]) -> None:
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(command) + "\n" + result.stdout + result.stderr)


def build_restatement() -> Path:
    target = HERE / "libftoracle.so"
    source = HERE / "host_gemm.c"
    if not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
        _run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", str(source), "-o", str(target), "-lm"])
    return target


def build_reference() -> Path | None:
    """Returns the library path, or None when there is no reference checkout."""
    target = HERE / "_ref" / "libflash_train_ref.so"
    if not (REFERENCE / "src").is_dir():
        return target if target.exists() else None
    if target.exists():
        return target
    out = HERE / "_ref"
    generated = out / "gen" / "flash_train"
    generated.mkdir(parents=True, exist_ok=True)
    control = (REFERENCE / "include/flash_train/control.h.in").read_text()
    control = control.replace("#cmakedefine01 FTRAIN_PLATFORM_HYGON_HIP", "#define FTRAIN_PLATFORM_HYGON_HIP 1")
    control = control.replace("@FTRAIN_HYGON_HIP_ARCHS@", "cpu")
    (generated / "control.h").write_text(control)
    version = (REFERENCE / "VERSION.txt").read_text().strip()
    major, minor, patch = version.split(".")
    (generated / "version.h").write_text(
        "#ifndef FTRAIN_VERSION_H_\n#define FTRAIN_VERSION_H_\n"
        f"#define FTRAIN_VERSION_MAJOR {major}\n#define FTRAIN_VERSION_MINOR {minor}\n"
        f"#define FTRAIN_VERSION_PATCH {patch}\n#define FTRAIN_VERSION \"{version}\"\n#endif\n")
    flags = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-DFTRAIN_BUILDING",
             f"-I{out / 'gen'}", f"-I{REFERENCE / 'include'}", f"-I{REFERENCE / 'src' / 'include'}",
             f"-I{HERE / 'hip_shim'}"]
    sources = sorted((REFERENCE / "src").rglob("*.cpp")) + sorted((REFERENCE / "src").rglob("*.hip"))
    objects = []
    jobs = []
    for index, source in enumerate(sources):
        obj = out / f"{index:02d}_{source.stem}.o"
        objects.append(obj)
        jobs.append(["g++", *flags, "-x", "c++", "-c", str(source), "-o", str(obj)])
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_run, jobs))
    _run(["g++", "-shared", "-o", str(target), *map(str, objects), "-lpthread"])
    return target


def main() -> int:
    print(build_restatement())
    print(build_reference())
    return 0


if __name__ == "__main__":
    sys.exit(main())
