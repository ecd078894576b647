"""Builds and runs the C++ white-box tests of the host pipeline (tests/cpp/):
foundation types, pattern matching, selection cache, engine selection with mock
policies, the Gemm family, and the extern "C" layer -- all linked against a fake
of the platform layer's C ABI, so no GPU is involved."""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
CSRC = REPO / "flash-train_b200" / "csrc"
CPP = REPO / "tests" / "cpp"
BUILD = CPP / "_build"


def _compile(job):
    source, target = job
    flags = ["-std=c++17", "-O1", "-g", "-Wall", "-Wextra", "-DFTRAIN_BUILDING", f"-I{CSRC}", f"-I{REPO / 'include'}",
             f"-I{CPP}", "-pthread"]
    result = subprocess.run(["g++", *flags, "-c", str(source), "-o", str(target)], capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    return target


@pytest.fixture(scope="module")
def test_binary():
    BUILD.mkdir(exist_ok=True)
    host = sorted(p for p in CSRC.rglob("*.cpp") if p.relative_to(CSRC).parts[0] not in ("cuda", "bench"))
    sources = host + sorted(CPP.glob("*.cpp"))
    headers = max(p.stat().st_mtime for base in (CSRC, CPP, REPO / "include") for p in base.rglob("*.h*"))
    jobs = []
    objects = []
    for source in sources:
        target = BUILD / (str(source.relative_to(REPO)).replace(os.sep, "__") + ".o")
        objects.append(target)
        if not target.exists() or target.stat().st_mtime < max(headers, source.stat().st_mtime):
            jobs.append((source, target))
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_compile, jobs))
    binary = BUILD / "host_tests"
    result = subprocess.run(["g++", "-o", str(binary), *map(str, objects), "-pthread"], capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    return binary


@pytest.mark.parametrize("group", ["result_", "exception_", "storage_view", "grouped_tensor", "builder_", "build_",
                                   "key_", "symmetric", "matching_", "ops_rejects", "cache_", "name_lists", "engine_",
                                   "create_plan", "problem_", "fp32_gemm_checklist", "configured_clone", "plan_dispatches",
                                   "finder_", "builtin_", "role_ids", "null_arguments", "ops_create", "args_setters",
                                   "tensor_list", "last_status", "one_shot", "grouped_"])
def test_cpp_group(test_binary, group):
    result = subprocess.run([str(test_binary), group], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout[-4000:] + result.stderr[-2000:]


def test_cpp_everything_ran(test_binary):
    result = subprocess.run([str(test_binary)], capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-4000:] + result.stderr[-2000:]
    assert " 0 failed checks" in result.stdout
