"""The C ABI without a GPU: the shared library loads, exports every function the
headers under include/ declare, lays out its structs like the reference, and the
device-free part of the staged API behaves like the reference's own build of the
same API (driven side by side where the reference checkout is available)."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
INCLUDE = REPO / "include"


def declared_functions():
    names = []
    for header in sorted(INCLUDE.rglob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"\b(?:FTRAIN_API|FTCUDA_API)\s+[\w\s\*]+?\b(ftrain\w+|ftcuda_\w+)\s*\(", text)
    return sorted(set(names))


def test_headers_declare_the_reference_api(capi):
    names = declared_functions()
    assert set(capi.EXPORTED_SYMBOLS) <= set(names)
    assert len([n for n in names if n.startswith("ftrain")]) == 29
    assert set(capi.PLATFORM_SYMBOLS) == {n for n in names if n.startswith("ftcuda_")}


def test_library_exports_every_declared_symbol(capi, native_library):
    exported = subprocess.run(["nm", "-D", "--defined-only", str(native_library)], capture_output=True, text=True).stdout
    defined = {line.split()[-1] for line in exported.splitlines() if " T " in line}
    for name in declared_functions():
        assert name in defined, f"{name} is declared in include/ but not exported"
        assert getattr(capi.lib, name) is not None
    # Nothing else leaks out of the library.
    assert {n for n in defined if not n.startswith(("ftrain", "ftcuda_"))} == set()


def test_headers_compile_as_c_and_struct_layout(tmp_path, capi):
    source = tmp_path / "abi.c"
    source.write_text(
        '#include <flash_train/flash_train.h>\n#include <flash_train/env.h>\n#include <ftcuda/ftcuda.h>\n#include <stdio.h>\n'
        '#include <stddef.h>\n'
        'int main(void) { printf("%zu %zu %zu %zu %zu %zu %d %d %s\\n", sizeof(FTrainStorageView), '
        'offsetof(FTrainStorageView, num_dims), offsetof(FTrainStorageView, is_host_memory), sizeof(FTrainTensorId), '
        'sizeof(FtcudaGemmDesc), sizeof(FtcudaGemmLaunch), FTRAIN_STATUS_INTERNAL_ERROR, FTRAIN_NUMERIC_TYPE_COUNT, '
        'FTRAIN_DISABLE_CACHE); return 0; }\n')
    binary = tmp_path / "abi"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", f"-I{INCLUDE}", str(source), "-o", str(binary)], check=True)
    fields = subprocess.run([str(binary)], capture_output=True, text=True, check=True).stdout.split()
    assert fields == ["32", "24", "27", "8", str(ctypes.sizeof(capi.GemmDesc)), "1280", "50", "24", "FTRAIN_DISABLE_CACHE"]
    assert ctypes.sizeof(capi.StorageView) == 32 and ctypes.sizeof(capi.GemmLaunch) == 1280


def api_script(capi, lib):
    """A fixed sequence of device-free calls; returns the list of (step, status)."""
    trace = []

    def record(step, call):
        try:
            call()
            trace.append((step, capi.STATUS_SUCCESS))
        except capi.FTrainError as error:
            trace.append((step, error.status))

    null = ctypes.c_void_p()
    trace.append(("create(NULL)", int(lib.ftrainPatternCreate(None))))
    trace.append(("destroy(NULL)", int(lib.ftrainPatternDestroy(null))))
    trace.append(("ops(NULL)", int(lib.ftrainOpsCreate(ctypes.byref(ctypes.c_void_p()), null))))
    trace.append(("args(NULL)", int(lib.ftrainArgsCreate(ctypes.byref(ctypes.c_void_p()), null))))
    trace.append(("plan(NULL)", int(lib.ftrainPlanCreate(ctypes.byref(ctypes.c_void_p()), null))))
    trace.append(("execute(NULL)", int(lib.ftrainPlanExecutePrimitive(null, 0, None, 0, None))))

    pattern = capi.Pattern(lib)
    ids = [pattern.add_tensor().opaque for _ in range(3)] + [pattern.add_tensor_list().opaque,
                                                            pattern.add_grouped_tensor().opaque]
    trace.append(("ids", tuple(ids)))
    record("ops(no operation, dangling operands)", lambda: capi.Ops(pattern))

    # Wiring errors are reported by OpsCreate, not by Add.
    bad = capi.Pattern(lib)
    t = [bad.add_tensor() for _ in range(6)]
    record("add duplicate input", lambda: bad.add_gemm(t[0], t[0], t[2], t[5], t[3], t[4]))
    record("ops(duplicate input)", lambda: capi.Ops(bad))
    out_of_range = capi.Pattern(lib)
    t = [out_of_range.add_tensor() for _ in range(6)]
    record("add out of range", lambda: out_of_range.add_gemm(t[0], t[1], t[2], capi.RoleId(40), t[3], t[4]))
    record("ops(out of range)", lambda: capi.Ops(out_of_range))

    # Two Gemm nodes chained through one matrix: a graph with no engine on either side.
    chained = capi.Pattern(lib)
    n = [chained.add_tensor() for _ in range(10)]
    record("add chained", lambda: (chained.add_gemm(n[0], n[1], n[2], n[3], n[4], n[5]), chained.add_gemm(n[3], n[6], n[7], n[8], n[4], n[5])))
    record("ops(chained: no engine)", lambda: capi.Ops(chained))

    for order in (("a", "b", "c", "alpha", "beta", "d"), ("d", "c", "b", "a", "beta", "alpha")):
        binding = capi.GemmBinding(order=order, lib=lib)
        args = capi.Args(binding.ops)
        cell = ctypes.c_float(1.0)
        dims_ok, keep1 = capi.make_view(0x1000, (4, 3))
        record("set a", lambda: args.set_tensor(binding.roles["a"], dims_ok))
        record("set role out of range", lambda: args.set_tensor(capi.RoleId(99), dims_ok))
        negative, keep2 = capi.make_view(0x1000, (4, -3))
        record("set negative dim", lambda: args.set_tensor(binding.roles["a"], negative))
        both, keep3 = capi.make_view(0x1000, (4, 3), strides=(3, 1), index_type=capi.INDEX_CONTINUOUS)
        record("set strides and index type", lambda: args.set_tensor(binding.roles["a"], both))
        neither, keep4 = capi.make_view(0x1000, (4, 3), index_type=capi.INDEX_INVALID)
        record("set no layout", lambda: args.set_tensor(binding.roles["a"], neither))
        scalar_null, keep5 = capi.make_view(0, (), host=True)
        record("set null scalar", lambda: args.set_tensor(binding.roles["alpha"], scalar_null))
        scalar, keep6 = capi.make_view(ctypes.addressof(cell), (), host=True)
        record("set scalar", lambda: args.set_tensor(binding.roles["alpha"], scalar))
        bad_type, keep7 = capi.make_view(0x1000, (4, 3), numeric_type=capi.NUMERIC_COUNT)
        record("set bad numeric type", lambda: args.set_tensor(binding.roles["b"], bad_type))
        record("set gemm invalid type", lambda: args.set_gemm(binding.gemm, 0))
        record("set gemm COUNT", lambda: args.set_gemm(binding.gemm, capi.NUMERIC_COUNT))
        record("set gemm wrong op id", lambda: args.set_gemm(capi.RoleId(5), capi.NUMERIC_FP32))
        record("set gemm", lambda: args.set_gemm(binding.gemm, capi.NUMERIC_FP32))
        record("set tensor list on a tensor role",
               lambda: capi.check(lib.ftrainArgsSetTensorList(args.handle, binding.roles["c"], None, 0), lib))
    return trace


def test_device_free_api_statuses(capi):
    trace = dict(api_script(capi, capi.lib))
    invalid, unsupported, ok = capi.STATUS_INVALID_ARGUMENT, capi.STATUS_UNSUPPORTED, capi.STATUS_SUCCESS
    for step in ("create(NULL)", "destroy(NULL)", "ops(NULL)", "args(NULL)", "plan(NULL)", "execute(NULL)"):
        assert trace[step] == invalid
    assert trace["ids"] == (0, 1, 2, 3, 4)
    assert trace["ops(no operation, dangling operands)"] == unsupported
    assert trace["add duplicate input"] == ok and trace["ops(duplicate input)"] == invalid
    assert trace["add out of range"] == ok and trace["ops(out of range)"] == invalid
    assert trace["add chained"] == ok and trace["ops(chained: no engine)"] == unsupported
    assert trace["set a"] == ok and trace["set scalar"] == ok and trace["set gemm"] == ok
    for step in ("set role out of range", "set negative dim", "set strides and index type", "set no layout",
                 "set null scalar", "set bad numeric type", "set gemm invalid type", "set gemm COUNT",
                 "set gemm wrong op id", "set tensor list on a tensor role"):
        assert trace[step] == invalid, step


def test_same_statuses_as_the_reference_build(capi, reference_capi):
    if reference_capi is None:
        pytest.skip("no reference checkout in this environment")
    assert api_script(capi, capi.lib) == api_script(capi, reference_capi)
    # And the wording of the messages that callers and the reference's tests match on.
    for lib in (capi.lib, reference_capi):
        assert int(lib.ftrainPatternCreate(None)) == capi.STATUS_INVALID_ARGUMENT
        assert capi.last_message(lib) == "ftrainPatternCreate: pattern output must not be null"
        assert capi.last_status(lib) == capi.STATUS_INVALID_ARGUMENT


def test_grouped_gemms_have_engines_here(capi, reference_capi):
    """The one place where this library answers differently from the reference on purpose: the three
    grouped GEMM graphs (declared by the reference's public header, without engines there) match."""
    def ops_status(lib, kind):
        pattern = capi.Pattern(lib)
        lists = capi.GroupedGemmBinding.LIST_ROLES[kind]
        roles = {name: (pattern.add_tensor_list() if name in lists else pattern.add_grouped_tensor()) for name in "abcd"}
        alpha, beta = pattern.add_tensor(), pattern.add_tensor()
        pattern.add_gemm(roles["a"], roles["b"], roles["c"], roles["d"], alpha, beta, kind=kind)
        try:
            capi.Ops(pattern)
            return capi.STATUS_SUCCESS
        except capi.FTrainError as error:
            return error.status

    for kind in ("GroupedABCDGemm", "GroupedBCDGemm", "GroupedABGemm"):
        assert ops_status(capi.lib, kind) == capi.STATUS_SUCCESS, kind
        if reference_capi is not None:
            assert ops_status(reference_capi, kind) == capi.STATUS_UNSUPPORTED, kind


def test_plan_creation_without_a_device_fails_loudly(capi):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    binding = capi.GemmBinding()
    with pytest.raises(capi.FTrainError) as info:
        binding.make_plan((0x1000, (4, 3), None), (0x2000, (3, 5), None), (0, (4, 5), None), (0x3000, (4, 5), None))
    assert info.value.status == capi.STATUS_INTERNAL_ERROR and "cudaGetDevice failed" in info.value.message
