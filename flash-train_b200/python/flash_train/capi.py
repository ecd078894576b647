"""ctypes view of libflash_train.so: the public C API, one-to-one.

This is the binding a Python caller that does not want the PyTorch extension
uses, and what the tests and the benchmark call, so that they exercise exactly
the exported C ABI (include/flash_train/common.h, flash_train.h). Nothing here
computes: every function forwards to the shared library, and importing this
module fails if the library has not been built.

The small classes (Pattern, Ops, Args, Plan) only own a handle and destroy it;
`GemmBinding` packages the staged sequence for the one supported graph,
D = alpha * A @ B + beta * C.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_bool, c_char_p, c_int64, c_uint8, c_uint32, c_uint64, c_void_p

STATUS_SUCCESS = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_OUT_OF_MEMORY = 2
STATUS_OVERFLOW = 3
STATUS_UNSUPPORTED = 4
STATUS_INTERNAL_ERROR = 50

NUMERIC_FP64 = 1
NUMERIC_INT64 = 2
NUMERIC_FP32 = 4
NUMERIC_FP16 = 7
NUMERIC_COUNT = 24

INDEX_INVALID = 0  # layout given by strides
INDEX_CONTINUOUS = 1
INDEX_NVIDIA_SF_128X4_SWIZZLED = 2
INDEX_GROUPED_CONTINUOUS = 3
INDEX_COUNT = 4

LIBRARY_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libflash_train.so")

EXPORTED_SYMBOLS = (
    "ftrainGetLastStatus ftrainGetLastMessage ftrainPatternCreate ftrainPatternDestroy ftrainPatternAddTensor "
    "ftrainPatternAddTensorList ftrainPatternAddGroupedTensor ftrainPatternAddGemm ftrainPatternAddGroupedABCDGemm "
    "ftrainPatternAddGroupedBCDGemm ftrainPatternAddGroupedABGemm ftrainOpsCreate ftrainOpsDestroy ftrainArgsCreate "
    "ftrainArgsDestroy ftrainArgsSetTensor ftrainArgsSetTensorList ftrainArgsSetGroupedTensor ftrainArgsSetGemm "
    "ftrainArgsSetGroupedABCDGemm ftrainArgsSetGroupedBCDGemm ftrainArgsSetGroupedABGemm ftrainPlanCreate "
    "ftrainPlanDestroy ftrainPlanGetNumPrimitives ftrainPlanGetPrimitiveName "
    "ftrainPlanGetPrimitiveRequiredWorkspaceBytes ftrainPlanExecutePrimitive ftrainGemm"
).split()

PLATFORM_SYMBOLS = (
    "ftcuda_current_device ftcuda_device_sm_count ftcuda_gemm_supports ftcuda_gemm_configure "
    "ftcuda_gemm_workspace_bytes ftcuda_gemm_launch ftcuda_launch_count ftcuda_trace_push ftcuda_trace_pop "
    "ftcuda_trace_mark ftcuda_gemm_splitk_static ftcuda_gemm_splitk_static_capacity ftcuda_gemm_launch_scatter "
    "ftcuda_device_status ftcuda_device_status_reset ftcuda_selftest_bounded_wait ftcuda_measure_ffma_tflops "
    "ftcuda_grouped_gemm_supports ftcuda_grouped_gemm_configure ftcuda_grouped_gemm_workspace_bytes "
    "ftcuda_grouped_gemm_launch ftcuda_grouped_gemm_destroy"
).split()


class StorageView(Structure):
    """FTrainStorageView (32 bytes on LP64)."""

    _fields_ = [
        ("memory", c_void_p),
        ("dims", POINTER(c_int64)),
        ("strides", POINTER(c_int64)),
        ("num_dims", c_uint8),
        ("numeric_type", c_uint8),
        ("index_type", c_uint8),
        ("is_host_memory", c_bool),
    ]


class RoleId(Structure):
    """Every FTrain*Id type: struct { uint64_t opaque; } passed by value."""

    _fields_ = [("opaque", c_uint64)]


class FTrainError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"flash_train status {status}: {message}")
        self.status = status
        self.message = message


def bind(path: str) -> ctypes.CDLL:
    """Loads a shared library exporting the flash_train C API and declares its signatures."""
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python flash-train_b200/build.py` "
            "(there is no pure-Python or CPU fallback)"
        )
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    status = c_uint8
    lib.ftrainGetLastStatus.restype = status
    lib.ftrainGetLastMessage.restype = c_char_p
    handle_out = POINTER(c_void_p)
    role_out = POINTER(RoleId)
    signatures = {
        "ftrainPatternCreate": [handle_out],
        "ftrainPatternDestroy": [c_void_p],
        "ftrainPatternAddTensor": [c_void_p, role_out],
        "ftrainPatternAddTensorList": [c_void_p, role_out],
        "ftrainPatternAddGroupedTensor": [c_void_p, role_out],
        "ftrainPatternAddGemm": [c_void_p, role_out] + [RoleId] * 6,
        "ftrainPatternAddGroupedABCDGemm": [c_void_p, role_out] + [RoleId] * 6,
        "ftrainPatternAddGroupedBCDGemm": [c_void_p, role_out] + [RoleId] * 6,
        "ftrainPatternAddGroupedABGemm": [c_void_p, role_out] + [RoleId] * 6,
        "ftrainOpsCreate": [handle_out, c_void_p],
        "ftrainOpsDestroy": [c_void_p],
        "ftrainArgsCreate": [handle_out, c_void_p],
        "ftrainArgsDestroy": [c_void_p],
        "ftrainArgsSetTensor": [c_void_p, RoleId, StorageView],
        "ftrainArgsSetTensorList": [c_void_p, RoleId, POINTER(StorageView), c_uint32],
        "ftrainArgsSetGroupedTensor": [c_void_p, RoleId, c_uint32, StorageView, POINTER(StorageView),
                                       POINTER(StorageView), POINTER(StorageView)],
        "ftrainArgsSetGemm": [c_void_p, RoleId, c_uint8],
        "ftrainArgsSetGroupedABCDGemm": [c_void_p, RoleId, c_uint8],
        "ftrainArgsSetGroupedBCDGemm": [c_void_p, RoleId, c_uint8],
        "ftrainArgsSetGroupedABGemm": [c_void_p, RoleId, c_uint8],
        "ftrainPlanCreate": [handle_out, c_void_p],
        "ftrainPlanDestroy": [c_void_p],
        "ftrainPlanGetNumPrimitives": [c_void_p, POINTER(c_uint64)],
        "ftrainPlanGetPrimitiveName": [c_void_p, c_uint64, POINTER(c_char_p)],
        "ftrainPlanGetPrimitiveRequiredWorkspaceBytes": [c_void_p, c_uint64, POINTER(c_uint64)],
        "ftrainPlanExecutePrimitive": [c_void_p, c_uint64, c_void_p, c_uint64, c_void_p],
        "ftrainGemm": [StorageView] * 6 + [c_uint8, c_void_p, c_uint64, c_void_p],
    }
    for name, argtypes in signatures.items():
        function = getattr(lib, name)
        function.argtypes = argtypes
        function.restype = status
    if hasattr(lib, "ftcuda_launch_count"):
        lib.ftcuda_launch_count.restype = c_uint64
        lib.ftcuda_launch_count.argtypes = []
    return lib


# The product library. Every class below takes an optional `lib=` so that the
# same Python code can drive another build of the same C API (the tests drive
# the reference's own sources, compiled for the CPU, this way).
lib = bind(LIBRARY_PATH)


def last_status(lib=lib) -> int:
    return int(lib.ftrainGetLastStatus())


def last_message(lib=lib) -> str:
    return lib.ftrainGetLastMessage().decode()


def launch_count() -> int:
    """Device kernels the library has enqueued from this process so far."""
    return int(lib.ftcuda_launch_count())


def check(status: int, lib=lib) -> None:
    if status != STATUS_SUCCESS:
        raise FTrainError(int(status), last_message(lib))


def make_view(memory, dims, strides=None, numeric_type=NUMERIC_FP32, index_type=None, host=False):
    """Builds an FTrainStorageView plus the ctypes arrays it points to.

    Returns (view, keepalive); keep `keepalive` referenced until the call that
    receives the view has returned (the library copies dims/strides then).
    """
    dims = list(dims)
    dims_array = (c_int64 * max(len(dims), 1))(*dims) if dims else None
    strides_array = (c_int64 * len(strides))(*strides) if strides is not None else None
    if index_type is None:
        index_type = INDEX_INVALID if strides is not None else INDEX_CONTINUOUS
    view = StorageView(
        c_void_p(memory),
        ctypes.cast(dims_array, POINTER(c_int64)) if dims_array is not None else None,
        ctypes.cast(strides_array, POINTER(c_int64)) if strides_array is not None else None,
        len(dims), numeric_type, index_type, host,
    )
    return view, (dims_array, strides_array)


class _Handle:
    _destroy = None

    def __init__(self, lib):
        self.lib = lib
        self.handle = c_void_p()

    def check(self, status: int) -> None:
        check(status, self.lib)

    def close(self):
        if self.handle:
            getattr(self.lib, self._destroy)(self.handle)
            self.handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Pattern(_Handle):
    _destroy = "ftrainPatternDestroy"

    def __init__(self, lib=lib):
        super().__init__(lib)
        self.check(lib.ftrainPatternCreate(byref(self.handle)))

    def _add(self, function) -> RoleId:
        role = RoleId()
        self.check(function(self.handle, byref(role)))
        return role

    def add_tensor(self) -> RoleId:
        return self._add(self.lib.ftrainPatternAddTensor)

    def add_tensor_list(self) -> RoleId:
        return self._add(self.lib.ftrainPatternAddTensorList)

    def add_grouped_tensor(self) -> RoleId:
        return self._add(self.lib.ftrainPatternAddGroupedTensor)

    def add_gemm(self, a, b, c, d, alpha, beta, kind="Gemm") -> RoleId:
        op = RoleId()
        self.check(getattr(self.lib, f"ftrainPatternAdd{kind}")(self.handle, byref(op), a, b, c, d, alpha, beta))
        return op


class Ops(_Handle):
    _destroy = "ftrainOpsDestroy"

    def __init__(self, pattern: Pattern):
        super().__init__(pattern.lib)
        self.check(self.lib.ftrainOpsCreate(byref(self.handle), pattern.handle))


class Args(_Handle):
    _destroy = "ftrainArgsDestroy"

    def __init__(self, ops: Ops):
        super().__init__(ops.lib)
        self.check(self.lib.ftrainArgsCreate(byref(self.handle), ops.handle))

    def set_tensor(self, role: RoleId, view: StorageView) -> None:
        self.check(self.lib.ftrainArgsSetTensor(self.handle, role, view))

    def set_gemm(self, op: RoleId, compute_type: int = NUMERIC_FP32) -> None:
        self.check(self.lib.ftrainArgsSetGemm(self.handle, op, compute_type))

    def set_grouped_tensor(self, role: RoleId, num_groups: int, data: StorageView, offsets=None, dim_sizes=None,
                           strides=None) -> None:
        """offsets: one StorageView or None; dim_sizes / strides: a sequence of data.num_dims StorageViews or None."""
        def array(views):
            return (StorageView * len(views))(*views) if views is not None else None

        self.check(self.lib.ftrainArgsSetGroupedTensor(self.handle, role, num_groups, data,
                                                       byref(offsets) if offsets is not None else None,
                                                       array(dim_sizes), array(strides)))

    def set_tensor_list(self, role: RoleId, views) -> None:
        array = (StorageView * max(len(views), 1))(*views)
        self.check(self.lib.ftrainArgsSetTensorList(self.handle, role, array if views else None, len(views)))

    def set_grouped_gemm(self, op: RoleId, kind: str = "GroupedABCDGemm", compute_type: int = NUMERIC_FP32) -> None:
        self.check(getattr(self.lib, f"ftrainArgsSet{kind}")(self.handle, op, compute_type))

    def set_grouped_abcd_gemm(self, op: RoleId, compute_type: int = NUMERIC_FP32) -> None:
        self.set_grouped_gemm(op, "GroupedABCDGemm", compute_type)


class Plan(_Handle):
    _destroy = "ftrainPlanDestroy"

    def __init__(self, args: Args):
        super().__init__(args.lib)
        self.check(self.lib.ftrainPlanCreate(byref(self.handle), args.handle))

    @property
    def num_primitives(self) -> int:
        count = c_uint64()
        self.check(self.lib.ftrainPlanGetNumPrimitives(self.handle, byref(count)))
        return int(count.value)

    def primitive_name(self, index: int) -> str:
        name = c_char_p()
        self.check(self.lib.ftrainPlanGetPrimitiveName(self.handle, index, byref(name)))
        return name.value.decode()

    def primitive_names(self) -> list[str]:
        return [self.primitive_name(i) for i in range(self.num_primitives)]

    def workspace_bytes(self, index: int) -> int:
        size = c_uint64()
        self.check(self.lib.ftrainPlanGetPrimitiveRequiredWorkspaceBytes(self.handle, index, byref(size)))
        return int(size.value)

    def index_of(self, name: str) -> int:
        return self.primitive_names().index(name)

    def execute(self, index: int = 0, workspace: int = 0, workspace_bytes: int = 0, stream: int = 0) -> None:
        self.check(self.lib.ftrainPlanExecutePrimitive(self.handle, index, c_void_p(workspace), workspace_bytes,
                                                       c_void_p(stream)))


class GemmBinding:
    """Pattern -> Ops for the plain Gemm graph, plus Args/Plan factories.

    `order` permutes the order in which the six Tensor roles are added to the
    Pattern, to show that matching does not depend on it.
    """

    def __init__(self, order=("a", "b", "c", "alpha", "beta", "d"), lib=lib):
        pattern = Pattern(lib)
        self.roles = {name: pattern.add_tensor() for name in order}
        r = self.roles
        self.gemm = pattern.add_gemm(r["a"], r["b"], r["c"], r["d"], r["alpha"], r["beta"])
        self.ops = Ops(pattern)
        pattern.close()

    def make_args(self, a, b, c, d, alpha: float, beta: float, compute_type: int = NUMERIC_FP32):
        """a, b, c, d: (address, (rows, cols), strides-or-None). Returns (Args, keepalive)."""
        args = Args(self.ops)
        keep = []
        for name, (address, dims, strides) in (("a", a), ("b", b), ("c", c), ("d", d)):
            view, alive = make_view(address, dims, strides)
            keep.append(alive)
            args.set_tensor(self.roles[name], view)
        scalars = (ctypes.c_float * 2)(alpha, beta)
        keep.append(scalars)
        for index, name in enumerate(("alpha", "beta")):
            view, alive = make_view(ctypes.addressof(scalars) + 4 * index, (), host=True)
            keep.append(alive)
            args.set_tensor(self.roles[name], view)
        args.set_gemm(self.gemm, compute_type)
        return args, keep

    def make_plan(self, a, b, c, d, alpha: float = 1.0, beta: float = 0.0) -> Plan:
        """alpha and beta are read during this call; the Args can go afterwards."""
        args, keep = self.make_args(a, b, c, d, alpha, beta)
        plan = Plan(args)
        args.close()
        del keep
        return plan


class GroupedGemmBinding:
    """Pattern -> Ops for one of the grouped GEMM graphs, plus a Plan factory.

    kind "GroupedABCDGemm": a, b, c, d are GroupedTensors; "GroupedBCDGemm": a is a TensorList;
    "GroupedABGemm": c and d are TensorLists.

    A GroupedTensor operand is given as a dict {address, rows, cols[, offsets, row_strides, col_strides]}
    (per-group lists; without offsets / strides the groups are dense row-major matrices stored one after
    another) and reaches the library as int64 host arrays, which it reads while the Plan is made. A
    TensorList operand is given as a list of (address, (rows, cols), strides-or-None), one entry per group.
    """

    LIST_ROLES = {"GroupedABCDGemm": (), "GroupedBCDGemm": ("a",), "GroupedABGemm": ("c", "d")}

    def __init__(self, order=("a", "b", "c", "alpha", "beta", "d"), kind="GroupedABCDGemm", lib=lib):
        pattern = Pattern(lib)
        self.kind = kind
        self.lists = set(self.LIST_ROLES[kind])

        def add(name):
            if name in ("alpha", "beta"):
                return pattern.add_tensor()
            return pattern.add_tensor_list() if name in self.lists else pattern.add_grouped_tensor()

        self.roles = {name: add(name) for name in order}
        r = self.roles
        self.gemm = pattern.add_gemm(r["a"], r["b"], r["c"], r["d"], r["alpha"], r["beta"], kind=kind)
        self.ops = Ops(pattern)
        pattern.close()

    def make_plan(self, a, b, c, d, alpha: float = 1.0, beta: float = 0.0, compute_type: int = NUMERIC_FP32) -> "Plan":
        args = Args(self.ops)
        keep = []

        def vector(values):
            array = (c_int64 * max(len(values), 1))(*values)
            view, alive = make_view(ctypes.addressof(array), (len(values),), numeric_type=NUMERIC_INT64, host=True)
            keep.extend((array, alive))
            return view

        for name, operand in (("a", a), ("b", b), ("c", c), ("d", d)):
            if name in self.lists:
                views = []
                for address, dims, strides in operand:
                    view, alive = make_view(address, dims, strides)
                    keep.append(alive)
                    views.append(view)
                args.set_tensor_list(self.roles[name], views)
                continue
            groups = len(operand["rows"])
            data, alive = make_view(operand["address"], (0, 0), index_type=INDEX_GROUPED_CONTINUOUS)
            keep.append(alive)
            dims = [vector(operand["rows"]), vector(operand["cols"])]
            offsets = vector(operand["offsets"]) if operand.get("offsets") is not None else None
            strides = ([vector(operand["row_strides"]), vector(operand["col_strides"])]
                       if operand.get("row_strides") is not None else None)
            args.set_grouped_tensor(self.roles[name], groups, data, offsets, dims, strides)
        scalars = (ctypes.c_float * 2)(alpha, beta)
        keep.append(scalars)
        for index, name in enumerate(("alpha", "beta")):
            view, alive = make_view(ctypes.addressof(scalars) + 4 * index, (), host=True)
            keep.append(alive)
            args.set_tensor(self.roles[name], view)
        args.set_grouped_gemm(self.gemm, self.kind, compute_type)
        plan = Plan(args)
        args.close()
        del keep
        return plan


def tensor_operand(tensor):
    """(address, dims, strides) of a 2-D torch tensor; strides only when it is not dense row-major."""
    if tensor is None:
        raise ValueError("use null_operand() for an absent matrix")
    dims = tuple(tensor.shape)
    strides = None if tensor.is_contiguous() else tuple(tensor.stride())
    return tensor.data_ptr(), dims, strides


def null_operand(rows: int, cols: int):
    return 0, (rows, cols), None


def gemm_once(a, b, c, d, alpha: float = 1.0, beta: float = 0.0, workspace: int = 0, workspace_bytes: int = 0,
              stream: int = 0, compute_type: int = NUMERIC_FP32, lib=lib) -> None:
    """ftrainGemm on (address, dims, strides) operands."""
    keep = []
    views = []
    for address, dims, strides in (a, b, c, d):
        view, alive = make_view(address, dims, strides)
        keep.append(alive)
        views.append(view)
    scalars = (ctypes.c_float * 2)(alpha, beta)
    for index in range(2):
        view, alive = make_view(ctypes.addressof(scalars) + 4 * index, (), host=True)
        keep.append(alive)
        views.append(view)
    check(lib.ftrainGemm(*views, compute_type, c_void_p(workspace), workspace_bytes, c_void_p(stream)), lib)


# ---- the platform layer's C ABI (include/ftcuda/ftcuda.h): one kernel family, no selection ----

KERNEL_SIMT = 0
KERNEL_TF32X3 = 1
KERNEL_TF32X3_SPLITK = 2
KERNEL_SKINNY = 3
KERNEL_SIMT_SPLITK = 4
KERNEL_TF32X3_ROWS = 5
KERNEL_NAMES = {
    KERNEL_SIMT: "Fp32Gemm",
    KERNEL_TF32X3: "Fp32Gemm3xTf32",
    KERNEL_TF32X3_ROWS: "Fp32Gemm3xTf32FewRows",
    KERNEL_TF32X3_SPLITK: "Fp32Gemm3xTf32SplitK",
    KERNEL_SKINNY: "Fp32GemmSkinny",
    KERNEL_SIMT_SPLITK: "Fp32GemmSplitK",
}


class GemmDesc(Structure):
    """FtcudaGemmDesc."""

    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("c", c_void_p), ("d", c_void_p),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("m", c_uint64), ("n", c_uint64), ("k", c_uint64),
        ("a_row_stride", c_int64), ("a_col_stride", c_int64),
        ("b_row_stride", c_int64), ("b_col_stride", c_int64),
        ("c_row_stride", c_int64), ("c_col_stride", c_int64),
        ("d_row_stride", c_int64), ("d_col_stride", c_int64),
        ("device", ctypes.c_int32),
    ]


class GemmLaunch(Structure):
    """FtcudaGemmLaunch: opaque; must sit at a 64-byte aligned address (see aligned_launch)."""

    _fields_ = [("words", c_uint64 * 160)]


def aligned_launch():
    """(GemmLaunch at a 64-byte boundary, the buffer that owns its memory)."""
    owner = ctypes.create_string_buffer(ctypes.sizeof(GemmLaunch) + 64)
    address = (ctypes.addressof(owner) + 63) & ~63
    return GemmLaunch.from_address(address), owner


def _declare_platform(lib) -> None:
    message = [ctypes.c_char_p, ctypes.c_size_t]
    lib.ftcuda_current_device.argtypes = [POINTER(ctypes.c_int32)] + message
    lib.ftcuda_device_sm_count.argtypes = [ctypes.c_int32, POINTER(ctypes.c_int32)] + message
    lib.ftcuda_gemm_supports.argtypes = [ctypes.c_int, POINTER(GemmDesc)] + message
    lib.ftcuda_gemm_configure.argtypes = [ctypes.c_int, POINTER(GemmDesc), POINTER(GemmLaunch)] + message
    lib.ftcuda_gemm_workspace_bytes.argtypes = [POINTER(GemmLaunch)]
    lib.ftcuda_gemm_workspace_bytes.restype = c_uint64
    lib.ftcuda_gemm_launch.argtypes = [POINTER(GemmLaunch), c_void_p, c_uint64, c_void_p] + message
    lib.ftcuda_gemm_splitk_static.argtypes = [POINTER(GemmDesc), c_void_p] + message
    lib.ftcuda_gemm_launch_scatter.argtypes = [POINTER(GemmLaunch), c_void_p, c_uint64, POINTER(c_void_p), ctypes.c_int32, c_uint64,
                                               c_void_p] + message
    lib.ftcuda_gemm_splitk_static_capacity.argtypes = []
    lib.ftcuda_gemm_splitk_static_capacity.restype = c_uint64
    lib.ftcuda_device_status.argtypes = [ctypes.c_int32, POINTER(ctypes.c_int32)] + message
    lib.ftcuda_device_status_reset.argtypes = [ctypes.c_int32] + message
    lib.ftcuda_selftest_bounded_wait.argtypes = [ctypes.c_int32, c_uint64, c_void_p] + message
    lib.ftcuda_measure_ffma_tflops.argtypes = [ctypes.c_int32, POINTER(ctypes.c_double)] + message
    lib.ftcuda_measure_ffma_tflops.restype = ctypes.c_int
    for name in ("ftcuda_current_device", "ftcuda_device_sm_count", "ftcuda_gemm_supports", "ftcuda_gemm_configure",
                 "ftcuda_gemm_launch", "ftcuda_gemm_splitk_static", "ftcuda_gemm_launch_scatter", "ftcuda_device_status",
                 "ftcuda_device_status_reset", "ftcuda_selftest_bounded_wait"):
        getattr(lib, name).restype = ctypes.c_int


_declare_platform(lib)


def make_desc(a, b, c, d, alpha: float, beta: float, device: int = 0) -> GemmDesc:
    """a, b, c, d: (address, (rows, cols), strides-or-None) as elsewhere in this module."""
    def layout(operand):
        _, dims, strides = operand
        return strides if strides is not None else (dims[1], 1)

    (m, k), (_, n) = a[1], b[1]
    return GemmDesc(a[0], b[0], c[0], d[0], alpha, beta, m, n, k, *layout(a), *layout(b), *layout(c), *layout(d), device)


class PlatformGemm:
    """One kernel family configured for one problem (ftcuda_gemm_configure), launchable many times."""

    def __init__(self, kernel: int, desc: GemmDesc):
        self.kernel = kernel
        self.desc = desc
        self.launch, self._owner = aligned_launch()
        buffer = ctypes.create_string_buffer(256)
        if lib.ftcuda_gemm_configure(kernel, byref(desc), byref(self.launch), buffer, 256) != 0:
            raise FTrainError(STATUS_UNSUPPORTED, buffer.value.decode())
        self.workspace_bytes = int(lib.ftcuda_gemm_workspace_bytes(byref(self.launch)))

    def run(self, workspace: int = 0, workspace_bytes: int = 0, stream: int = 0) -> None:
        buffer = ctypes.create_string_buffer(256)
        if lib.ftcuda_gemm_launch(byref(self.launch), c_void_p(workspace), workspace_bytes, c_void_p(stream), buffer,
                                  256) != 0:
            raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())


    def run_scatter(self, owner_rows, rows_per_owner: int, stream: int = 0, workspace: int = 0, workspace_bytes: int = 0) -> None:
        """ftcuda_gemm_launch_scatter: add alpha * (A B) into the row buffers of the rows' owners
        (device addresses, possibly peer-mapped); tensor-core families only. With a workspace of
        self.workspace_bytes the K slices are combined locally before they travel."""
        pointers = (c_void_p * len(owner_rows))(*[c_void_p(int(pointer)) for pointer in owner_rows])
        buffer = ctypes.create_string_buffer(256)
        if lib.ftcuda_gemm_launch_scatter(byref(self.launch), c_void_p(workspace), workspace_bytes, pointers, len(owner_rows),
                                          rows_per_owner, c_void_p(stream), buffer, 256) != 0:
            raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())


def platform_supports(kernel: int, desc: GemmDesc) -> str | None:
    """None when the kernel family accepts the problem, else its reason."""
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_gemm_supports(kernel, byref(desc), buffer, 256) != 0:
        return buffer.value.decode()
    return None


def splitk_static(desc: GemmDesc, stream: int = 0) -> None:
    """ftcuda_gemm_splitk_static: split-K GEMM on the library's own static scratch; allocates nothing."""
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_gemm_splitk_static(byref(desc), c_void_p(stream), buffer, 256) != 0:
        raise FTrainError(STATUS_UNSUPPORTED, buffer.value.decode())


def splitk_static_capacity() -> int:
    return int(lib.ftcuda_gemm_splitk_static_capacity())


def device_status(device: int = 0) -> int:
    """ftcuda_device_status: the device's status word (0 = no kernel has given up on a wait since it was last cleared)."""
    code = ctypes.c_int32(0)
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_device_status(device, byref(code), buffer, 256) != 0:
        raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())
    return int(code.value)


def device_status_reset(device: int = 0) -> None:
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_device_status_reset(device, buffer, 256) != 0:
        raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())


def selftest_bounded_wait(device: int, budget_ns: int, stream: int = 0) -> None:
    """ftcuda_selftest_bounded_wait: one warp waits `budget_ns` on a barrier nothing arrives on, then sets the status word."""
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_selftest_bounded_wait(device, budget_ns, c_void_p(stream), buffer, 256) != 0:
        raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())


def measure_ffma_tflops(device: int = 0) -> float:
    """ftcuda_measure_ffma_tflops: the device's measured FP32 FFMA rate (register-only probe kernel)."""
    value = ctypes.c_double(0.0)
    buffer = ctypes.create_string_buffer(256)
    if lib.ftcuda_measure_ffma_tflops(device, byref(value), buffer, 256) != 0:
        raise FTrainError(STATUS_INTERNAL_ERROR, buffer.value.decode())
    return float(value.value)
