"""One large FP32 GEMM over the GPUs of one box, one process per GPU.

The reference is a single-device library: a Plan is bound to the device that
was current when it was created (src/plan.cpp:42-48 there) and the selection
cache is keyed by device (src/include/flash_train/constraints.hpp:30-32). The
two partitionings here sit above the C API and keep that model -- every rank
creates its own Plan on its own device:

  RowShardedGemm   rows of A, C and D are split into `world` contiguous blocks,
                   B is replicated. No communication at all.
  KShardedGemm     columns of A and rows of B are split into `world` K ranges;
                   every rank computes a full m x n partial product (scaled by
                   alpha, which is linear), the partials are summed with one
                   reduce-scatter so that rank r ends up owning rows
                   [r*m/world, (r+1)*m/world) of D, and the owner adds beta * C
                   to its rows exactly once, after the sum.

  FusedKShardedGemm  the same partitioning without the reduce-scatter pass: the
                   tensor-core kernel of every rank ADDS its results straight
                   into the rows' owners' buffers over NVLink (peer-mapped
                   symmetric memory, FP32 atomics), so the reduction is part of
                   the GEMM's epilogue and no m x n partial is ever stored.

Process-group plumbing is torch.distributed (NCCL over NVLink on GPUs). The
local product is a Plan of libflash_train.so executed on torch's current
stream; `local_gemm` can be replaced by another callable with the same
signature, which is how the partitioning logic is tested on CPU ranks.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

K_GRANULE = 32  # K ranges start on multiples of the kernels' K block


def row_range(m: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the rows rank `rank` owns: contiguous blocks, the first m % world one row longer."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    base, extra = divmod(m, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def k_range(k: int, world: int, rank: int, granule: int = K_GRANULE) -> Tuple[int, int]:
    """[start, stop) of the K range of rank `rank`: whole granules, spread as evenly as they go;
    the last range takes the ragged end. Ranges may be empty when K is short."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    granules = -(-k // granule)
    first, _ = row_range(granules, world, rank)
    _, last = row_range(granules, world, rank)
    return min(first * granule, k), min(last * granule, k)


class _LibraryGemm:
    """d = alpha * a @ b + beta * c through one reusable Plan per (addresses, scalars)."""

    def __init__(self):
        from . import capi

        self._capi = capi
        self._binding = capi.GemmBinding()
        self._plans = {}

    def __call__(self, a, b, c, d, alpha: float, beta: float) -> None:
        import torch

        capi = self._capi
        key = (a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else 0, d.data_ptr(), tuple(a.shape),
               tuple(b.shape), tuple(a.stride()), tuple(b.stride()), float(alpha), float(beta), a.device.index)
        entry = self._plans.get(key)
        if entry is None:
            rows, cols = d.shape
            plan = self._binding.make_plan(
                capi.tensor_operand(a), capi.tensor_operand(b),
                capi.tensor_operand(c) if c is not None else capi.null_operand(rows, cols),
                capi.tensor_operand(d), alpha, beta)
            size = plan.workspace_bytes(0)
            workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=a.device)
            entry = (plan, workspace, size)
            self._plans[key] = entry
        plan, workspace, size = entry
        plan.execute(0, workspace.data_ptr() if size else 0, size, torch.cuda.current_stream(a.device).cuda_stream)


LocalGemm = Callable[..., None]


class RowShardedGemm:
    """D[rows of this rank] = alpha * A[rows of this rank] @ B + beta * C[rows of this rank]."""

    def __init__(self, m: int, world: int, rank: int, local_gemm: Optional[LocalGemm] = None):
        self.start, self.stop = row_range(m, world, rank)
        self.local_gemm = local_gemm if local_gemm is not None else _LibraryGemm()

    def __call__(self, a_rows, b, c_rows=None, alpha: float = 1.0, beta: float = 0.0, out=None):
        import torch

        rows = self.stop - self.start
        if a_rows.shape[0] != rows:
            raise ValueError(f"this rank owns {rows} rows of A, got {a_rows.shape[0]}")
        if out is None:
            out = torch.empty(rows, b.shape[1], dtype=a_rows.dtype, device=a_rows.device)
        if rows:
            self.local_gemm(a_rows, b, c_rows, out, alpha, beta)
        return out


class KShardedGemm:
    """A[:, K range of this rank] @ B[K range of this rank, :] summed over ranks by reduce-scatter.

    Returns this rank's rows of D. m must be divisible by the world size (the
    reduce-scatter hands out equal row blocks).
    """

    def __init__(self, m: int, n: int, k: int, group=None, local_gemm: Optional[LocalGemm] = None):
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if m % self.world != 0:
            raise ValueError(f"m = {m} is not divisible by {self.world} ranks")
        self.m, self.n, self.k = m, n, k
        self.k_start, self.k_stop = k_range(k, self.world, self.rank)
        self.row_start, self.row_stop = row_range(m, self.world, self.rank)
        self.local_gemm = local_gemm if local_gemm is not None else _LibraryGemm()
        self._partial = None

    def __call__(self, a_cols, b_rows, c_rows=None, alpha: float = 1.0, beta: float = 0.0, out=None):
        import torch
        import torch.distributed as dist

        depth = self.k_stop - self.k_start
        if a_cols.shape != (self.m, depth) or b_rows.shape != (depth, self.n):
            raise ValueError(f"this rank owns K range [{self.k_start}, {self.k_stop}): expected A {self.m}x{depth} "
                             f"and B {depth}x{self.n}")
        if self._partial is None or self._partial.device != a_cols.device:
            self._partial = torch.empty(self.m, self.n, dtype=a_cols.dtype, device=a_cols.device)
        partial = self._partial
        # alpha is linear, so it is applied to the partials; beta * C must enter the
        # sum once, which the owner of the rows does after the reduction.
        self.local_gemm(a_cols, b_rows, None, partial, alpha, 0.0)
        rows = self.row_stop - self.row_start
        if out is None:
            out = torch.empty(rows, self.n, dtype=partial.dtype, device=partial.device)
        if self.world == 1:
            out.copy_(partial)
        elif dist.get_backend(self.group) == "gloo":
            # gloo has no reduce-scatter: sum everywhere, keep the own rows.
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            out.copy_(partial[self.row_start:self.row_stop])
        else:
            dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=self.group)
        if c_rows is not None and beta != 0.0:
            out.add_(c_rows, alpha=beta)
        return out


class FusedKShardedGemm:
    """K-sharded GEMM whose reduction across ranks happens inside the kernel's epilogue.

    Every rank owns rows [rank * m / world, (rank + 1) * m / world) of D in a buffer of symmetric
    memory (torch.distributed._symmetric_memory), so that every rank holds a peer-mapped address of
    every other rank's rows. A call: the owner writes beta * C (or zeros) into its rows; a barrier;
    every rank launches the tensor-core kernel on its K range through ftcuda_gemm_launch_scatter,
    whose epilogue adds alpha * (A_r B_r) into the owners' rows with FP32 atomics over NVLink; a
    barrier; the rows are complete. No reduce-scatter. When the local kernel splits K (to even out its
    waves) the slices are, by default, first summed on this GPU (a workspace, the library's reduction
    kernel adding into the owners' rows), so that every element crosses NVLink once; with
    local_combine=False every slice adds directly and nothing is stored at all. The order of the
    additions is not fixed: results agree with the reduce-scatter form to rounding, not bitwise.

    Operands must suit the tensor-core kernels (16-byte aligned bases and pitches).
    """

    def __init__(self, m: int, n: int, k: int, group=None, device=None, local_combine: bool = True):
        """local_combine: give the local split-K a workspace so that its K slices are summed on this GPU
        and every element crosses NVLink once; False: no workspace, every slice adds directly."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric_memory

        from . import capi

        self._capi = capi
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if m % self.world != 0:
            raise ValueError(f"m = {m} is not divisible by {self.world} ranks")
        if self.world > 8:
            raise ValueError("at most 8 owners")
        self.m, self.n, self.k = m, n, k
        self.rows = m // self.world
        self.k_start, self.k_stop = k_range(k, self.world, self.rank)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.out = symmetric_memory.empty((self.rows, n), dtype=torch.float32, device=self.device)
        self._handle = symmetric_memory.rendezvous(self.out, self.group)
        self._owner_rows = [int(self._handle.buffer_ptrs[r]) for r in range(self.world)]
        self._launches = {}
        self._local_combine = local_combine
        self._workspace = None

    def _launch_for(self, a_cols, b_rows, alpha: float):
        capi = self._capi
        key = (a_cols.data_ptr(), b_rows.data_ptr(), tuple(a_cols.stride()), tuple(b_rows.stride()), float(alpha))
        launch = self._launches.get(key)
        if launch is None:
            operand = lambda t: (t.data_ptr(), tuple(t.shape), None if t.is_contiguous() else tuple(t.stride()))  # noqa: E731
            # The descriptor's output is not written in scatter mode; it only carries the shape.
            desc = capi.make_desc(operand(a_cols), operand(b_rows), (0, (self.m, self.n), None),
                                  (self.out.data_ptr(), (self.m, self.n), None), alpha, 0.0, self.device.index or 0)
            kernel = capi.KERNEL_TF32X3_SPLITK if capi.platform_supports(capi.KERNEL_TF32X3_SPLITK, desc) is None \
                else capi.KERNEL_TF32X3
            launch = capi.PlatformGemm(kernel, desc)
            self._launches[key] = launch
        return launch

    def __call__(self, a_cols, b_rows, c_rows=None, alpha: float = 1.0, beta: float = 0.0):
        """Returns this rank's rows of D (the symmetric buffer itself: copy it before the next call)."""
        import torch

        depth = self.k_stop - self.k_start
        if a_cols.shape != (self.m, depth) or b_rows.shape != (depth, self.n):
            raise ValueError(f"this rank owns K range [{self.k_start}, {self.k_stop}): expected A {self.m}x{depth} "
                             f"and B {depth}x{self.n}")
        if c_rows is not None and beta != 0.0:
            torch.mul(c_rows, beta, out=self.out)
        else:
            self.out.zero_()
        self._handle.barrier()  # every owner's rows are initialised before anybody adds to them
        if depth > 0:
            launch = self._launch_for(a_cols, b_rows, alpha)
            workspace, size = 0, 0
            if self._local_combine and launch.workspace_bytes > 0:
                if self._workspace is None or self._workspace.numel() < launch.workspace_bytes:
                    self._workspace = torch.empty(launch.workspace_bytes, dtype=torch.uint8, device=self.device)
                workspace, size = self._workspace.data_ptr(), launch.workspace_bytes
            launch.run_scatter(self._owner_rows, self.rows, torch.cuda.current_stream(self.device).cuda_stream, workspace, size)
        self._handle.barrier()  # every rank's additions have been issued and are complete
        return self.out
