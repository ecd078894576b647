"""GEMM on operands that live in (pinned) host memory, result back in host memory.

`flash_train.torch.gemm` wants device tensors. When A, B, C sit on the host,
copying everything in, multiplying, and copying D out runs the three phases one
after the other, and the PCIe copies dominate. `HostGemm` overlaps them: B goes
to the device once per call, then A (and C) travel in bands of rows while the
previous band is multiplied and the one before that is copied back. Three
streams (copy-in, the caller's current stream for the kernels, copy-out), two
device buffers per banded operand, events in between. Every band is one
ordinary `flash_train.torch.gemm` call, so kernel selection, the selection
cache and the numerics are those of the library.

Several GPUs multiplying their own rows of A by the SAME B (the row-sharded GEMM): given a process
group, every rank uploads only its 1/world share of B's rows and the ranks exchange the shares over
NVLink with one all-gather (NCCL), so that B crosses each GPU's PCIe link once in total instead of once
per GPU.

The reference has no counterpart: its binding takes device tensors only
(python/flash_train/torch/csrc/flash_train_torch.cpp:34-75 there).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

DEFAULT_BAND_ROWS = 2048


def band_ranges(m: int, band_rows: int) -> List[Tuple[int, int]]:
    """[start, stop) row ranges of the bands: full bands, then the ragged end."""
    if band_rows <= 0:
        raise ValueError("band_rows must be positive")
    return [(start, min(start + band_rows, m)) for start in range(0, m, band_rows)]


def _check_host_matrix(tensor: torch.Tensor, name: str) -> None:
    if tensor.is_cuda:
        raise RuntimeError(f"{name} must be a host tensor")
    if tensor.dtype != torch.float32:
        raise RuntimeError(f"{name} must be FP32")
    if tensor.dim() != 2:
        raise RuntimeError(f"{name} must be rank two")
    if not tensor.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


class HostGemm:
    """Reusable pipeline for one (m, n, k) shape on one device.

    The device buffers (B, two bands of A, two of D, two of C when used) and the
    streams are made once; `__call__` may be repeated with other host tensors of
    the same shape. Host tensors should be pinned -- pageable memory still works
    but its copies do not overlap.
    """

    def __init__(self, m: int, n: int, k: int, device=None, band_rows: int = DEFAULT_BAND_ROWS, with_c: bool = False,
                 group=None):
        """group: a torch.distributed process group whose ranks all call with the same host matrix B (each
        with its own rows of A): every rank then uploads rows [rank * k / world, (rank + 1) * k / world)
        of B only and receives the others' rows by an all-gather over NVLink. k must divide evenly."""
        from . import gemm as device_gemm

        self._gemm = device_gemm
        self._group, self._world, self._rank = None, 1, 0
        if group is not None:
            import torch.distributed as dist

            world = dist.get_world_size(group)
            if world > 1 and k % world == 0:
                self._group, self._world, self._rank = group, world, dist.get_rank(group)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.bands = band_ranges(m, band_rows)
        rows = min(band_rows, m) if m else 0
        with torch.cuda.device(self.device):
            self._b = torch.empty(k, n, dtype=torch.float32, device=self.device)
            self._a = [torch.empty(rows, k, dtype=torch.float32, device=self.device) for _ in range(2)]
            self._c = [torch.empty(rows, n, dtype=torch.float32, device=self.device) for _ in range(2)] if with_c else None
            self._copy_in = torch.cuda.Stream(self.device)
            self._copy_out = torch.cuda.Stream(self.device)

    def join(self) -> None:
        """Makes the caller's current stream wait for the copy-outs of earlier calls (what a call does by itself
        unless it was made with overlap_calls=True). Does not block the host."""
        with torch.cuda.device(self.device):
            torch.cuda.current_stream(self.device).wait_stream(self._copy_out)

    def synchronize(self) -> None:
        """Blocks until every copy and kernel of earlier calls has finished (all three streams)."""
        with torch.cuda.device(self.device):
            torch.cuda.current_stream(self.device).synchronize()
            self._copy_in.synchronize()
            self._copy_out.synchronize()

    def __call__(self, a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
                 beta: float = 0.0, out: Optional[torch.Tensor] = None, overlap_calls: bool = False) -> torch.Tensor:
        """overlap_calls=False: when the call returns, the caller's current stream waits for the last copy-out,
        so one synchronize on it is enough before reading `out`. overlap_calls=True: consecutive calls pipeline
        -- the next call's copy-in starts as soon as this call's kernels have read the device buffers, while
        this call's results are still leaving --; the caller's stream does NOT wait for the copy-out then:
        call synchronize() (or synchronise the device) before reading `out`, and give calls whose results are
        still in flight different `out` buffers or accept that they are written in call order."""
        _check_host_matrix(a, "a")
        _check_host_matrix(b, "b")
        if tuple(a.shape) != (self.m, self.k) or tuple(b.shape) != (self.k, self.n):
            raise RuntimeError(f"this pipeline was made for A {self.m}x{self.k} and B {self.k}x{self.n}")
        if c is not None:
            _check_host_matrix(c, "c")
            if tuple(c.shape) != (self.m, self.n):
                raise RuntimeError("c must have the shape of the result")
            if self._c is None:
                raise RuntimeError("this pipeline was made without buffers for c (with_c=False)")
        if out is None:
            out = torch.empty(self.m, self.n, dtype=torch.float32).pin_memory()
        else:
            _check_host_matrix(out, "out")
            if tuple(out.shape) != (self.m, self.n):
                raise RuntimeError("out must have the shape of the result")
        if self.m == 0 or self.n == 0:
            return out

        with torch.cuda.device(self.device):
            compute = torch.cuda.current_stream(self.device)
            copy_in, copy_out = self._copy_in, self._copy_out
            # Buffers of an earlier call (or whatever the caller queued) come first. The device buffers are
            # read by kernels on the compute stream only; the products leave through blocks of their own.
            copy_in.wait_stream(compute)
            if not overlap_calls:
                copy_in.wait_stream(copy_out)
            with torch.cuda.stream(copy_in):
                if self._group is None:
                    self._b.copy_(b, non_blocking=True)
                else:
                    import torch.distributed as dist

                    share = self.k // self._world
                    mine = slice(self._rank * share, (self._rank + 1) * share)
                    self._b[mine].copy_(b[mine], non_blocking=True)
                    # In place: the share already lies where the gathered matrix wants it.
                    dist.all_gather_into_tensor(self._b, self._b[mine], group=self._group)
            band_used = [None, None]  # event: kernels of the band that last used buffer pair i are done
            for index, (start, stop) in enumerate(self.bands):
                pair, rows = index % 2, stop - start
                with torch.cuda.stream(copy_in):
                    if band_used[pair] is not None:
                        copy_in.wait_event(band_used[pair])
                    a_band = self._a[pair][:rows]
                    a_band.copy_(a[start:stop], non_blocking=True)
                    c_band = None
                    if c is not None:
                        c_band = self._c[pair][:rows]
                        c_band.copy_(c[start:stop], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(copy_in)
                compute.wait_event(arrived)
                product = self._gemm(a_band, self._b, c_band, alpha=alpha, beta=beta)
                done = torch.cuda.Event()
                done.record(compute)
                band_used[pair] = done
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(done)
                    out[start:stop].copy_(product, non_blocking=True)
                    # `product` came from the allocator on the compute stream: tell it the
                    # copy-out stream still reads the block.
                    product.record_stream(copy_out)
            # The caller's stream sees the finished result: one synchronize on it is enough.
            if not overlap_calls:
                compute.wait_stream(copy_out)
        return out


def gemm_host(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
              beta: float = 0.0, out: Optional[torch.Tensor] = None, band_rows: int = DEFAULT_BAND_ROWS) -> torch.Tensor:
    """One-shot form of HostGemm: buffers are made for this call."""
    _check_host_matrix(a, "a")
    _check_host_matrix(b, "b")
    if a.shape[1] != b.shape[0]:
        raise RuntimeError("a's reduction depth must equal b's rows")
    pipeline = HostGemm(a.shape[0], b.shape[1], a.shape[1], band_rows=band_rows, with_c=c is not None)
    return pipeline(a, b, c, alpha=alpha, beta=beta, out=out)
