"""Row- and K-sharded GEMM on real GPUs: one process per GPU (NCCL), results
checked against a float64 product. Needs at least two GPUs; on a one-GPU box the
same classes are exercised with a world of one."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parents[1]


def worker(rank, world, port, failures):
    for entry in (str(REPO), str(REPO / "flash-train_b200" / "python")):
        sys.path.insert(0, entry)
    # No NVLink multicast objects anywhere: NCCL without NVLS, symmetric memory without multicast.
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from flash_train import sharded

    torch.backends.cuda.matmul.allow_tf32 = False
    generator = torch.Generator(device=device).manual_seed(5)  # same seed: every rank builds the same matrices
    m, k, n = 512, 16400, 384
    a = torch.rand(m, k, device=device, generator=generator) * 2 - 1
    b = torch.rand(k, n, device=device, generator=generator) * 2 - 1
    c = torch.rand(m, n, device=device, generator=generator)
    exact = 1.25 * (a.double() @ b.double()) - 0.5 * c.double()

    rows = sharded.RowShardedGemm(m, world, rank)
    d_rows = rows(a[rows.start:rows.stop].contiguous(), b, c[rows.start:rows.stop].contiguous(), 1.25, -0.5)
    torch.cuda.synchronize()
    if not torch.allclose(d_rows.double(), exact[rows.start:rows.stop], rtol=1e-4, atol=2e-2):
        failures.append(f"rank {rank}: row-sharded result is off")

    split = sharded.KShardedGemm(m, n, k)
    d_split = split(a[:, split.k_start:split.k_stop].contiguous(), b[split.k_start:split.k_stop].contiguous(),
                    c[split.row_start:split.row_stop].contiguous(), 1.25, -0.5)
    torch.cuda.synchronize()
    if not torch.allclose(d_split.double(), exact[split.row_start:split.row_stop], rtol=1e-4, atol=2e-2):
        failures.append(f"rank {rank}: K-sharded result is off")
    # The same K-sharded product with the reduction fused into the kernel's epilogue: every rank adds
    # its results into the owners' rows through peer-mapped symmetric memory.
    try:
        for local_combine in (True, False):
          fused = sharded.FusedKShardedGemm(m, n, k, local_combine=local_combine)
          for _ in range(2):  # the second call reuses the symmetric buffer
            d_fused = fused(a[:, fused.k_start:fused.k_stop].contiguous(), b[fused.k_start:fused.k_stop].contiguous(),
                            c[split.row_start:split.row_stop].contiguous(), 1.25, -0.5)
            torch.cuda.synchronize()
            if not torch.allclose(d_fused.double(), exact[split.row_start:split.row_stop], rtol=1e-4, atol=2e-2):
                failures.append(f"rank {rank}: fused K-sharded result is off (local_combine={local_combine})")
    except Exception as error:  # noqa: BLE001 - reported to the parent, the process leaves in order
        failures.append(f"rank {rank}: fused K-sharded GEMM raised {type(error).__name__}: {error}")
    # Host operands, rows split over the ranks, B uploaded once in total: every rank sends its share of
    # B's rows over PCIe and the ranks all-gather the rest over NVLink.
    try:
        import flash_train.torch as ft_torch

        k_host = 8192  # divisible by every world size used here
        host_generator = torch.Generator().manual_seed(9)
        a_host = torch.randn(m, k_host, generator=host_generator)
        b_host = torch.randn(k_host, n, generator=host_generator).pin_memory()
        mine = slice(rows.start, rows.stop)
        pipeline = ft_torch.HostGemm(rows.stop - rows.start, n, k_host, device=device, band_rows=32, group=dist.group.WORLD)
        a_mine = a_host[mine].contiguous().pin_memory()
        for _ in range(2):
            d_host = pipeline(a_mine, b_host)
            torch.cuda.synchronize()
            expected = a_host[mine].double() @ b_host.double()
            if not torch.allclose(d_host.double(), expected, rtol=1e-4, atol=2e-2):
                failures.append(f"rank {rank}: HostGemm with a shared upload of B is off")
    except Exception as error:  # noqa: BLE001
        failures.append(f"rank {rank}: HostGemm with a process group raised {type(error).__name__}: {error}")
    # Integer-valued operands: every product and every partial sum is exact in FP32 (|sum| < 2^24), so the
    # fused form -- up to `world` GPUs adding into one element at the same time -- must reproduce the
    # reduce-scatter form and the float64 product bit for bit. A lost addition cannot hide in rounding.
    try:
        a_int = torch.randint(-2, 3, (m, k), device=device, generator=generator).float()
        b_int = torch.randint(-2, 3, (k, n), device=device, generator=generator).float()
        exact_int = (a_int.double() @ b_int.double())[split.row_start:split.row_stop]
        a_cols = a_int[:, split.k_start:split.k_stop].contiguous()
        b_rows = b_int[split.k_start:split.k_stop].contiguous()
        d_scattered = split(a_cols, b_rows, None, 1.0, 0.0).clone()
        torch.cuda.synchronize()
        if not torch.equal(d_scattered.double(), exact_int):
            failures.append(f"rank {rank}: K-sharded integer product is not exact")
        for local_combine in (True, False):
            fused = sharded.FusedKShardedGemm(m, n, k, local_combine=local_combine)
            for repeat in range(3):
                d_fused = fused(a_cols, b_rows, None, 1.0, 0.0)
                torch.cuda.synchronize()
                if not torch.equal(d_fused, d_scattered):
                    failures.append(f"rank {rank}: fused integer product differs from the reduce-scatter form "
                                    f"(local_combine={local_combine}, call {repeat})")
    except Exception as error:  # noqa: BLE001
        failures.append(f"rank {rank}: integer-valued K-sharded check raised {type(error).__name__}: {error}")
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_gemm_on_all_visible_gpus(native_library):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    import torch.multiprocessing as mp

    world = torch.cuda.device_count()  # every visible GPU (1, 2, 4 or 8 ranks; m = 512 divides)
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(worker, args=(world, port, failures), nprocs=world, join=True)
    assert list(failures) == []
