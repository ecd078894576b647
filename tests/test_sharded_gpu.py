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
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_gemm_on_all_visible_gpus(native_library):
    if not torch.cuda.is_available():
        pytest.fail("the GPU tests need a CUDA device")
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(worker, args=(world, port, failures), nprocs=world, join=True)
    assert list(failures) == []
