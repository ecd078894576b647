"""The multi-GPU partitioning logic on CPU ranks: two gloo processes, with the
CPU oracle standing in for the device GEMM (the partition arithmetic, the
placement of alpha and beta, and the reduction are what is tested here)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parents[1]


def oracle_local_gemm(a, b, c, d, alpha, beta):
    from oracle import oracle

    if a.shape[1] == 0:
        result = np.zeros(tuple(d.shape), np.float32)
        if c is not None:
            result += beta * c.numpy()
    else:
        result = oracle.host_gemm(a.contiguous().numpy(), b.contiguous().numpy(),
                                  c.contiguous().numpy() if c is not None else None, alpha, beta)
    d.copy_(torch.from_numpy(result))


def worker(rank, world, port, results):
    for entry in (str(REPO), str(REPO / "flash-train_b200" / "python")):
        sys.path.insert(0, entry)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flash_train import sharded

    generator = torch.Generator().manual_seed(9)
    m, k, n = 6, 70, 5  # K is not a multiple of the granule: ranges 64 and 6
    a = torch.randn(m, k, generator=generator)
    b = torch.randn(k, n, generator=generator)
    c = torch.randn(m, n, generator=generator)

    rows = sharded.RowShardedGemm(m, world, rank, local_gemm=oracle_local_gemm)
    d_rows = rows(a[rows.start:rows.stop], b, c[rows.start:rows.stop], alpha=1.5, beta=-0.5)

    split = sharded.KShardedGemm(m, n, k, local_gemm=oracle_local_gemm)
    d_split = split(a[:, split.k_start:split.k_stop].contiguous(), b[split.k_start:split.k_stop].contiguous(),
                    c[split.row_start:split.row_stop], alpha=1.5, beta=-0.5)
    results[rank] = (rows.start, d_rows.numpy(), split.row_start, d_split.numpy(), (split.k_start, split.k_stop))
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def test_partition_arithmetic():
    sys.path.insert(0, str(REPO / "flash-train_b200" / "python"))
    from flash_train import sharded

    assert [sharded.row_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [sharded.row_range(16384, 8, r) for r in (0, 7)] == [(0, 2048), (14336, 16384)]
    ranges = [sharded.k_range(262144, 8, r) for r in range(8)]
    assert ranges[0] == (0, 32768) and ranges[-1] == (229376, 262144)
    assert all(start % 32 == 0 for start, _ in ranges)
    assert [sharded.k_range(70, 2, r) for r in range(2)] == [(0, 64), (64, 70)]
    assert [sharded.k_range(20, 4, r) for r in range(4)] == [(0, 20), (20, 20), (20, 20), (20, 20)]
    with pytest.raises(ValueError):
        sharded.row_range(4, 2, 2)


def test_two_ranks_match_the_unsplit_product(oracle):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
    generator = torch.Generator().manual_seed(9)
    a = torch.randn(6, 70, generator=generator).numpy()
    b = torch.randn(70, 5, generator=generator).numpy()
    c = torch.randn(6, 5, generator=generator).numpy()
    expected = oracle.host_gemm(a, b, c, 1.5, -0.5)
    d_rows = np.zeros_like(expected)
    d_split = np.zeros_like(expected)
    for rank in range(world):
        row_start, rows, split_start, split_rows, k_span = results[rank]
        d_rows[row_start:row_start + rows.shape[0]] = rows
        d_split[split_start:split_start + split_rows.shape[0]] = split_rows
    assert results[0][4] == (0, 64) and results[1][4] == (64, 70)
    # Row split: every row is computed exactly as in the unsplit product.
    assert np.array_equal(d_rows, expected)
    # K split: another summation order, and beta * C added exactly once.
    assert np.allclose(d_split, expected, rtol=1e-5, atol=1e-5)
