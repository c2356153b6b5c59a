"""-m gpu, needs two GPUs: column- and row-parallel layers over NCCL, one process per GPU.

Each rank checks its assembled output against the CPU oracle of the unsharded layer.  Skipped on a
single-GPU machine (the CPU-rank version of the same logic is tests/test_sharded_gloo.py).
"""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nibble_b200 import quantize_and_pack_weights
        from nibble_b200.sharded import ColumnParallelQuantizedLinear, RowParallelQuantizedLinear
        from oracle import w4a16_oracle as oracle

        g = torch.Generator().manual_seed(0)
        n, k = 512, 2048
        packed, scales = quantize_and_pack_weights(torch.randn((n, k), generator=g) * 0.02, 128)
        for m in (1, 8):
            x = torch.randn((m, k), generator=g).half()
            exact = oracle.linear_fp64(x.numpy(), packed.numpy(), scales.numpy(), 128)
            bound = oracle.error_bound(x.numpy(), packed.numpy(), scales.numpy(), 128)
            col = ColumnParallelQuantizedLinear.from_full(packed.cuda(), scales.cuda(), 128)
            row = RowParallelQuantizedLinear.from_full(packed.cuda(), scales.cuda(), 128)
            for layer in (col, row):
                got = layer(x.cuda()).cpu().numpy().astype(np.float64)
                assert got.shape == (m, n)
                assert (np.abs(got - exact) <= bound).all(), type(layer).__name__
        # the same two cuts with the exchange done by the kernel epilogue (peer stores + flags)
        from nibble_b200.sharded import (PeerColumnParallelQuantizedLinear, PeerRowParallelQuantizedLinear, shard_k,
                                         shard_rows)

        p_rows, s_rows = shard_rows(packed.cuda(), scales.cuda(), rank, world)
        p_k, s_k = shard_k(packed.cuda(), scales.cuda(), rank, world, 128)
        peer_col = PeerColumnParallelQuantizedLinear(p_rows, s_rows, 128, max_rows=8)
        peer_row = PeerRowParallelQuantizedLinear(p_k, s_k, 128, max_rows=8)
        for repeat in range(3):          # epochs advance; buffers and flags are reused
            for m in (1, 8, 3):
                x = torch.randn((m, k), generator=g).half()
                exact = oracle.linear_fp64(x.numpy(), packed.numpy(), scales.numpy(), 128)
                bound = oracle.error_bound(x.numpy(), packed.numpy(), scales.numpy(), 128)
                got = peer_col(x.cuda()).float().cpu().numpy().astype(np.float64)
                assert got.shape == (m, n) and (np.abs(got - exact) <= bound).all(), ("peer column", repeat, m)
                x_mine = x[:, rank * k // world:(rank + 1) * k // world].contiguous()
                got = peer_row(x_mine.cuda()).float().cpu().numpy().astype(np.float64)
                assert got.shape == (m, n) and (np.abs(got - exact) <= bound).all(), ("peer row", repeat, m)
                dist.barrier()           # nobody overwrites a buffer a slower rank is still reading
        peer_col.region.check()
        peer_row.region.check()
        torch.cuda.synchronize()
        dist.barrier()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_and_row_parallel_over_nccl(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
