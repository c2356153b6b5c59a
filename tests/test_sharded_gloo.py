"""World-size-2 CPU ranks (gloo): the column- and row-parallel wrappers assemble the same result as
the unsharded oracle.  Device arithmetic is the CPU oracle (patched in per rank); the slicing, the
collectives and the single final rounding are the shipped code."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nibble_b200.sharded import shard_k, shard_rows


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _patch_device_routines():
    import nibble_b200.sharded as sharded
    from oracle import w4a16_oracle as oracle

    def fused(flat, packed, scales, gs):
        return torch.from_numpy(oracle.linear_reference(flat.numpy(), packed.numpy(), scales.numpy(), gs))

    def partial(flat, packed, scales, gs):
        w = oracle.dequantize_weights(packed.numpy(), scales.numpy(), gs)
        return torch.from_numpy(flat.numpy().astype(np.float32) @ w.T)

    sharded._run_fused = fused
    sharded._run_partial_f32 = partial
    sharded._require_cuda = lambda tensor: None


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        _patch_device_routines()
        from nibble_b200 import quantize_and_pack_weights
        from nibble_b200.sharded import ColumnParallelQuantizedLinear, RowParallelQuantizedLinear
        from oracle import w4a16_oracle as oracle

        g = torch.Generator().manual_seed(0)
        n, k, m = 64, 512, 3
        packed, scales = quantize_and_pack_weights(torch.randn((n, k), generator=g) * 0.02, 128)
        bias = torch.randn((n,), generator=g).half()
        x = torch.randn((2, m, k), generator=g).half()
        want = torch.from_numpy(
            oracle.linear_reference(x.reshape(-1, k).numpy(), packed.numpy(), scales.numpy(), 128)
        ).reshape(2, m, n)

        col = ColumnParallelQuantizedLinear.from_full(packed, scales, 128, bias=bias)
        assert col.local.out_features == n // world
        got = col(x)
        assert got.shape == (2, m, n)
        assert torch.equal(got, want + bias), "column-parallel gather must reproduce the full result"
        ungathered = ColumnParallelQuantizedLinear.from_full(packed, scales, 128, gather_output=False)(x)
        assert torch.equal(ungathered, want[..., rank * n // world:(rank + 1) * n // world])

        row = RowParallelQuantizedLinear.from_full(packed, scales, 128)
        assert row.local.in_features == k // world
        got = row(x)
        exact = oracle.linear_fp64(x.reshape(-1, k).numpy(), packed.numpy(), scales.numpy(), 128).reshape(2, m, n)
        bound = oracle.error_bound(x.reshape(-1, k).numpy(), packed.numpy(), scales.numpy(), 128).reshape(2, m, 1)
        assert (np.abs(got.numpy().astype(np.float64) - exact) <= bound).all()
        torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2)
        pre_split = RowParallelQuantizedLinear.from_full(packed, scales, 128, input_is_parallel=True)
        mine = x[..., rank * k // world:(rank + 1) * k // world]
        assert torch.equal(pre_split(mine), got)
        # every rank holds the identical reduced result
        both = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(both, got)
        assert all(torch.equal(both[0], other) for other in both)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_world_size_2(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_shard_helpers():
    packed = torch.arange(8 * 128, dtype=torch.int64).reshape(8, 128).to(torch.uint8)   # N=8, K=256
    scales = torch.arange(16, dtype=torch.float32).reshape(8, 2).half()
    p1, s1 = shard_rows(packed, scales, 1, 4)
    assert torch.equal(p1, packed[2:4]) and torch.equal(s1, scales[2:4])
    assert p1.is_contiguous() and p1.data_ptr() == packed[2:4].data_ptr()   # a view: no repack
    pk, sk = shard_k(packed, scales, 1, 2, 128)
    assert pk.is_contiguous() and torch.equal(pk, packed[:, 64:]) and torch.equal(sk, scales[:, 1:])
    with pytest.raises(ValueError):
        shard_rows(packed, scales, 0, 3)
    with pytest.raises(ValueError):
        shard_k(packed, scales, 0, 4, 128)
