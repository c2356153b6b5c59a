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
        _check_sharded_checkpoint_load(rank, world, out_dir)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _check_sharded_checkpoint_load(rank: int, world: int, out_dir: str) -> None:
    """A model checkpoint in the reference's dict format, read shard by shard: every rank keeps only its rows
    (column-parallel layers) or its K slice (row-parallel down_proj) and the block still computes what the
    unsharded block computes."""
    import nibble_b200.linear as linear_module
    from nibble_b200 import load_packed_model, replace_linear_layers, save_quantized_model_checkpoint
    from nibble_b200.sharded import ColumnParallelQuantizedLinear, RowParallelQuantizedLinear
    from oracle import w4a16_oracle as oracle
    from test_fusion_host_logic import Block

    def fused(flat, packed, scales, gs):
        return torch.from_numpy(oracle.linear_reference(flat.numpy(), packed.numpy(), scales.numpy(), gs))

    linear_module._run_fused = fused
    linear_module._require_cuda = lambda tensor: None
    torch.manual_seed(11)
    source = Block(hidden=512, kv=128, inter=512).half()
    replace_linear_layers(source, group_size=128)
    path = os.path.join(out_dir, "model.pt")
    if rank == 0:
        save_quantized_model_checkpoint(path, source, group_size=128, source_model="gloo-test")
    dist.barrier()
    plan = {"q_proj": "column", "k_proj": "column", "v_proj": "column", "o_proj": "column", "gate_proj": "column",
            "up_proj": "column", "down_proj": "row"}
    with torch.device("meta"):
        target = Block(hidden=512, kv=128, inter=512).half()
    assert load_packed_model(target, path, device="cpu", plan=plan) == 7
    assert isinstance(target.q_proj, ColumnParallelQuantizedLinear) and isinstance(target.down_proj, RowParallelQuantizedLinear)
    assert target.k_proj.local.packed_weights.shape == (128 // world, 256)       # this rank's rows only
    assert target.down_proj.local.packed_weights.shape == (512, 512 // world // 2)  # this rank's K slice only
    assert torch.equal(target.k_proj.local.packed_weights,
                       source.k_proj.packed_weights[rank * 64:(rank + 1) * 64])
    x = torch.randn((3, 512), generator=torch.Generator().manual_seed(2)).half()
    torch.testing.assert_close(target(x), source(x), rtol=2e-2, atol=2e-2)
    with pytest.raises(ValueError, match="plan values"):
        load_packed_model(target, path, device="cpu", plan={"q_proj": "diagonal"})


def test_column_and_row_parallel_world_size_2(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(name for name in os.listdir(tmp_path) if name.startswith("ok")) == ["ok0", "ok1"]


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
