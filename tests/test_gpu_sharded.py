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
        # the same two cuts with the exchange done by the kernels themselves (peer stores + flags); calls follow
        # each other without any barrier between them: the two result buffers and the release flags keep a
        # fast rank from overwriting what a slow rank still reads
        from nibble_b200.sharded import (PeerColumnParallelQuantizedLinear, PeerRowParallelQuantizedLinear, shard_k,
                                         shard_rows)

        p_rows, s_rows = shard_rows(packed.cuda(), scales.cuda(), rank, world)
        p_k, s_k = shard_k(packed.cuda(), scales.cuda(), rank, world, 128)
        peer_col = PeerColumnParallelQuantizedLinear(p_rows, s_rows, 128, max_rows=8)
        peer_row = PeerRowParallelQuantizedLinear(p_k, s_k, 128, max_rows=8)
        results = []
        for repeat in range(4):          # publication numbers advance; buffers and flags are reused
            for m in (1, 8, 3):
                x = torch.randn((m, k), generator=g).half()
                x_mine = x[:, rank * k // world:(rank + 1) * k // world].contiguous()
                if rank == 1 and repeat == 1:
                    torch.cuda._sleep(20_000_000)      # a slow rank: the other one runs ahead as far as the protocol lets it
                results.append((x, peer_col(x.cuda()), peer_row(x_mine.cuda())))
        torch.cuda.synchronize()
        for x, got_col, got_row in results:
            exact = oracle.linear_fp64(x.numpy(), packed.numpy(), scales.numpy(), 128)
            bound = oracle.error_bound(x.numpy(), packed.numpy(), scales.numpy(), 128)
            for name, got in (("peer column", got_col), ("peer row", got_row)):
                got = got.float().cpu().numpy().astype(np.float64)
                assert got.shape == exact.shape and (np.abs(got - exact) <= bound).all(), name
        peer_col.region.check()
        peer_row.region.check()

        # a chain: column-parallel -> column-parallel reading the first one's result in its own prologue ->
        # row-parallel reading a column slice -> sum; twelve steps back to back
        g2 = torch.Generator().manual_seed(5)
        w_a = quantize_and_pack_weights(torch.randn((512, 1024), generator=g2) * 0.05, 128)
        w_b = quantize_and_pack_weights(torch.randn((1024, 512), generator=g2) * 0.05, 128)
        w_c = quantize_and_pack_weights(torch.randn((256, 1024), generator=g2) * 0.05, 128)
        col_a = PeerColumnParallelQuantizedLinear(*shard_rows(w_a[0].cuda(), w_a[1].cuda(), rank, world), 128, max_rows=8)
        col_b = PeerColumnParallelQuantizedLinear(*shard_rows(w_b[0].cuda(), w_b[1].cuda(), rank, world), 128, max_rows=8)
        row_c = PeerRowParallelQuantizedLinear(*shard_k(w_c[0].cuda(), w_c[1].cuda(), rank, world, 128), 128, max_rows=8)
        k_local = 1024 // world
        chained = []
        for step in range(12):
            m = (1, 8, 4)[step % 3]
            x = torch.randn((m, 1024), generator=g2).half()
            view_b = col_b.launch(col_a.launch(x.cuda()))
            row_c.launch(view_b.narrow(rank * k_local, k_local))
            chained.append((x, row_c.finish(m)))
        torch.cuda.synchronize()
        for x, got in chained:
            a = oracle.linear_reference(x.numpy(), w_a[0].numpy(), w_a[1].numpy(), 128)
            b = oracle.linear_reference(a, w_b[0].numpy(), w_b[1].numpy(), 128)
            c = oracle.linear_reference(b, w_c[0].numpy(), w_c[1].numpy(), 128)
            torch.testing.assert_close(got.cpu(), torch.from_numpy(c), rtol=3e-2, atol=3e-2)
        for layer in (col_a, col_b, row_c):
            layer.region.check()
        # a model checkpoint in the reference's dict format, read shard by shard straight onto this rank's GPU
        from nibble_b200 import load_packed_model, replace_linear_layers, save_quantized_model_checkpoint
        from nibble_b200.linear import QuantizedLinear
        from test_fusion_host_logic import Block

        torch.manual_seed(11)
        source = Block(hidden=512, kv=128, inter=512).half()
        replace_linear_layers(source, group_size=128)
        path = os.path.join(out_dir, "model.pt")
        if rank == 0:
            save_quantized_model_checkpoint(path, source, group_size=128, source_model="two-gpu-test")
        dist.barrier()
        plan = {"q_proj": "column", "k_proj": "column", "v_proj": "column", "o_proj": "column", "gate_proj": "column",
                "up_proj": "column", "down_proj": "row"}
        xb = torch.randn((3, 512), generator=torch.Generator().manual_seed(2)).half().cuda()
        want = source.cuda()(xb)
        for exchange in ("nccl", "peer"):
            with torch.device("meta"):
                target = Block(hidden=512, kv=128, inter=512).half()
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            assert load_packed_model(target, path, device=f"cuda:{rank}", plan=plan, exchange=exchange) == 7
            shard = target.k_proj.local.packed_weights
            assert shard.is_cuda and shard.shape == (128 // world, 256)
            assert torch.equal(shard, source.k_proj.packed_weights[rank * 64:(rank + 1) * 64])
            torch.testing.assert_close(target(xb), want, rtol=3e-2, atol=3e-2)
            torch.testing.assert_close(target(xb), want, rtol=3e-2, atol=3e-2)
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
    assert sorted(name for name in os.listdir(tmp_path) if name.startswith("ok")) == ["ok0", "ok1"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_devices():
    """A model split over two GPUs by one process: the shared-memory opt-in and the occupancy of every kernel variant
    are per device, so the second device must work as the first does (streaming kernel, prefill kernel, decode kernels,
    the allocation-free entry point)."""
    import ctypes

    from capi_helpers import check_against_oracle
    from nibble_b200 import _native, linear_cuda, quantize_and_pack_weights

    g = torch.Generator().manual_seed(0)
    packed, scales = quantize_and_pack_weights(torch.randn((320, 4096), generator=g) * 0.02, 128)
    for m in (1, 8, 96):
        x = torch.randn((m, 4096), generator=g).half()
        outs = []
        for device in ("cuda:1", "cuda:0", "cuda:1"):
            with torch.cuda.device(device):
                y = linear_cuda(x.to(device), packed.to(device), scales.to(device), 128)
                torch.cuda.synchronize()
            check_against_oracle(y, x, packed, scales, fp16_weights=m >= 65)
            outs.append(y.cpu())
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    lib = _native.core()
    for device in ("cuda:1", "cuda:0"):
        with torch.cuda.device(device):
            x = torch.randn((1, 8192), generator=g).half().to(device)
            p = torch.randint(0, 256, (1024, 4096), dtype=torch.uint8, device=device)
            s = (torch.rand((1024, 64), device=device) * 0.002 + 0.001).half()
            y = torch.full((1, 1024), float("nan"), dtype=torch.float16, device=device)
            status = lib.w4a16_linear_f16_static_scratch(x.data_ptr(), p.data_ptr(), s.data_ptr(), y.data_ptr(), 1, 1024, 8192, 128, 0,
                                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            assert status == 0 and not torch.isnan(y).any()
            assert torch.equal(y, linear_cuda(x, p, s, 128))
