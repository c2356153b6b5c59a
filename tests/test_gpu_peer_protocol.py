"""-m gpu, one GPU: the tensor-parallel exchange protocol of the fused kernels (include/w4a16_b200.h,
w4a16_peer_target / w4a16_peer_source) with all ranks of a sharded layer emulated in one process.

The ranks' kernels run one after the other on one stream (``LocalRanks``): every rank's senders are launched
before any rank's readers, so no kernel ever waits for a kernel that has not run.  What is covered: tagged
elements, the two result buffers alternating by publication number, readers inside the consuming linear (re-reading
what has not arrived, parity offset, release), the reader kernels (``materialize``, ``finish``), column slices as inputs, and -- with a rank that never
launches -- every bounded wait running out: the call returns, the status word names the missing rank, and the
GPU goes on working.  Nothing here hangs, traps or faults by design.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from capi_helpers import capi_linear, check_against_oracle
from nibble_b200 import quantize_and_pack_weights
from nibble_b200.sharded import (LocalRanks, PeerColumnParallelQuantizedLinear, PeerRowParallelQuantizedLinear, shard_k,
                                 shard_rows)

pytestmark = pytest.mark.gpu


def _layer(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    packed, scales = quantize_and_pack_weights(torch.randn((n, k), generator=g) * 0.05, 128)
    return packed.cuda(), scales.cuda()


def _result(region, epoch, rows, ld):
    """The FP16 result of publication `epoch` as a [rows, ld] tensor, decoded from the tagged elements of the
    result buffer it went to (value in the low half of each 32-bit word, tag 0x8000 | epoch in the high half)."""
    start = (epoch & 1) * region.result_bytes
    words = region.buffer[start:start + rows * ld * 4].view(torch.int32).view(rows, ld)
    assert bool((((words >> 16) & 0xFFFF) == (0x8000 | (epoch & 0x7FFF))).all()), "an element carries the wrong tag"
    return (words & 0xFFFF).to(torch.int16).view(torch.float16)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_chain_of_sharded_layers_over_six_publications(world):
    ranks = LocalRanks(world)
    k0, n_a, n_b, n_c = 1024, 512, 1024, 256
    w_a, w_b, w_c = _layer(n_a, k0, 1), _layer(n_b, n_a, 2), _layer(n_c, n_b, 3)
    col_a = [PeerColumnParallelQuantizedLinear(*shard_rows(*w_a, r, world), local=ranks, rank=r, name="a") for r in range(world)]
    col_b = [PeerColumnParallelQuantizedLinear(*shard_rows(*w_b, r, world), local=ranks, rank=r, name="b") for r in range(world)]
    row_c = [PeerRowParallelQuantizedLinear(*shard_k(*w_c, r, world, 128), local=ranks, rank=r, name="c") for r in range(world)]
    k_local = n_b // world
    g = torch.Generator().manual_seed(0)
    for step, m in enumerate([1, 8, 3, 1, 5, 8]):
        epoch = step + 1
        x = torch.randn((m, k0), generator=g).half().cuda()
        views_a = [layer.launch(x) for layer in col_a]                       # senders of A on every rank
        views_b = [layer.launch(view) for layer, view in zip(col_b, views_a)]  # readers of A, senders of B
        for r, (layer, view) in enumerate(zip(row_c, views_b)):                # readers of a column slice of B
            layer.launch(view.narrow(r * k_local, k_local))
        outs = [layer.finish(m) for layer in row_c]                           # readers of C's partials
        torch.cuda.synchronize()
        a = [_result(layer.region, epoch, m, n_a).clone() for layer in col_a]
        b = [_result(layer.region, epoch, m, n_b).clone() for layer in col_b]
        for r in range(1, world):
            assert torch.equal(a[r], a[0]) and torch.equal(b[r], b[0]) and torch.equal(outs[r], outs[0])
        check_against_oracle(a[0], x, *w_a)
        check_against_oracle(b[0], a[0], *w_b)
        check_against_oracle(outs[0], b[0], *w_c)
        for layer in col_a + col_b + row_c:
            layer.region.check()
            assert int(layer.region.counters[0]) == 0 and int(layer.region.counters[2]) == 0   # done / staged are back at zero
            assert int(layer.region.counters[1]) == epoch


def test_forward_gathers_and_copies_out():
    world = 2
    ranks = LocalRanks(world)
    w = _layer(384, 512, 5)
    layers = [PeerColumnParallelQuantizedLinear(*shard_rows(*w, r, world), local=ranks, rank=r, name="w") for r in range(world)]
    for m in (1, 8, 2):
        x = torch.randn((m, 512), device="cuda").half()
        views = [layer.launch(x) for layer in layers]
        outs = [view.materialize() for view in views]
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1])
        check_against_oracle(outs[0], x, *w)
        full = capi_linear(x, *w)
        torch.testing.assert_close(outs[0], full, rtol=1e-2, atol=1e-2)


def test_a_sender_that_never_publishes_is_reported_not_waited_for_forever():
    """Rank 1 of 2 never launches: rank 0's readers give up after their poll limit and say who was missing."""
    world = 2
    ranks = LocalRanks(world)
    w = _layer(256, 512, 7)
    col = PeerColumnParallelQuantizedLinear(*shard_rows(*w, 0, world), local=ranks, rank=0, name="w", max_polls=1000)
    nxt = PeerColumnParallelQuantizedLinear(*shard_rows(*_layer(128, 256, 8), 0, world), local=ranks, rank=0, name="n",
                                            max_polls=1000)
    x = torch.randn((2, 512), device="cuda").half()
    # (a) the reader kernel
    col.launch(x).materialize()
    torch.cuda.synchronize()
    assert int(col.region.counters[3]) == 2          # sender 1, reported as index + 1
    with pytest.raises(RuntimeError, match="rank 1 never published"):
        col.region.check()
    # (b) the reader inside a consuming linear
    col.region.counters[3] = 0
    nxt.launch(col.launch(x))
    torch.cuda.synchronize()
    assert int(col.region.counters[3]) == 0 and int(nxt.region.counters[3]) == 2   # reported through the consumer's word
    # (c) the reader inside the partial-sum kernel
    row = PeerRowParallelQuantizedLinear(*shard_k(*w, 0, world, 128), local=ranks, rank=0, name="r", max_polls=1000)
    row.forward(x[:, :256].contiguous())
    torch.cuda.synchronize()
    assert int(row.region.counters[3]) == 2
    # the device is healthy: an ordinary launch still gives the right answer
    check_against_oracle(capi_linear(x, *w), x, *w)


def test_a_reader_that_never_releases_is_reported():
    """Nobody reads what rank 0 publishes: its third launch would overwrite the first result buffer, waits
    (bounded) for the readers' release and reports them."""
    world = 2
    ranks = LocalRanks(world)
    w = _layer(256, 512, 9)
    col = PeerColumnParallelQuantizedLinear(*shard_rows(*w, 0, world), local=ranks, rank=0, name="w", max_polls=1000)
    x = torch.randn((1, 512), device="cuda").half()
    col.launch(x)
    col.launch(x)
    torch.cuda.synchronize()
    assert int(col.region.counters[3]) == 0          # two result buffers: two publications need no release
    col.launch(x)
    torch.cuda.synchronize()
    assert int(col.region.counters[3]) == 32 + world  # the highest-numbered reader that never released, + 33 - 1
    with pytest.raises(RuntimeError, match="never released"):
        col.region.check()
    check_against_oracle(capi_linear(x, *w), x, *w)


def test_plain_sum_of_partials():
    import ctypes

    from nibble_b200 import _native

    parts = torch.randn((3, 1000), device="cuda")
    out = torch.empty((1000,), dtype=torch.float16, device="cuda")
    status = _native.core().w4a16_sum_partials_f16(parts.data_ptr(), out.data_ptr(), 1000, 3, None, 0,
                                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == 0
    expect = ((parts[0] + parts[1]) + parts[2]).half()
    assert torch.equal(out, expect)
