"""-m gpu: the allocation-free entry point ``w4a16_linear_f16_static_scratch``.

It exists for callers that are not allowed to allocate device memory (a serving loop that forbids
cudaMalloc after start-up, a plugin that receives buffers but no workspace, code inside a stream
capture) and therefore cannot give ``w4a16_linear_f16`` the split-K workspace it wants.  The test
calls it through the C ABI on shapes that do split K, twice in a row on the same stream -- the
second call finds the scratch as the first one left it -- and compares with the ordinary entry
point given a caller-owned workspace.  This file sorts last so that a run stopping at the first
failure has already run everything else; it also passes on its own in a fresh process (the first
call does the one-time address lookup).
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from capi_helpers import capi_linear, check_against_oracle, new_workspace
from nibble_b200 import _native, quantize_and_pack_weights

pytestmark = pytest.mark.gpu


def _static_scratch_linear(x, packed, scales, expect=0):
    m, k = x.shape
    n = packed.shape[0]
    y = torch.full((m, n), float("nan"), dtype=torch.float16, device=x.device)
    status = _native.core().w4a16_linear_f16_static_scratch(
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(scales.data_ptr()),
        ctypes.c_void_p(y.data_ptr()), m, n, k, 128, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert status == expect, f"status {status}: {_native.status_string(status)}"
    return y


@pytest.mark.parametrize(("m", "n", "k"), [(1, 1024, 8192), (4, 1000, 8192), (1, 8192, 28672), (8, 256, 2048)])
def test_matches_the_workspace_entry_point_twice_in_a_row(m, n, k):
    lib = _native.core()
    assert lib.w4a16_linear_workspace_bytes(m, n, k) > 0 or (n, k) == (256, 2048), "shape should split K"
    g = torch.Generator().manual_seed(n + k + m)
    if n * k <= 16 * 2**20:
        w = torch.randn((n, k), generator=g) * 0.02
        packed, scales = quantize_and_pack_weights(w, 128)
        packed, scales = packed.cuda(), scales.cuda()
    else:   # large: random codes straight on the device
        torch.manual_seed(n + k)
        packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        scales = (torch.rand((n, k // 128), device="cuda") * 0.01 + 1e-3).half()
    x = torch.randn((m, k), generator=g).half().cuda()

    expected = capi_linear(x, packed, scales, workspace=new_workspace(m, n, k))
    first = _static_scratch_linear(x, packed, scales)
    second = _static_scratch_linear(x, packed, scales)
    torch.cuda.synchronize()
    for got in (first, second):
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got, expected, rtol=1e-2, atol=1e-2)
    assert torch.equal(first, second), "same inputs, same scratch, same order of summation"
    rows = None if n * k <= 16 * 2**20 else list(range(0, n, 97))
    check_against_oracle(second, x, packed, scales, rows=rows)


@pytest.mark.parametrize(("m", "n", "k"), [(128, 5632, 2048), (512, 8192, 8192), (65, 300, 1024)])
def test_batches_that_need_no_scratch_are_forwarded(m, n, k):
    """From 65 rows on the ordinary entry point runs the tcgen05 GEMM, which has no split-K scratch, so the
    allocation-free entry point must run such batches too, whatever their size, and give the same bits."""
    lib = _native.core()
    # (no scratch at all, or -- a layer of few tiles, whose K the GEMM would share between CTAs -- more than the
    # built-in array holds, in which case the GEMM runs unsplit)
    need = lib.w4a16_linear_workspace_bytes_flags(m, n, k, 0)
    assert need == 0 or need > lib.w4a16_static_scratch_bytes()
    torch.manual_seed(m + n)
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
    scales = (torch.rand((n, k // 128), device="cuda") * 0.01 + 1e-3).half()
    x = torch.randn((m, k), device="cuda").half()
    expected = capi_linear(x, packed, scales)
    first = _static_scratch_linear(x, packed, scales)
    second = _static_scratch_linear(x, packed, scales)
    torch.cuda.synchronize()
    assert torch.equal(first, expected) and torch.equal(second, expected)
    rows = list(range(0, n, max(1, n // 64)))
    check_against_oracle(second[:32].contiguous(), x[:32].contiguous(), packed, scales, rows=rows, fp16_weights=True)
    value = ctypes.c_uint32(7)
    assert lib.w4a16_device_status(ctypes.byref(value)) == 0 and value.value == 0


def test_scratch_size_is_reported_and_oversized_problems_are_refused():
    lib = _native.core()
    capacity = lib.w4a16_static_scratch_bytes()
    assert capacity == 4 * 2**20
    # A problem that wants split-K scratch beyond the built-in array is refused, nothing launched.
    m, n, k = 16, 32768, 8192      # sixteen rows of this layer stay on the streaming kernel, K split four ways
    assert lib.w4a16_linear_workspace_bytes(m, n, k) > capacity
    before = lib.w4a16_launch_count()
    x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    packed = torch.zeros((n, k // 2), dtype=torch.uint8, device="cuda")
    scales = torch.ones((n, k // 128), dtype=torch.float16, device="cuda")
    _static_scratch_linear(x, packed, scales, expect=-8)
    assert lib.w4a16_launch_count() == before
    assert "exceeds" in _native.status_string(-8)
