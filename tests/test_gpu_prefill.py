"""-m gpu: prefill-sized batches (M >= 65) take the tcgen05 GEMM with the dequantisation fused into its
producer warps.  Checked against the oracle on the same packed codes, against the mma.sync kernel,
and for a clean device status word (no barrier wait gave up)."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from capi_helpers import capi_linear, check_against_oracle
from nibble_b200 import _native, quantize_and_pack_weights
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu


def _device_status() -> int:
    value = ctypes.c_uint32(123)
    assert _native.core().w4a16_device_status(ctypes.byref(value)) == 0
    return value.value


def _case(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((n, k), generator=g) * 0.02
    x = torch.randn((m, k), generator=g).half()
    packed, scales = quantize_and_pack_weights(w, 128)
    return x.cuda(), packed.cuda(), scales.cuda()


@pytest.mark.parametrize("m", [65, 128, 129, 300])
@pytest.mark.parametrize(("k", "n"), [(128, 128), (512, 256), (1024, 250), (2048, 2048), (5632, 384)])
def test_tcgen05_path_matches_oracle(m, k, n):
    _device_status()   # clear
    x, packed, scales = _case(m, k, n, seed=m + k + n)
    before = _native.core().w4a16_launch_count()
    y = capi_linear(x, packed, scales)
    torch.cuda.synchronize()
    assert _device_status() == 0, "a barrier wait inside the tcgen05 kernel gave up"
    assert _native.core().w4a16_launch_count() == before + 1
    check_against_oracle(y, x, packed, scales)
    # the product of FP16-rounded weights, FP32 accumulate: what dequantise-then-matmul computes
    w16 = oracle.dequantize_weights(packed.cpu().numpy(), scales.cpu().numpy(), 128).astype(np.float16)
    ref = torch.from_numpy(x.cpu().numpy().astype(np.float32) @ w16.astype(np.float32).T)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=2e-3, atol=2e-3)
    # and the streaming mma.sync kernel on the same inputs
    other = capi_linear(x, packed, scales, flags=_native.FLAG_NO_TCGEN05)
    torch.testing.assert_close(y, other, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize(("m", "k", "n"), [
    (600, 512, 8192),      # 3 x 64 tiles: more tiles than SMs, every CTA reuses an accumulator buffer
    (1024, 256, 16384),    # 512 tiles: at least three per CTA, both accumulator buffers recycled
    (257, 1024, 1000),     # two ragged batch tiles, ragged last weight slab
    (2048, 2048, 640),     # 8 batch tiles walked in groups
])
def test_tcgen05_many_tiles(m, k, n):
    _device_status()
    x, packed, scales = _case(m, k, n, seed=m ^ n)
    y = capi_linear(x, packed, scales)
    torch.cuda.synchronize()
    assert _device_status() == 0
    w16 = torch.from_numpy(oracle.dequantize_weights(packed.cpu().numpy(), scales.cpu().numpy(), 128).astype(np.float16))
    ref = (x.float() @ w16.cuda().float().t())
    torch.testing.assert_close(y.float(), ref, rtol=2e-3, atol=2e-3)
    rows = np.random.default_rng(m).choice(n, size=64, replace=False)
    check_against_oracle(y, x, packed, scales, rows=np.sort(rows), fp16_weights=True)


def test_all_nibble_values_and_repeatability(golden):
    data = golden("all_nibbles.npz")
    packed = torch.from_numpy(data["packed"]).cuda()
    scales = torch.from_numpy(data["scales"]).cuda()
    x = torch.randn((96, 1024), generator=torch.Generator().manual_seed(5)).half().cuda()
    first = capi_linear(x, packed, scales)
    second = capi_linear(x, packed, scales)
    assert torch.equal(first, second)
    assert _device_status() == 0
    check_against_oracle(first, x, packed, scales, fp16_weights=True)
