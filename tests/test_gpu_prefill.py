"""-m gpu: prefill-sized batches (M >= 65) take the tcgen05 GEMM with the dequantisation fused into its
producer warps.  Checked against the oracle on the same packed codes, against the mma.sync kernel,
and for a clean device status word (no barrier wait gave up)."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from capi_helpers import capi_linear, check_against_oracle, new_workspace
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


@pytest.mark.parametrize(("m", "k", "n"), [
    (17, 384, 128),       # three 128-wide stages: the last copy of codes of a tile is half used
    (40, 640, 256),       # five stages, two tiles
    (64, 1152, 384),      # nine stages
    (128, 896, 200),      # seven stages, 128-row batch tile (three operand stages, three working groups)
    (130, 640, 128),      # 64-wide stages (batch tile above 128 rows), ten of them: a half-used last copy
    (256, 384, 256),      # six 64-wide stages
    (200, 128, 128),      # two 64-wide stages: half a copy in all
])
def test_forced_gemm_on_odd_stage_counts(m, k, n):
    """Stage counts that do not fill the last copy of codes, for both stage widths, through the flag that
    sends any batch to the GEMM."""
    _device_status()
    x, packed, scales = _case(m, k, n, seed=m * 7 + k)
    y = capi_linear(x, packed, scales, flags=_native.FLAG_FORCE_TCGEN05)
    torch.cuda.synchronize()
    assert _device_status() == 0
    check_against_oracle(y, x, packed, scales, fp16_weights=True)
    again = capi_linear(x, packed, scales, flags=_native.FLAG_FORCE_TCGEN05)
    assert torch.equal(y, again)


@pytest.mark.parametrize("m", [16, 17, 33, 64])
def test_medium_batches_on_a_large_layer_take_the_gemm(m):
    """A layer of K = 8192, N = 4096 is cheaper on the GEMM than on the streaming kernel from 17 rows on: the default
    route then gives what the forced GEMM gives, bit for bit; up to 16 rows, what the streaming kernel gives.  The
    two agree within the tolerance."""
    k, n = 8192, 4096
    takes_gemm = m > 16        # the cost model's verdict for this layer; the bit comparison below pins it
    _device_status()
    x, packed, scales = _case(m, k, n, seed=m)
    ws = new_workspace(m, n, k)
    y = capi_linear(x, packed, scales, workspace=ws)
    forced = capi_linear(x, packed, scales, workspace=ws, flags=_native.FLAG_FORCE_TCGEN05)
    streaming = capi_linear(x, packed, scales, workspace=ws, flags=_native.FLAG_NO_TCGEN05)
    torch.cuda.synchronize()
    assert _device_status() == 0
    assert torch.equal(y, forced if takes_gemm else streaming)
    torch.testing.assert_close(forced, streaming, rtol=1e-2, atol=1e-2)
    rows = np.sort(np.random.default_rng(m).choice(n, size=32, replace=False))
    check_against_oracle(forced, x, packed, scales, rows=rows, fp16_weights=True)


def test_batch_too_large_for_the_streaming_kernel_without_scratch_takes_the_gemm():
    """32 rows of K = 28672 do not fit one CTA's shared memory unsplit; without a workspace the call used to fall
    to the generic kernel (milliseconds) and now runs the GEMM."""
    m, k, n = 32, 28672, 256
    _device_status()
    x, packed, scales = _case(m, k, n, seed=5)
    y = capi_linear(x, packed, scales, workspace=None)
    forced = capi_linear(x, packed, scales, flags=_native.FLAG_FORCE_TCGEN05)
    torch.cuda.synchronize()
    assert _device_status() == 0
    assert torch.equal(y, forced)
    check_against_oracle(y, x, packed, scales, fp16_weights=True)


@pytest.mark.parametrize(("m", "k", "n"), [
    (65, 4096, 256),       # 2 tiles: four K ranges of 1024 (ranges are not made shorter than that)
    (65, 4096, 250),       # the same with M x N not a multiple of four: the element-wise sum kernel
    (128, 4096, 1024),     # 8 tiles: four ranges
    (100, 4352, 640),      # 5 tiles, K = 17 x 256: three ranges of 1280 and one of 512
    (300, 8192, 512),      # two batch tiles (64-wide stages), 8 tiles in all: four ranges of 2048
    (32, 8192, 4096),      # a medium batch on the forced GEMM: 32 tiles, four ranges
])
def test_gemm_splits_k_when_the_layer_has_few_tiles(m, k, n):
    """With a workspace the GEMM shares the K of an output tile between CTAs (FP32 partial sums, added in order by a
    second kernel); without one it runs unsplit.  Both agree with the oracle, and the workspace's counter prefix,
    which the streaming kernel relies on, is left at zero."""
    lib = _native.core()
    flags = _native.FLAG_FORCE_TCGEN05
    need = lib.w4a16_linear_workspace_bytes_flags(m, n, k, flags)
    assert need > 256 * 1024, "this layer should want K split"
    _device_status()
    x, packed, scales = _case(m, k, n, seed=m + n)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    split = capi_linear(x, packed, scales, workspace=ws, flags=flags)
    again = capi_linear(x, packed, scales, workspace=ws, flags=flags)
    unsplit = capi_linear(x, packed, scales, flags=flags)
    torch.cuda.synchronize()
    assert _device_status() == 0
    assert torch.equal(split, again)
    torch.testing.assert_close(split, unsplit, rtol=2e-3, atol=2e-3)
    check_against_oracle(split, x, packed, scales, fp16_weights=True)
    assert int(ws[: 256 * 1024].sum()) == 0
    # a workspace that is too small is not an error: the GEMM runs unsplit
    small = torch.zeros(256 * 1024 + 64, dtype=torch.uint8, device="cuda")
    assert torch.equal(capi_linear(x, packed, scales, workspace=small, flags=flags), unsplit)


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
