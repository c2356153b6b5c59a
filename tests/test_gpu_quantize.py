"""-m gpu: the device quantise+pack kernel produces the reference quantiser's bits."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from nibble_b200 import _native, quantize_and_pack_cuda, quantize_and_pack_weights
from nibble_b200.quantization import pack_int4, quantize_groupwise
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu


def _host(weights: torch.Tensor, group: int):
    codes, scales = quantize_groupwise(weights.cpu(), group)
    return pack_int4(codes), scales


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize(("n", "k", "group"), [(8, 128, 128), (33, 1024, 128), (250, 2048, 128), (7, 96, 32),
                                               (5, 24, 4), (3, 12, 6), (4, 8, 2), (2048, 5632, 128)])
def test_device_quantiser_matches_host_and_oracle(dtype, n, k, group):
    g = torch.Generator().manual_seed(n * k + group)
    w = (torch.randn((n, k), generator=g) * 0.02).to(dtype)
    packed, scales = quantize_and_pack_cuda(w.cuda(), group)
    want_packed, want_scales = _host(w, group)
    assert packed.dtype == torch.uint8 and scales.dtype == torch.float16
    assert torch.equal(packed.cpu(), want_packed)
    assert torch.equal(scales.cpu(), want_scales)
    o_packed, o_scales = oracle.quantize_and_pack_weights(w.numpy(), group)
    assert np.array_equal(packed.cpu().numpy(), o_packed) and np.array_equal(scales.cpu().numpy(), o_scales)
    # the public host entry point takes the same route for CUDA tensors
    again_packed, again_scales = quantize_and_pack_weights(w.cuda(), group)
    assert torch.equal(again_packed, packed) and torch.equal(again_scales, scales)


def test_zero_groups_ties_and_clamp():
    w = torch.zeros((3, 256), dtype=torch.float32)
    # row 1, group 0: step 1 (amax 7); halves round to even; row 1, group 1 stays all zero -> scale 1
    w[1, :16] = torch.tensor([7, -7, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5, 6.5, -6.5, 4.4999, 4.5, 5.5, -5.5])
    # row 2: a large outlier makes every other weight quantise to 0 or +-1
    w[2, 128:] = 0.01
    w[2, 200] = -3.0
    packed, scales = quantize_and_pack_cuda(w.cuda(), 128)
    want_packed, want_scales = _host(w, 128)
    assert torch.equal(packed.cpu(), want_packed) and torch.equal(scales.cpu(), want_scales)
    assert scales[0, 0].item() == 1.0 and scales[1, 1].item() == 1.0
    codes = oracle.unpack_int4(packed.cpu().numpy())
    assert codes[1, :16].tolist() == [7, -7, 0, 2, 2, 0, -2, -2, 4, -4, 6, -6, 4, 4, 6, -6]
    assert codes.min() >= -7 and codes.max() <= 7


def test_quantise_then_fused_linear_round_trip():
    from capi_helpers import capi_linear, check_against_oracle

    w = (torch.randn((512, 1024), generator=torch.Generator().manual_seed(9)) * 0.02).half().cuda()
    packed, scales = quantize_and_pack_cuda(w, 128)
    x = torch.randn((4, 1024), generator=torch.Generator().manual_seed(10)).half().cuda()
    check_against_oracle(capi_linear(x, packed, scales), x, packed, scales)


def test_c_abi_validation():
    lib = _native.core()
    w = torch.zeros((4, 128), dtype=torch.float16, device="cuda")
    p = torch.empty((4, 64), dtype=torch.uint8, device="cuda")
    s = torch.empty((4, 1), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.w4a16_quantize_pack_f16(w.data_ptr(), p.data_ptr(), s.data_ptr(), 4, 128, 128, stream) == 0
    assert lib.w4a16_quantize_pack_f16(w.data_ptr(), p.data_ptr(), s.data_ptr(), 4, 128, 3, stream) == -3
    assert lib.w4a16_quantize_pack_f16(w.data_ptr(), p.data_ptr(), s.data_ptr(), 4, 128, 48, stream) == -2
    assert lib.w4a16_quantize_pack_f16(None, p.data_ptr(), s.data_ptr(), 4, 128, 128, stream) == -1
    assert lib.w4a16_quantize_pack_f32(w.data_ptr(), p.data_ptr(), s.data_ptr(), 0, 128, 128, stream) == 0
    torch.cuda.synchronize()


def test_near_tie_quotients_match_the_host_division():
    # weights placed within a few ulp of every rounding tie k + 0.5 of w / step, for awkward steps
    g = torch.Generator().manual_seed(21)
    rows = []
    for _ in range(64):
        amax = float(torch.rand((), generator=g) * 3 + 0.01)
        step = torch.tensor(amax, dtype=torch.float32) / 7.0
        ties = (torch.arange(-7, 7, dtype=torch.float32) + 0.5) * step
        near = torch.cat([ties, torch.nextafter(ties, torch.tensor(10.0)), torch.nextafter(ties, torch.tensor(-10.0)),
                          ties * (1 + 3e-7), ties * (1 - 3e-7)])
        row = torch.zeros(128)
        row[: near.numel()] = near
        row[-1] = amax
        rows.append(row)
    w = torch.stack(rows)
    packed, scales = quantize_and_pack_cuda(w.cuda(), 128)
    want_packed, want_scales = _host(w, 128)
    assert torch.equal(packed.cpu(), want_packed) and torch.equal(scales.cpu(), want_scales)
