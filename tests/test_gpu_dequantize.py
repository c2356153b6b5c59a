"""-m gpu: the dequantise kernel through the C ABI and the torch op, bit-exact against the oracle
(cases of the reference's tests/test_cuda.py:482-531)."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from capi_helpers import capi_dequantize
from conftest import TINYLLAMA_LAYERS, seeded_weights
from nibble_b200 import dequantize_cuda, quantize_and_pack_weights
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu


def _expect(packed, scales, gs):
    return oracle.dequantize_weights(packed.cpu().numpy(), scales.cpu().numpy(), gs).astype(np.float16)


def _same_bits(t: torch.Tensor, ref: np.ndarray) -> bool:
    return np.array_equal(t.cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("group_size", [32, 64, 128])
@pytest.mark.parametrize(("k", "n"), [(256, 8), (2048, 2048), (2048, 5632), (5632, 2048), (384, 13)])
def test_bit_identical_to_oracle(k, n, group_size):
    if k % group_size:
        pytest.skip("K not divisible")
    torch.manual_seed(0)
    w = torch.randn((n, k), dtype=torch.float16)
    packed, scales = quantize_and_pack_weights(w, group_size)
    out = capi_dequantize(packed.cuda(), scales.cuda(), group_size)
    assert _same_bits(out, _expect(packed, scales, group_size))
    out_op = dequantize_cuda(packed.cuda(), scales.cuda(), group_size)
    assert out_op.dtype == torch.float16 and out_op.shape == (n, k)
    assert torch.equal(out_op, out)


def test_all_nibble_values(golden):
    data = golden("all_nibbles.npz")
    packed = torch.from_numpy(data["packed"]).cuda()
    scales = torch.from_numpy(data["scales"]).cuda()
    out = capi_dequantize(packed, scales, 128)
    assert _same_bits(out, data["dequant"].astype(np.float16))


def test_subnormal_and_large_scales_round_like_the_oracle():
    g = torch.Generator().manual_seed(5)
    packed = torch.randint(0, 256, (32, 256), dtype=torch.uint8, generator=g)
    tiny = torch.tensor([6e-8, 1.2e-7, 3e-6, 6.1e-5, 6.2e-5, 1e-4, 8000.0, 65504.0 / 8]).half()
    scales = tiny[torch.randint(0, 8, (32, 4), generator=g)]
    out = capi_dequantize(packed.cuda(), scales.cuda(), 128)
    assert _same_bits(out, _expect(packed, scales, 128))


@pytest.mark.parametrize(("name", "k", "n"), TINYLLAMA_LAYERS)
def test_full_size_layers_match_reference_digest(golden, name, k, n):
    """Digest of the reference's own dequantised FP16 matrix for the seeded layer."""
    data = golden("tinyllama_m1.npz")
    index = [layer[0] for layer in TINYLLAMA_LAYERS].index(name)
    packed, scales = quantize_and_pack_weights(seeded_weights(n, k, seed=index), 128)
    assert hashlib.sha256(packed.numpy().tobytes()).hexdigest() == str(data[f"{name}/packed_sha256"])
    out = capi_dequantize(packed.cuda(), scales.cuda(), 128)
    assert hashlib.sha256(out.cpu().numpy().tobytes()).hexdigest() == str(data[f"{name}/dequant_fp16_sha256"])


def test_largest_layer_shape_by_row_sampling():
    """70B down_proj shape (K=28672, N=8192): random bytes on the device, oracle on sampled rows."""
    n, k = 8192, 28672
    torch.manual_seed(1)
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
    scales = (torch.rand((n, k // 128), device="cuda") * 0.05 + 1e-3).half()
    out = capi_dequantize(packed, scales, 128)
    rows = torch.cat([torch.arange(0, 8), torch.randint(0, n, (48,)), torch.arange(n - 8, n)])
    ref = _expect(packed[rows.cuda()], scales[rows.cuda()], 128)
    assert _same_bits(out[rows.cuda()], ref)


def test_op_rejects_bad_arguments():
    packed = torch.zeros((8, 48), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        dequantize_cuda(packed, torch.ones((8, 2), dtype=torch.float16, device="cuda"), 48)
    with pytest.raises(RuntimeError):
        dequantize_cuda(packed.cpu(), torch.ones((8, 3), dtype=torch.float16), 32)
    with pytest.raises(RuntimeError):
        dequantize_cuda(packed, torch.ones((8, 2), dtype=torch.float16, device="cuda"), 32)  # scale shape
    assert dequantize_cuda(packed[:0], torch.ones((0, 3), dtype=torch.float16, device="cuda"), 32).shape == (0, 96)
